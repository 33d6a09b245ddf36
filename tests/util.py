"""Helpers shared by the tests: 16-bit pattern <-> torch tensors, seeded inputs."""
import numpy as np
import torch


def to_dev(bits: np.ndarray, dtype: str, device="cuda:0") -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device)
    return t.view(torch.float16 if dtype == "f16" else torch.bfloat16)


def bits_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def seeded_weight(rows, K, dtype, seed, sigma=0.02):
    """W ~ N(0, sigma) generated on the CPU in fp32 then narrowed: identical bits for oracle and GPU."""
    import oracle as o
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.randn(rows, K, generator=g, dtype=torch.float32) * sigma
    return o.from_f32(w.numpy(), dtype)


def seeded_act(M, K, dtype, seed):
    import oracle as o
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    return o.from_f32(x.numpy(), dtype)


def big_gemm_ref(x_bits: np.ndarray, w_pruned_bits: np.ndarray, dtype: str) -> np.ndarray:
    """``oracle.gemm_ref`` (fp32 matmul on the pruned weights, experiments/gen_pruned_ref.py:5-8) with the
    product itself done by torch's multi-threaded CPU sgemm, for the full-size configurations."""
    import oracle as o
    x = torch.from_numpy(o.to_f32(x_bits, dtype))
    w = torch.from_numpy(o.to_f32(w_pruned_bits, dtype))
    return (x @ w.t()).numpy()


def big_ffn_ref(x_bits, wg_pruned, wu_pruned, wd_pruned, dtype: str, round_gate_up: bool = False) -> dict:
    """``oracle.ffn_ref`` with the same rounding points, matmuls through ``big_gemm_ref``."""
    import oracle as o
    g = big_gemm_ref(x_bits, wg_pruned, dtype)
    u = big_gemm_ref(x_bits, wu_pruned, dtype)
    if round_gate_up:
        g = o.to_f32(o.from_f32(g, dtype), dtype)
        u = o.to_f32(o.from_f32(u, dtype), dtype)
    h = o.from_f32(o.silu_mul_ref(g, u), dtype)
    out = big_gemm_ref(h, wd_pruned, dtype)
    return dict(hidden=h, out=o.from_f32(out, dtype), out_f32=out)
