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
