"""Shape sweeps of the sparse path against cuBLAS dense on the same 2:4-pruned weights.

    python -m sparseflow_b200.shape_sweep gemm [--json out.json]
        standalone GEMM, fp16 and bf16, M in {16,128,1024,4096,16384} x (K,N) in
        {(4096,4096),(4096,11008),(11008,4096),(8192,8192)}: dense-equivalent TFLOP/s, algorithmic GB/s,
        speed-up, and whether the shape gate would pick sparse.
    python -m sparseflow_b200.shape_sweep ffn [--hidden 4096 --inter 14336] [--json out.json]
        gated FFN token sweep M in {1,8,32,128,512,2048,8192}: pruned-dense (three library GEMMs + SiLU.mul),
        always-sparse (the fused two-kernel chain) and gated ("auto": the shape gate decides per GEMM).

Same role as the reference's tools/bench_semistructured_gemm.py, tools/sweep_shapes.py and
tools/bench_mlp_mistral.py (dense vs pruned-dense vs sparse over shapes).  Weights N(0, 0.02),
activations N(0, 1), fixed seeds; weights rotate over several copies (> L2 in total); token counts up to
512 are timed as CUDA graphs of 20 launches (device time), larger ones eagerly with CUDA events.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import dispatch, ops
from .fused_mlp import SparseFlowFusedMLP
from .gate_sweep import _time, _time_graph

GEMM_SHAPES = [(4096, 4096), (4096, 11008), (11008, 4096), (8192, 8192)]     # (K, N)
GEMM_TOKENS = [16, 128, 1024, 4096, 16384]
FFN_TOKENS = [1, 8, 32, 128, 512, 2048, 8192]


def _timeit(fn, M):
    return _time_graph(fn) if M <= 512 else _time(fn, 12)


def sweep_gemm() -> list:
    dev = torch.device("cuda:0")
    rows = []
    for dt, name in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        for K, N in GEMM_SHAPES:
            copies = max(2, min(6, int(400e6 // (N * K * 2)) + 1))
            g = torch.Generator(device=dev).manual_seed(1)
            ws = [ops.compress_weight((torch.randn(N, K, device=dev, generator=g) * 0.02).to(dt)) for _ in range(copies)]
            wd = [ops.decompress_24(c) for c in ws]
            for M in GEMM_TOKENS:
                gx = torch.Generator(device=dev).manual_seed(1234)
                x = torch.randn(M, K, device=dev, generator=gx).to(dt)
                y = torch.empty(M, N, device=dev, dtype=dt)
                yd = torch.empty(M, N, device=dev, dtype=dt)
                i = [0]

                def fs():
                    ops.sparse_gemm(x, ws[i[0] % copies], out=y)
                    i[0] += 1

                def fd():
                    torch.matmul(x, wd[i[0] % copies].t(), out=yd)
                    i[0] += 1
                ts, td = _timeit(fs, M), _timeit(fd, M)
                i[0] = 0
                fs()
                i[0] = 0
                fd()
                ref = x.float() @ wd[0].float().t()
                err = ((y.float() - ref).abs().max() / ref.abs().max()).item()
                byts = N * K * 1.125 + M * K * 2 + M * N * 2
                rows.append(dict(dtype=name, K=K, N=N, M=M, sparse_us=ts * 1e3, dense_us=td * 1e3, speedup=td / ts,
                                 sparse_tflops=2.0 * M * N * K / ts / 1e9, dense_tflops=2.0 * M * N * K / td / 1e9,
                                 sparse_gbs=byts / ts / 1e6, max_err_over_max=err,
                                 gate_picks_sparse=dispatch.should_use_sparse(M, K, N)))
                r = rows[-1]
                print(f"{name} K={K:5d} N={N:5d} M={M:5d}: sparse {r['sparse_us']:8.1f} us {r['sparse_tflops']:7.1f} TF "
                      f"{r['sparse_gbs']:6.0f} GB/s | dense {r['dense_us']:8.1f} us | x{r['speedup']:.2f} "
                      f"gate={'sparse' if r['gate_picks_sparse'] else 'dense'} err {err:.1e}", flush=True)
            del ws, wd
    ops.device_status()
    return rows


def sweep_ffn(H: int, I: int) -> list:
    dev = torch.device("cuda:0")
    dt = torch.bfloat16
    mods = []
    for c in range(2):           # two weight sets (2 x 352 MB dense at Mistral size) rotate through L2
        lin = []
        for seed, (o, i) in zip((1, 2, 3), ((I, H), (I, H), (H, I))):
            g = torch.Generator(device=dev).manual_seed(seed + 10 * c)
            w = (torch.randn(o, i, device=dev, generator=g) * 0.02).to(dt)
            l = nn.Linear(i, o, bias=False, device=dev, dtype=dt)
            l.weight.data = ops.prune_compress_24(w, want_values=False, want_meta=False, want_pruned=True)["pruned"]
            lin.append(l)
        mods.append(dict(lin=lin, sparse=SparseFlowFusedMLP(*lin, force_mode="sparse"),
                         auto=SparseFlowFusedMLP(*lin, force_mode="auto")))
    rows = []
    for M in FFN_TOKENS:
        gx = torch.Generator(device=dev).manual_seed(1234)
        x = torch.randn(M, H, device=dev, generator=gx).to(dt)
        i = [0]

        def dense():
            g, u, d = mods[i[0] % 2]["lin"]
            i[0] += 1
            return d(F.silu(g(x)) * u(x))

        def arm(name):
            def f():
                m = mods[i[0] % 2][name]
                i[0] += 1
                return m(x)
            return f
        with torch.no_grad():
            td, ts, ta = _timeit(dense, M), _timeit(arm("sparse"), M), _timeit(arm("auto"), M)
            ref = dense().float()
            i[0] -= 1
            got = arm("auto")().float()
        err = ((got - ref).abs().max() / ref.abs().max()).item()
        flops = 6.0 * M * H * I
        wbytes = 3 * H * I * 1.125
        rows.append(dict(M=M, dense_us=td * 1e3, sparse_us=ts * 1e3, auto_us=ta * 1e3,
                         auto_tflops=flops / ta / 1e9, sparse_tflops=flops / ts / 1e9,
                         sparse_weight_gbs=wbytes / ts / 1e6, speedup_sparse=td / ts, speedup_auto=td / ta,
                         gate_gate_up="sparse" if dispatch.should_use_sparse(M, H, 2 * I) else "dense",
                         gate_down="sparse" if dispatch.should_use_sparse(M, I, H) else "dense",
                         auto_vs_dense_max_err_over_max=err))
        r = rows[-1]
        print(f"M={M:5d}: dense {r['dense_us']:8.1f} us | sparse {r['sparse_us']:8.1f} us x{r['speedup_sparse']:.2f} "
              f"({r['sparse_tflops']:.0f} TF, weights {r['sparse_weight_gbs']:.0f} GB/s) | gated {r['auto_us']:8.1f} us "
              f"x{r['speedup_auto']:.2f} (gate|up {r['gate_gate_up']}, down {r['gate_down']}) err {err:.1e}", flush=True)
    ops.device_status()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "ffn"])
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    ops.force_token_tile(0)
    rows = sweep_gemm() if a.what == "gemm" else sweep_ffn(a.hidden, a.inter)
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"gpu": torch.cuda.get_device_name(0), "sweep": a.what, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
