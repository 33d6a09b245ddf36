"""Run one kernel of the hot path a few times on a small case, for `ncu` captures.

    python -m sparseflow_b200.profile_case --case gate_up --tokens 2048 --iters 2

Cases (Llama-7B shapes, bf16): gate_up (fused gate|up GEMM with SiLU.mul epilogue, 22016 x 4096
weight), down (4096 x 11008 weight), prune (prune+compress of the 11008 x 4096 gate weight),
decode (small-M GEMM, tokens <= 16).  Working sets stay between the 126 MB L2 and a few hundred MB.
"""
from __future__ import annotations

import argparse

import torch

from . import ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="gate_up", choices=["gate_up", "down", "prune", "decode"])
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--tile", type=int, default=0, help="token-tile override (see sfb200_debug_force_token_tile)")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=11008)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    H, I, M = a.hidden, a.inter, a.tokens
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, sigma=1.0: (torch.randn(*s, generator=g, device=dev, dtype=torch.float32) * sigma).to(torch.bfloat16)
    ops.force_token_tile(a.tile)
    if a.case == "prune":
        w = rnd(I, H, sigma=0.02)
        fn = lambda: ops.prune_compress_24(w)
    elif a.case == "gate_up":
        cw = ops.compress_gate_up(rnd(I, H, sigma=0.02), rnd(I, H, sigma=0.02))
        x = rnd(M, H)
        out = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.sparse_gemm_swiglu(x, cw, out=out)
    else:
        cw = ops.compress_weight(rnd(H, I, sigma=0.02))
        x = rnd(M, I)
        out = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.sparse_gemm(x, cw, out=out)
    fn()                                    # warm-up launch
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(f"{a.case} tokens={M} tile={a.tile}: {e0.elapsed_time(e1) / a.iters * 1e3:.1f} us per launch; "
          f"device status {ops.device_status()}")


if __name__ == "__main__":
    main()
