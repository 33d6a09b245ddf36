"""Release gate on a real GPU: exit code != 0 if correctness or speed regresses.

Same checks, arguments and thresholds as the reference's ``tools/gpu_gate.py``: (1) the sparse gate/up GEMM
at 512 tokens against the dense GEMM on the same pruned weight, max abs error <= 0.30 with N(0,1) fp16
operands (:60-68); (2) speed-up over pruned-dense for gate/up at M >= 256 and for down at M >= 512, each
>= 1.10 by default (:71-96).  The sparse side is this library (prune+compress kernel, tcgen05 GEMMs)
instead of ``torch.sparse.to_sparse_semi_structured``; timing uses CUDA events over a CUDA graph of 20
launches (device time) instead of the reference's wall clock around 400 eager launches, because at these
sizes (15-60 us) an eager loop measures host enqueue cost.

    python -m sparseflow_b200.gpu_gate [--hidden 4096 --inter 14336 --Ms 256,512,1024]
"""
from __future__ import annotations

import argparse

import torch

from . import ops
from .gate_sweep import _time_graph

torch.backends.cuda.matmul.allow_tf32 = False


def run(hidden=4096, inter=14336, Ms=(256, 512, 1024), min_speedup_gateup=1.10, min_speedup_down=1.10,
        dtype=torch.float16, verbose=True) -> dict:
    assert torch.cuda.is_available(), "CUDA not available"
    cc = torch.cuda.get_device_capability(0)
    assert cc[0] == 10, "sm_100 required for the tcgen05 2:4 kernels"
    say = print if verbose else (lambda *a, **k: None)
    say(f"GPU: {torch.cuda.get_device_name(0)}  CC: {cc}")
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(dtype)
    out = {"failures": 0, "rows": []}

    def weight(o, i):
        w = rnd(o, i)
        o_ = ops.prune_compress_24(w, want_pruned=True)
        return o_["pruned"], ops.Compressed24(o_["values"], o_["meta"], o, i)

    Wg_p, Wg_s = weight(inter, hidden)
    Wd_p, Wd_s = weight(hidden, inter)

    Xc = rnd(512, hidden)
    err = (torch.nn.functional.linear(Xc, Wg_p).float() - ops.sparse_gemm(Xc, Wg_s).float()).abs().max().item()
    out["gate_up_max_abs_err"] = err
    say(f"[correctness] gate/up max abs err vs pruned-dense: {err:.6f}")
    if err > 0.30:
        out["failures"] += 1
        out["correctness_failed"] = True
        return out

    say("\n=== Microbench (speedup vs pruned-dense) ===")
    for M in Ms:
        say(f"\nM={M}")
        for name, Wp, Ws, kin, m_min, thr in (("gate/up", Wg_p, Wg_s, hidden, 256, min_speedup_gateup),
                                              ("down", Wd_p, Wd_s, inter, 512, min_speedup_down)):
            X = rnd(M, kin)
            y = torch.empty(M, Ws.rows, device=dev, dtype=dtype)
            t_pd = _time_graph(lambda: torch.matmul(X, Wp.t(), out=y)) * 1e3
            t_sp = _time_graph(lambda: ops.sparse_gemm(X, Ws, out=y)) * 1e3
            sp = t_pd / t_sp
            bad = M >= m_min and sp < thr
            out["rows"].append(dict(op=name, M=M, dense_us=t_pd, sparse_us=t_sp, speedup=sp, gated=M >= m_min, failed=bad))
            say(f" {name + ':':9s}{t_pd:8.2f}us -> {t_sp:8.2f}us  ({sp:.2f}x)" + (f"   below threshold {thr}x" if bad else ""))
            out["failures"] += int(bad)
    ops.device_status()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--Ms", type=str, default="256,512,1024")
    ap.add_argument("--min-speedup-gateup", type=float, default=1.10)
    ap.add_argument("--min-speedup-down", type=float, default=1.10)
    a = ap.parse_args()
    r = run(a.hidden, a.inter, [int(x) for x in a.Ms.split(",")], a.min_speedup_gateup, a.min_speedup_down)
    if r.get("correctness_failed"):
        raise SystemExit(f"FAIL: correctness error too high: {r['gate_up_max_abs_err']}")
    if r["failures"]:
        raise SystemExit(f"\nGPU GATE FAILED: {r['failures']} regressions detected.")
    print("\nGPU GATE PASSED")


if __name__ == "__main__":
    main()
