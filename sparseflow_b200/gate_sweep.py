"""Measure sparse vs dense on this GPU and write the shape-gate table.

    python -m sparseflow_b200.gate_sweep [--out gate_sm100.json] [--min-speedup 1.05]

Per projection class (the classes of ``dispatch.classify_projection``) and token count M, time the
sparse path of this library against the dense library GEMM on the same 2:4-pruned weight stored
dense (the reference's "pruned-dense" baseline, tools/bench_mlp_mistral.py:50-53), CUDA events,
rotating over several weight copies so small-M timings stream weights from HBM rather than L2.
Token counts up to 512 are timed as a CUDA graph of 20 launches (device time; the eager figures, which
include host enqueue cost, are recorded beside them).
Decision rule as in the reference's override generator
(tools/make_shape_overrides_sm89_from_results.py:18-22,99-127): sparse iff speed-up >= min_speedup.
``min_m`` = smallest measured M from which every larger M is a sparse win; ``decode_max_m`` = largest
measured M up to which every smaller M is a sparse win (0 if M = 1 is not).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import ops

SHAPES = {   # class -> list of (in_features K, out_features N)
    "attn_proj": [(4096, 4096), (8192, 8192)],
    "ffn_gate_up": [(4096, 22016), (4096, 28672)],
    "ffn_down": [(11008, 4096), (14336, 4096)],
}
TOKENS = [1, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192]


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _time_graph(fn, launches=20, replays=5):
    """Device time per launch: `launches` calls captured in one CUDA graph (each call rotates to the
    next weight copy), replayed `replays` times.  Host enqueue cost, which dominates eager timings of
    kernels shorter than ~15 us, is excluded."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(launches):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (launches * replays)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "gate_sm100.json"))
    ap.add_argument("--min-speedup", type=float, default=1.05)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    ops.force_token_tile(0)
    rows = []
    for cls, shapes in SHAPES.items():
        for K, N in shapes:
            copies = max(2, min(6, int(400e6 // (N * K * 2)) + 1))    # > L2 in total
            ws = [ops.compress_weight((torch.randn(N, K, device=dev, dtype=torch.float32) * 0.02).to(dt))
                  for _ in range(copies)]
            wd = [ops.decompress_24(c) for c in ws]
            for M in TOKENS:
                x = torch.randn(M, K, device=dev, dtype=dt)
                y = torch.empty(M, N, device=dev, dtype=dt)
                iters = 40 if M <= 512 else 12
                i = [0]

                def fs():
                    ops.sparse_gemm(x, ws[i[0] % copies], out=y)
                    i[0] += 1

                def fd():
                    torch.matmul(x, wd[i[0] % copies].t(), out=y)
                    i[0] += 1
                ts, td = _time(fs, iters), _time(fd, iters)
                row = {"class": cls, "K": K, "N": N, "M": M, "eager_sparse_us": ts * 1e3, "eager_dense_us": td * 1e3}
                if M <= 512:      # short kernels: decide on device time, not on host enqueue time
                    ts, td = _time_graph(fs), _time_graph(fd)
                    row["timing"] = "cuda graph of 20 launches"
                else:
                    row["timing"] = "eager, CUDA events"
                row.update({"sparse_us": ts * 1e3, "dense_us": td * 1e3, "speedup": td / ts,
                            "sparse_tflops": 2.0 * M * N * K / ts / 1e9,
                            "sparse_gbs": (N * K * 1.125 + M * K * 2 + M * N * 2) / ts / 1e6})
                rows.append(row)
                print(f"{cls:12s} K={K:6d} N={N:6d} M={M:5d} sparse {ts*1e3:8.1f} us dense {td*1e3:8.1f} us  x{td/ts:.2f}"
                      f"   (eager {row['eager_sparse_us']:.1f} / {row['eager_dense_us']:.1f})", flush=True)
            del ws, wd
    ops.device_status()
    table = {"min_m": {}, "max_m": {}, "decode_max_m": {}}
    for cls in SHAPES:
        win = {}
        for M in TOKENS:      # a class wins at M only if every shape of the class wins
            win[M] = all(r["speedup"] >= a.min_speedup for r in rows if r["class"] == cls and r["M"] == M)
        min_m = None
        for M in reversed(TOKENS):
            if win[M]:
                min_m = M
            else:
                break
        dec = 0
        for M in TOKENS:
            if win[M]:
                dec = M
            else:
                break
        if all(win.values()):                  # one band covering everything
            min_m, dec = 1, 0
        table["min_m"][cls] = min_m if min_m is not None else 1 << 30
        table["max_m"][cls] = 1 << 20
        table["decode_max_m"][cls] = dec
    out = {"gpu": torch.cuda.get_device_name(0), "dtype": a.dtype, "min_speedup": a.min_speedup, **table,
           "measurements": rows}
    with open(a.out, "w") as fh:
        json.dump(out, fh, indent=1)
    print(json.dumps(table))


if __name__ == "__main__":
    main()
