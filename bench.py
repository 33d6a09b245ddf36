#!/usr/bin/env python3
"""Benchmark of the 2:4-sparse gated FFN hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = one forward of the gated FFN  out = down(silu(gate(x)) * up(x))  over one batch of
synthetic tokens, both GEMMs 2:4-sparse.  Default workload: Llama-7B shapes (hidden 4096,
intermediate 11008), 4096 prefill tokens, bf16, weights N(0, 0.02) pruned 2:4, x ~ N(0, 1), seeded.
With N > 1 the same FFN is tensor-parallel (column-parallel gate/up, row-parallel down, NCCL
all-reduce): total work fixed, "scaling": "strong".

Prints ONE JSON line (rank 0).  `value` is dense-equivalent TFLOP/s (6*M*H*I / t) with inputs
resident in HBM; `e2e` is the same metric through the host-buffer C-ABI call, with the host->device
copy of x and the device->host copy of the result inside the timed region.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
_REAL_STDOUT = 1

WORKLOADS = {
    # name: (hidden, intermediate, tokens)
    "llama7b_ffn": (4096, 11008, 4096),
    "mistral7b_ffn": (4096, 14336, 4096),
    "llama70b_ffn": (8192, 28672, 8192),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the gate|up kernel, from the ncu
# capture summarised in profiles/ (None until a capture of that workload exists).
NCU_TRAFFIC_BYTES = {
    # profiles/sparse_gemm_pair_gate_up_llama7b.md: 149.2 MB measured at M = 2048, scaled to M = 4096
    # (weights fixed, activations and outputs proportional to M)
    "llama7b_ffn": 196.2e6,
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama7b_ffn", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="override the token count")
    ap.add_argument("--tp-switch", action="store_true", help="N > 1, fused path: all-gather through NVSwitch-replicated stores")
    ap.add_argument("--tp-phases", action="store_true", help="N > 1, fused path: print per-phase device times to stderr")
    ap.add_argument("--chunks", type=int, default=1, help="token chunks for all-reduce overlap (N > 1, --tp nccl)")
    ap.add_argument("--tp", default="fused", choices=["fused", "nccl"],
                    help="N > 1: exchange step fused into the kernels over peer memory, or NCCL all-reduce")
    ap.add_argument("--cpu-tokens", type=int, default=0, help="tokens of the CPU baseline sample (0 = auto)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------
# clocks
class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs (read-only NVML queries,
    every 2 ms; falls back to polling nvidia-smi when the NVML binding is missing)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.sm = []
        self.power = []
        self.max_sm = 0.0
        self.reasons = set()
        self._stop = threading.Event()
        self._t = None
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self._nvml = pynvml
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    @staticmethod
    def _physical_index(index: int) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                return int(vis.split(",")[index])
            except (ValueError, IndexError):
                return index
        return index

    def _sample_nvml(self):
        n = self._nvml
        self.sm.append(float(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
        try:
            self.power.append(n.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
        except Exception:
            pass
        r = n.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons") \
            else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        for name, bit in (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20),
                          ("hw_thermal_slowdown", 0x40)):
            if r & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                              "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
        f = [v.strip() for v in out.strip().split(",")]
        if len(f) >= 7:
            self.sm.append(float(f[0]))
            self.max_sm = max(self.max_sm, float(f[1]))
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.002)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_sm or None,
                "reasons": sorted(self.reasons), "samples": len(sm),
                "power_w_max": max(self.power) if self.power else None,
                "source": "nvml" if self._nvml is not None else "nvidia-smi"}


# ------------------------------------------------------------------------------------------------
def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return float(p["bf16_tflops"]), float(p["bf16_tflops_sustained"]), float(p["hbm_gbs"]), "measured"
    except Exception:
        return 1590.0, 1400.0, 6650.0, "fallback"


def cpu_reference_ffn(H, I, tokens, threads, reps=1):
    """The reference's CPU path on a sample of `tokens` tokens: oracle pruning of seeded weights is
    done once outside the timing (weights are pruned at load time in both arms); timed: the
    fp32-accumulated gated FFN on the pruned weights, all host threads."""
    import numpy as np
    import torch
    import oracle as o
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(1)
    ws = []
    for shape, seed in (((I, H), 1), ((I, H), 2), ((H, I), 3)):
        gen = torch.Generator().manual_seed(seed)
        w = (torch.randn(shape, generator=gen) * 0.02).numpy()
        ws.append(torch.from_numpy(o.to_f32(o.prune_24_pruned_chunked(o.from_f32(w, "bf16"), "bf16"), "bf16")))
    x = torch.randn(tokens, H, generator=g).bfloat16().float()
    wg, wu, wd = ws

    def step():
        gt = (x @ wg.T)
        ut = (x @ wu.T)
        h = (torch.nn.functional.silu(gt) * ut).bfloat16().float()
        return (h @ wd.T).bfloat16()

    step()
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        best = min(best, time.perf_counter() - t0)
    return best


def pick_cpu_tokens(H, I, threads, want_seconds=3.0):
    # assume ~15 GFLOP/s per thread for fp32 sgemm; clamp to [64, 1024]
    flops_per_tok = 6.0 * H * I
    toks = int(want_seconds * threads * 15e9 / flops_per_tok)
    return max(64, min(1024, (toks // 64) * 64))


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU path (oracle port) timed on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    H, I, M = WORKLOADS[args.workload]
    if args.tokens:
        M = args.tokens
    threads = os.cpu_count() or 1
    toks = args.cpu_tokens or pick_cpu_tokens(H, I, threads)
    steps = max(1, min(args.steps, 5))
    warm = 1
    t = cpu_reference_ffn(H, I, toks, threads, reps=steps)     # one untimed warm-up step inside
    tflops = 6.0 * toks * H * I / t / 1e12
    line = {
        "impl": "reference", "metric": "dense_equiv_tflops_gated_ffn", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": t * 1e3 * (M / toks),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: hidden {H}, intermediate {I}, {M} tokens, bf16, 2:4-pruned gate/up/down",
                   "hidden": H, "intermediate": I, "tokens": M},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"{toks} of {M} tokens, fp32 matmul on oracle-pruned weights, torch CPU, best of {steps}"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------------------------------
def emit(line: dict) -> None:
    """Write the one JSON line to the process's ORIGINAL stdout."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


def _p50_p95(xs):
    """Median and 95th percentile of per-step device times (the reference's demo reports these two,
    demo/demo_harness.py:90-102)."""
    xs = sorted(xs)
    return [xs[len(xs) // 2], xs[min(len(xs) - 1, int(round(0.95 * (len(xs) - 1))))]]


def main():
    args = parse_args()
    # Libraries (NCCL's version banner, for one) print to file descriptor 1.  Point fd 1 at stderr for
    # the rest of the run and keep the original for the JSON line, so stdout carries exactly one line.
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from sparseflow_b200 import _lib, ops, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    H, I, M = WORKLOADS[args.workload]
    if args.tokens:
        M = args.tokens
    dt = torch.bfloat16

    # ---- synthetic, seeded inputs (generated on the CPU so every rank and the oracle see the same bits)
    def seeded(shape, seed, sigma):
        g = torch.Generator().manual_seed(seed)
        return (torch.randn(shape, generator=g, dtype=torch.float32) * sigma).to(dt)

    wg = seeded((I, H), 1, 0.02).to(dev)
    wu = seeded((I, H), 2, 0.02).to(dev)
    wd = seeded((H, I), 3, 0.02).to(dev)
    x_host = seeded((M, H), 1234, 1.0).pin_memory()
    x = x_host.to(dev)

    # ---- weights: prune + compress once (load time), timed separately
    # (output buffers allocated once: the timed loop is 20 back-to-back launches through the C ABI)
    pv = torch.empty((H, I // 2), dtype=dt, device=dev)
    pm = torch.empty(_lib.lib().sfb200_meta_bytes(H, I), dtype=torch.uint8, device=dev)
    st0 = torch.cuda.current_stream().cuda_stream

    def prune_once():
        _lib.check("sfb200_prune_compress_24", _lib.lib().sfb200_prune_compress_24(
            wd.data_ptr(), H, I, I, ops.BF16, 0, pv.data_ptr(), pm.data_ptr(), None, None, st0))
    for _ in range(5):
        prune_once()
    torch.cuda.synchronize()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(20):
        prune_once()
    t1.record(); torch.cuda.synchronize()
    prune_ms = t0.elapsed_time(t1) / 20
    del pv, pm
    prune_gbs = H * I * 3.125 / (prune_ms * 1e-3) / 1e9

    tp_mode = "single GPU"
    ffn = None
    if world > 1 and args.tp == "fused":
        try:
            ffn = parallel.FusedTensorParallelFFN(wg, wu, wd, max_tokens=M, use_switch_stores=args.tp_switch)
            tp_mode = "fused: reduce-scatter in the down-GEMM epilogue (TMA stores to peer memory), all-gather in the reduction kernel"
        except Exception as exc:      # symmetric memory unavailable on this box: NCCL path
            sys.stderr.write(f"fused tensor-parallel path unavailable ({exc!r}); using NCCL all-reduce\n")
            ffn = None
    if ffn is None:
        ffn = parallel.TensorParallelFFN(wg, wu, wd, chunks=args.chunks)
        if world > 1:
            tp_mode = f"NCCL all-reduce after the down GEMM, {args.chunks} chunk(s)"
    fused_tp = isinstance(ffn, parallel.FusedTensorParallelFFN)
    del wg, wu
    hidden = torch.empty((M, ffn.Ip), dtype=dt, device=dev)
    out = torch.empty((M, H), dtype=dt, device=dev)

    def run_step():
        if fused_tp:
            return ffn.forward(x)
        return ffn.forward(x, hidden, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up
    for _ in range(max(3, args.warmup)):
        run_step()
    barrier()
    ops.device_status()

    timed_step = run_step

    # ---- timed region: K steps; per-step events also bracket the gate|up kernel for the roofline
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches0 = ffn.kernel_launches
    barrier()
    s0 = torch.cuda.Event(enable_timing=True); s1 = torch.cuda.Event(enable_timing=True)
    s0.record()
    host_t0 = time.perf_counter()
    if world == 1 and args.chunks == 1:
        for k in range(args.steps):
            ev[k][0].record()
            ops.sparse_gemm_swiglu(x, ffn.gu, out=hidden)
            ev[k][1].record()
            ops.sparse_gemm(hidden, ffn.dn, out=out)
            ev[k][2].record()
            ffn.kernel_launches += 2
    else:
        for k in range(args.steps):
            timed_step()
    host_enqueue_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps
    s1.record()
    barrier()
    clocks = sampler.stop()
    launches = ffn.kernel_launches - launches0
    if fused_tp and args.tp_phases:       # after the timed region: ten more steps with events between the phases
        names = ["gate_up_gemm", "down_gemm_scatter", "barrier_1", "reduce_allgather", "barrier_2"]
        acc = [0.0] * 5
        for _ in range(10):
            evs = []
            ffn.forward(x, phase_events=evs)
            torch.cuda.synchronize()
            for i in range(5):
                acc[i] += evs[i].elapsed_time(evs[i + 1]) / 10
        sys.stderr.write(f"rank {rank} phases (ms): " + ", ".join(f"{n} {t:.4f}" for n, t in zip(names, acc)) + "\n")
    ops.device_status()
    ms_total = s0.elapsed_time(s1)
    tmax = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms_step = float(tmax.item()) / args.steps
    flops = 6.0 * M * H * I
    value = flops / (ms_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel (gate|up GEMM with SiLU.mul epilogue)
    burst, sustained, hbm, src = measured_peaks()
    roof = None
    if world == 1 and args.chunks == 1:
        gu_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
        dn_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
        gu_flops = 2.0 * M * (2 * I) * H
        achieved = gu_flops / (gu_ms * 1e-3) / 1e12
        peak = 2.0 * burst          # 2:4-sparse rate = 2 x the measured dense bf16 burst figure
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                "kernel": "sparse_gemm_pair_kernel<256,128,4,SwiGLU> (gate|up)",
                "peak_source": f"2 x bf16_tflops ({src}); of {'measured' if src == 'measured' else 'fallback'}",
                "frac_of_sustained": achieved / (2.0 * sustained),
                "ms_per_launch": gu_ms,
                "step_ms_p50_p95": _p50_p95([e[0].elapsed_time(e[2]) for e in ev]),
                "down_kernel": {"ms_per_launch": dn_ms, "achieved": 2.0 * M * H * I / (dn_ms * 1e-3) / 1e12}}

    # ---- end to end through the host-buffer C-ABI call (H2D of x, FFN, D2H of out, every step)
    e2e = None
    if world == 1:
        L = _lib.lib()
        W = _lib.FFNWeights(H, I, ops.BF16, ffn.gu.values.data_ptr(), ffn.gu.meta.data_ptr(),
                            ffn.dn.values.data_ptr(), ffn.dn.meta.data_ptr(), None)
        out_host = torch.empty((M, H), dtype=dt).pin_memory()
        st = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            _lib.check("sfb200_ffn_forward_host", L.sfb200_ffn_forward_host(C.byref(W), x_host.data_ptr(), out_host.data_ptr(), M, st))
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            L.sfb200_ffn_forward_host(C.byref(W), x_host.data_ptr(), out_host.data_ptr(), M, st)
        e1.record(); torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / args.steps
        launches += 2 * args.steps
        assert torch.equal(out_host.to(dev), out), "host-buffer path and device path disagree"
        e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": M * H * 2, "d2h_bytes_per_step": M * H * 2, "ms_per_step": e2e_ms}
    else:
        # TP: every rank copies the replicated x in and rank 0 reads the result back
        out_host = torch.empty((M, H), dtype=dt).pin_memory()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            x.copy_(x_host, non_blocking=True)
            res = timed_step()
            if rank == 0:
                out_host.copy_(res, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        e1.record(); barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / args.steps
        e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": M * H * 2 * world, "d2h_bytes_per_step": M * H * 2, "ms_per_step": e2e_ms}

    # ---- dense cuBLAS on the same pruned weights, same shapes (library GEMM; the comparison line)
    dense = None
    if world == 1:
        wgu_d = torch.cat([ops.decompress_24(ops.compress_weight(seeded((I, H), s, 0.02).to(dev))) for s in (1, 2)], 0)
        wd_d = ops.decompress_24(ffn.dn)

        def dense_step():
            gu = torch.matmul(x, wgu_d.t())
            g, u = gu.chunk(2, dim=-1)
            h = torch.nn.functional.silu(g) * u
            return torch.matmul(h, wd_d.t())

        for _ in range(3):
            dense_step()
        torch.cuda.synchronize()
        d0 = torch.cuda.Event(enable_timing=True); d1 = torch.cuda.Event(enable_timing=True); d2 = torch.cuda.Event(enable_timing=True)
        d0.record()
        for _ in range(args.steps):
            dense_step()
        d1.record()
        for _ in range(args.steps):
            torch.matmul(x, wgu_d.t())
        d2.record(); torch.cuda.synchronize()
        dense_ms = d0.elapsed_time(d1) / args.steps
        gemm_gu_ms = d1.elapsed_time(d2) / args.steps
        dense = {"ffn_ms": dense_ms, "ffn_tflops": flops / (dense_ms * 1e-3) / 1e12,
                 "speedup_ffn": dense_ms / ms_step,
                 "gate_up_gemm_ms": gemm_gu_ms, "gate_up_gemm_tflops": 2.0 * M * 2 * I * H / (gemm_gu_ms * 1e-3) / 1e12,
                 "what": "torch.matmul (cuBLAS) on the same 2:4-pruned weights stored dense + torch silu*mul"}
        del wgu_d, wd_d

    # ---- CPU baseline (rank 0, N = 1): the oracle's FFN on a bounded token sample
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        toks = args.cpu_tokens or pick_cpu_tokens(H, I, threads)
        t = cpu_reference_ffn(H, I, toks, threads, reps=2)
        cpu = {"value": 6.0 * toks * H * I / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"{toks} of {M} tokens, fp32 matmul on oracle-pruned weights, torch CPU, best of 2"}

    if rank == 0:
        line = {
            "metric": "dense_equiv_tflops_gated_ffn", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: hidden {H}, intermediate {I}, {M} tokens, bf16, 2:4-pruned gate/up/down",
                       "hidden": H, "intermediate": I, "tokens": M,
                       "parallelism": "single GPU" if world == 1 else f"tp{world}: column-parallel gate/up, row-parallel down; {tp_mode}",
                       "l2": "no flush: per-step working set (weights 152 MB + activations 157 MB for the default workload) exceeds the 126 MB L2"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "host_enqueue_ms_per_step": host_enqueue_ms,
            "roofline": roof, "cpu_baseline": cpu, "dense_cublas": dense,
            "prune_compress": {"ms": prune_ms, "gbs": prune_gbs, "frac_of_hbm": prune_gbs / hbm,
                               "what": f"down weight {H}x{I}, 3.125 B/element algorithmic"},
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
