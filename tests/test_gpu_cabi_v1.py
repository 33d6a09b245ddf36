"""The reference's C ABI v1 compute calls and its runtime selection API, run on the GPU through ctypes.

Upstream declares ``sparseflow_sparse_gemm / _compress_2_4 / _validate_2_4 / _benchmark_kernel``
(experiments/old_structure/include/sparseflow/c_api.h:151-195) and leaves them as NOT_SUPPORTED stubs
(src/runtime/context.cpp:248-300); here they run the sm_100a kernels, so they are checked like any other
compute path: compressed values and metadata bit for bit against the oracle, GEMM outputs within 1e-2 of the
fp32 oracle for every epilogue kind.  The selection API (``sf_select_kernel*``) is driven through its
measure-and-persist branch (runtime/dispatch/kernel_dispatcher.cpp:105-185), and the bounded device-side
wait is made to run out once, harmlessly, to check the failure report and the quarantine that follows it
(runtime/dispatch/eligibility_policy.cpp:72-84).
"""
import ctypes as C
import sqlite3

import numpy as np
import pytest
import torch

import oracle as o
from sparseflow_b200 import _lib, ops
from tests.util import bits_of, seeded_act, seeded_weight, to_dev

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2

FP16, BF16 = 0, 3                     # SparseFlowDataType
EPI = {"none": 0, "relu": 1, "silu": 2, "gelu": 3, "bias": 4, "bias_relu": 5, "bias_silu": 6}


class EpilogueConfig(C.Structure):
    _fields_ = [("kind", C.c_int), ("params", C.c_void_p), ("params_size", C.c_size_t)]


class KernelConfig(C.Structure):
    _fields_ = [("tile_m", C.c_int), ("tile_n", C.c_int), ("tile_k", C.c_int), ("epilogue", EpilogueConfig)]


class BenchResult(C.Structure):
    _fields_ = [("elapsed_ms", C.c_double), ("tflops_effective", C.c_double), ("tflops_real", C.c_double),
                ("bandwidth_gb_s", C.c_double)]


@pytest.fixture(scope="module")
def abi():
    L = _lib.lib()
    vp, i = C.c_void_p, C.c_int
    L.sparseflow_create_context.argtypes = [C.POINTER(vp), i]
    L.sparseflow_destroy_context.argtypes = [vp]
    L.sparseflow_compile_kernel.argtypes = [vp, C.POINTER(vp), C.POINTER(KernelConfig)]
    L.sparseflow_destroy_kernel.argtypes = [vp]
    L.sparseflow_sparse_gemm.argtypes = [vp, vp, vp, vp, i, i, i, i, vp]
    L.sparseflow_compress_2_4.argtypes = [vp, vp, vp, vp, i, i, i]
    L.sparseflow_validate_2_4.argtypes = [vp, i, i, i, C.POINTER(i)]
    L.sparseflow_benchmark_kernel.argtypes = [vp, i, i, i, i, C.POINTER(BenchResult)]
    L.sparseflow_compressed_meta_offset.restype = C.c_size_t
    L.sparseflow_compressed_meta_offset.argtypes = [i, i]
    L.sparseflow_get_last_error.restype = C.c_char_p
    L.sparseflow_get_device_info.argtypes = [vp, C.POINTER(i), C.POINTER(i), C.POINTER(C.c_size_t)]
    return L


@pytest.fixture()
def ctx(abi):
    h = C.c_void_p()
    assert abi.sparseflow_create_context(C.byref(h), 0) == 0, abi.sparseflow_get_last_error()
    yield h
    assert abi.sparseflow_destroy_context(h) == 0


def _compressed_block(abi, ctx, w_dev, N, K, dtype_code):
    """dense [N, K] on the device -> the block sparseflow_sparse_gemm takes (values | pad | metadata)."""
    moff = abi.sparseflow_compressed_meta_offset(N, K)
    blk = torch.zeros(moff + abi.sfb200_meta_bytes(N, K), dtype=torch.uint8, device="cuda")
    rc = abi.sparseflow_compress_2_4(ctx, w_dev.data_ptr(), blk.data_ptr(), blk.data_ptr() + moff, N, K, dtype_code)
    assert rc == 0, abi.sparseflow_get_last_error()
    torch.cuda.synchronize()
    return blk, moff


@pytest.mark.parametrize("dt,code", [("f16", FP16), ("bf16", BF16)])
def test_device_info_compress_and_validate(abi, ctx, dt, code):
    cc, sms, mem = C.c_int(), C.c_int(), C.c_size_t()
    assert abi.sparseflow_get_device_info(ctx, C.byref(cc), C.byref(sms), C.byref(mem)) == 0
    assert cc.value == 100 and sms.value >= 100 and mem.value > (100 << 30)
    N, K = 392, 1088                                  # rows not a multiple of 128, K with a 64-wide tail
    w = seeded_weight(N, K, dt, 21)
    wd = to_dev(w, dt)
    blk, moff = _compressed_block(abi, ctx, wd, N, K, code)
    oc = o.prune_24(w, dt)
    host = blk.cpu().numpy()
    vals = host[:N * (K // 2) * 2].view(np.uint16).reshape(N, K // 2)
    assert (vals == oc["values"]).all()                                           # compressed values: bit-exact
    meta = host[moff:].view(np.uint32)
    assert (meta == o.hw_meta_tiled(oc["idx0"], oc["idx1"]).reshape(-1)).all()   # metadata: bit-exact
    # validate: the dense weight is not 2:4, its pruned form is
    ok = C.c_int(-1)
    assert abi.sparseflow_validate_2_4(wd.data_ptr(), N, K, code, C.byref(ok)) == 0 and ok.value == 0
    pruned = to_dev(oc["pruned"], dt)
    assert abi.sparseflow_validate_2_4(pruned.data_ptr(), N, K, code, C.byref(ok)) == 0 and ok.value == 1
    # compressing the pruned form again changes nothing (idempotent on a 2:4 tensor)
    blk2, _ = _compressed_block(abi, ctx, pruned, N, K, code)
    assert torch.equal(blk, blk2)
    # argument errors keep the reference's codes
    assert abi.sparseflow_validate_2_4(None, N, K, code, C.byref(ok)) == 1
    assert abi.sparseflow_compress_2_4(ctx, wd.data_ptr(), None, None, N, K, code) == 1
    assert abi.sparseflow_compress_2_4(ctx, wd.data_ptr(), blk.data_ptr(), blk.data_ptr() + moff, N, K, 1) == 4   # FP32


@pytest.mark.parametrize("kind", list(EPI))
@pytest.mark.parametrize("dt,code", [("f16", FP16), ("bf16", BF16)])
def test_sparse_gemm_every_epilogue_kind(abi, ctx, kind, dt, code):
    M, N, K = 200, 392, 512
    w, x = seeded_weight(N, K, dt, 31), seeded_act(M, K, dt, 32)
    bias = seeded_act(1, N, dt, 33)[0]
    bias_dev = to_dev(bias, dt)
    blk, _ = _compressed_block(abi, ctx, to_dev(w, dt), N, K, code)
    cfg = KernelConfig(0, 0, 0, EpilogueConfig(EPI[kind], bias_dev.data_ptr() if "bias" in kind else None, N * 2))
    kern = C.c_void_p()
    assert abi.sparseflow_compile_kernel(ctx, C.byref(kern), C.byref(cfg)) == 0, abi.sparseflow_get_last_error()
    xd = to_dev(x, dt)
    y = torch.zeros(M, N, device="cuda", dtype=xd.dtype)
    st = torch.cuda.current_stream().cuda_stream
    rc = abi.sparseflow_sparse_gemm(kern, xd.data_ptr(), blk.data_ptr(), y.data_ptr(), M, N, K, code, st)
    assert rc == 0, abi.sparseflow_get_last_error()
    assert ops.device_status() == 0
    ref = o.gemm_ref(x, o.prune_24(w, dt)["pruned"], dt)
    if "bias" in kind:
        ref = ref + o.to_f32(bias, dt)[None, :]
    if "relu" in kind:
        ref = np.maximum(ref, 0)
    elif "silu" in kind:
        ref = ref / (1 + np.exp(-ref))
    elif "gelu" in kind:
        ref = torch.nn.functional.gelu(torch.from_numpy(ref)).numpy()
    m = o.rel_err_metrics(o.to_f32(bits_of(y), dt), ref)
    assert m["floor"] <= REL_TOL, (kind, m)
    # errors: FP32 has no sparse kernel, NULL matrices are refused, a NULL handle is invalid
    assert abi.sparseflow_sparse_gemm(kern, xd.data_ptr(), blk.data_ptr(), y.data_ptr(), M, N, K, 1, st) == 4
    assert abi.sparseflow_sparse_gemm(kern, None, blk.data_ptr(), y.data_ptr(), M, N, K, code, st) == 1
    assert abi.sparseflow_sparse_gemm(None, xd.data_ptr(), blk.data_ptr(), y.data_ptr(), M, N, K, code, st) == 5
    assert abi.sparseflow_destroy_kernel(kern) == 0


def test_compile_kernel_rejects_bias_epilogue_without_params(abi, ctx):
    cfg = KernelConfig(0, 0, 0, EpilogueConfig(EPI["bias"], None, 0))
    kern = C.c_void_p()
    assert abi.sparseflow_compile_kernel(ctx, C.byref(kern), C.byref(cfg)) == 1
    cfg = KernelConfig(0, 100, 0, EpilogueConfig(EPI["none"], None, 0))     # not a token tile the kernels have
    assert abi.sparseflow_compile_kernel(ctx, C.byref(kern), C.byref(cfg)) == 6


def test_benchmark_kernel_reports_sane_figures(abi, ctx):
    cfg = KernelConfig(0, 0, 0, EpilogueConfig(EPI["none"], None, 0))
    kern = C.c_void_p()
    assert abi.sparseflow_compile_kernel(ctx, C.byref(kern), C.byref(cfg)) == 0
    r = BenchResult()
    M, N, K = 2048, 4096, 4096
    assert abi.sparseflow_benchmark_kernel(kern, M, N, K, 10, C.byref(r)) == 0, abi.sparseflow_get_last_error()
    assert 0.005 < r.elapsed_ms < 5.0
    assert abs(r.tflops_effective - 2.0 * M * N * K / (r.elapsed_ms * 1e9)) < 1e-6 * r.tflops_effective
    assert abs(r.tflops_real - 0.5 * r.tflops_effective) < 1e-9 + 1e-6 * r.tflops_effective
    assert 50 < r.tflops_effective < 4500 and r.bandwidth_gb_s > 10
    assert abi.sparseflow_benchmark_kernel(kern, M, N, 100, 10, C.byref(r)) == 1     # K % 64 != 0
    assert abi.sparseflow_destroy_kernel(kern) == 0


# ------------------------------------------------------------------------------------------------ sf_*
def _gpu_info():
    p = torch.cuda.get_device_properties(0)
    return _lib.GpuInfo(p.major * 10 + p.minor, p.multi_processor_count, 227)


def _row(db, like):
    con = sqlite3.connect(db)
    r = con.execute("SELECT best_kernel, best_gflops, sparse_failed, failure_count FROM kernel_cache WHERE key_hash LIKE ?",
                    (like,)).fetchone()
    con.close()
    return r


def _counters(L, db):
    out = (C.c_int64 * 8)()
    assert L.sf_get_counters(db, out, 8) == 8
    return dict(zip(("calls", "hits", "misses", "benchmarks", "dense", "sparse", "failures", "forced"), out))


@pytest.mark.parametrize("wm,tokens,K", [(4096, 4096, 4096), (22016, 2048, 4096)])
def test_select_kernel_measures_persists_and_hits(tmp_path, wm, tokens, K):
    """An eligible 2:4 shape whose weight is known to be compressed: both candidates are timed, the winner
    (the sparse prefill kernel at these sizes) is persisted with its GFLOPS, the second call is a hit."""
    L = _lib.lib()
    db = str(tmp_path / "sel.db").encode()
    g = _gpu_info()
    d = _lib.MatmulDesc(wm, tokens, K, 1, 1, 0.5, 0)          # M = weight rows, N = tokens, bf16, 2:4
    L.sf_note_compressed(db, C.byref(d))
    k = L.sf_select_kernel(db, C.byref(d), C.byref(g))
    assert k == 2
    row = _row(db.decode(), f"M={L.sf_bucket_dimension(wm)};N={L.sf_bucket_dimension(tokens)};%")
    assert row is not None and row[0] == 2 and row[1] > 1e5 and row[2] == 0, row      # > 100 TFLOP/s recorded
    c = _counters(L, db)
    assert c["benchmarks"] == 1 and c["sparse"] == 1 and c["hits"] == 0
    assert L.sf_select_kernel(db, C.byref(d), C.byref(g)) == 2
    c = _counters(L, db)
    assert c["hits"] == 1 and c["benchmarks"] == 1
    assert ops.device_status() == 0


def test_select_kernel_ex_uses_content_keyed_compressed_store(tmp_path):
    """The dispatcher call with device matrices (upstream's C++ form): a weight that has not been compressed is
    not eligible and the shape is cached as dense; once sf_compress_weight has stored its compressed form the
    same call on a fresh cache measures on the caller's matrices and picks sparse; the compressed form in the
    store is the oracle's, bit for bit."""
    L = _lib.lib()
    dt, wm, tokens, K = "bf16", 4096, 2048, 4096
    w, x = seeded_weight(wm, K, dt, 41), seeded_act(tokens, K, dt, 42)
    wd, xd = to_dev(w, dt), to_dev(x, dt)
    y = torch.zeros(tokens, wm, device="cuda", dtype=torch.bfloat16)
    g = _gpu_info()
    d = _lib.MatmulDesc(wm, tokens, K, 1, 1, 0.5, 0)
    L.sf_compressed_cache_clear()
    db1 = str(tmp_path / "a.db").encode()
    assert L.sf_select_kernel_ex(db1, C.byref(d), C.byref(g), wd.data_ptr(), xd.data_ptr(), y.data_ptr()) == 0
    assert _row(db1.decode(), "M=4096;%")[:2] == (0, 0.0)              # "compression not cached": dense, unmeasured
    vals, meta = C.c_void_p(), C.c_void_p()
    assert L.sf_compress_weight(C.byref(d), wd.data_ptr(), C.byref(vals), C.byref(meta)) == 1
    assert L.sf_compressed_cache_count() == 1
    assert L.sf_compressed_cache_bytes() == L.sfb200_values_bytes(wm, K) + L.sfb200_meta_bytes(wm, K)
    v2, m2 = C.c_void_p(), C.c_void_p()
    assert L.sf_compress_weight(C.byref(d), wd.data_ptr(), C.byref(v2), C.byref(m2)) == 1
    assert (v2.value, m2.value) == (vals.value, meta.value) and L.sf_compressed_cache_count() == 1    # same content: a hit
    oc = o.prune_24(w, dt)
    back = torch.empty(wm, K, dtype=torch.bfloat16, device="cuda")     # the stored form, decompressed: the oracle's pruned weight
    assert L.sfb200_decompress_24(vals, meta, wm, K, back.data_ptr(), K, None) == 0
    torch.cuda.synchronize()
    assert (bits_of(back) == oc["pruned"]).all()
    db2 = str(tmp_path / "b.db").encode()
    assert L.sf_select_kernel_ex(db2, C.byref(d), C.byref(g), wd.data_ptr(), xd.data_ptr(), y.data_ptr()) == 2
    assert _row(db2.decode(), "M=4096;%")[0] == 2
    # the timed launches wrote the caller's output; the dense candidate ran last, on the caller's weight as given
    ref = o.gemm_ref(x[:64], w, dt)
    assert o.rel_err_metrics(o.to_f32(bits_of(y[:64]), dt), ref)["floor"] <= REL_TOL
    # a different weight of the same shape is a different key
    w2 = to_dev(seeded_weight(wm, K, dt, 43), dt)
    db3 = str(tmp_path / "c.db").encode()
    assert L.sf_select_kernel_ex(db3, C.byref(d), C.byref(g), w2.data_ptr(), xd.data_ptr(), y.data_ptr()) == 0
    # a shape the sparse kernel does not take (K % 64 != 0) is dense even when declared compressed
    odd = _lib.MatmulDesc(4096, 2048, 4000, 1, 1, 0.5, 0)
    L.sf_note_compressed(db3, C.byref(odd))
    assert L.sf_select_kernel(db3, C.byref(odd), C.byref(g)) == 0
    L.sf_compressed_cache_clear()
    assert L.sf_compressed_cache_count() == 0 and L.sf_compressed_cache_bytes() == 0
    assert ops.device_status() == 0


# ------------------------------------------------------------------------------------------------ failure path
def test_bounded_wait_runs_out_reports_and_quarantines(tmp_path):
    """One small CTA waits 2 ms on a barrier nothing arrives on: the wait gives up, the kernel records the
    status and returns by itself.  The host then sees SFB200_ERROR_DEVICE with (1 << 8) | where, the word is
    cleared by the read, the next GEMM on the device is correct, and three failure reports quarantine the
    shape in the selection cache."""
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    assert ops.device_status() == 0
    assert L.sfb200_debug_wait_timeout(2000, 7, 0, st) == 0
    w = C.c_int(0)
    assert L.sfb200_device_status(C.byref(w)) == 9                  # SFB200_ERROR_DEVICE
    assert w.value == (1 << 8) | 7
    assert L.sfb200_device_status(C.byref(w)) == 0 and w.value == 0      # cleared by the read
    with pytest.raises(_lib.SfbError):
        L.sfb200_debug_wait_timeout(1000, 3, 0, st)
        ops.device_status()
    assert ops.device_status() == 0
    # the context is intact: a GEMM right after is correct
    dt = "bf16"
    wt, x = seeded_weight(256, 512, dt, 51), seeded_act(100, 512, dt, 52)
    y = ops.sparse_gemm(to_dev(x, dt), ops.compress_weight(to_dev(wt, dt)))
    assert ops.device_status() == 0
    assert o.rel_err_metrics(o.to_f32(bits_of(y), dt), o.gemm_ref(x, o.prune_24(wt, dt)["pruned"], dt))["floor"] <= REL_TOL
    # the word of the allocation-free entry point is read by its own call and folded into the general one
    assert L.sfb200_debug_wait_timeout(1000, 9, 1, st) == 0
    assert L.sfb200_noalloc_device_status(C.byref(w)) == 9 and w.value == (1 << 8) | 9
    assert L.sfb200_noalloc_device_status(C.byref(w)) == 0 and w.value == 0
    assert L.sfb200_debug_wait_timeout(1000, 11, 1, st) == 0
    assert L.sfb200_device_status(C.byref(w)) == 9 and w.value == (1 << 8) | 11
    assert ops.device_status() == 0
    # argument checks of the probe: the limit is capped at 0.1 s
    assert L.sfb200_debug_wait_timeout(0, 1, 0, st) == 1 and L.sfb200_debug_wait_timeout(200000, 1, 0, st) == 1
    # what a caller does with such a report: three of them and the shape is never offered sparse again
    db = str(tmp_path / "q.db").encode()
    g = _gpu_info()
    d = _lib.MatmulDesc(4096, 2048, 4096, 1, 1, 0.5, 0)
    L.sf_note_compressed(db, C.byref(d))
    for _ in range(3):
        L.sf_record_sparse_failure(db, C.byref(d), C.byref(g))
    assert L.sf_select_kernel(db, C.byref(d), C.byref(g)) == 0
    row = _row(db.decode(), "M=4096;%")
    assert row[2] == 1 and row[3] == 3
    assert _counters(L, db)["benchmarks"] == 0
