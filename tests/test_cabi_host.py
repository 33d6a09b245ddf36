"""Host-side checks of the C-ABI library: it loads, exports every symbol the header declares, keeps
the reference's sf_* selection semantics (tests/test_c_api.cpp) and the C ABI v1 error behaviour
(tests/abi/test_abi_stability.c).  No compute call is made, so no GPU is needed."""
import ctypes as C
import os
import re
import sqlite3
import subprocess

import pytest

from sparseflow_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "sparseflow_b200.h")).read()
    hdr = hdr.replace('#define SFB200_API __attribute__((visibility("default")))', "")
    declared = set(re.findall(r"SFB200_API[^;(]*?\b(\w+)\s*\(", hdr))
    assert len(declared) >= 35
    out = subprocess.check_output(["nm", "-D", "--defined-only", _lib.LIB_PATH]).decode()
    exported = {line.split()[-1] for line in out.splitlines() if line.strip()}
    assert declared <= exported, sorted(declared - exported)


def test_sizes_and_strings(lib):
    assert lib.sfb200_values_bytes(128, 128) == 128 * 64 * 2
    assert lib.sfb200_meta_bytes(128, 128) == 2048
    assert lib.sfb200_meta_bytes(129, 130) == 4 * 2048
    assert lib.sfb200_meta_bytes(22016, 4096) == 172 * 32 * 2048
    assert b"invalid" in lib.sfb200_status_string(1)
    assert lib.sfb200_version() >= 100


def _desc(M=512, N=512, K=512, dtype=0, sp=0, ratio=0.0):
    return _lib.MatmulDesc(M, N, K, dtype, sp, ratio, 0)


def _sf(lib):
    lib.sf_select_kernel.restype = C.c_int32
    lib.sf_select_kernel.argtypes = [C.c_char_p, C.POINTER(_lib.MatmulDesc), C.POINTER(_lib.GpuInfo)]
    lib.sf_cache_size.restype = C.c_int32
    lib.sf_cache_size.argtypes = [C.c_char_p]
    lib.sf_cache_clear.argtypes = [C.c_char_p]
    lib.sf_bucket_dimension.restype = C.c_int32
    lib.sf_bucket_dimension.argtypes = [C.c_int32]
    lib.sf_note_compressed.argtypes = [C.c_char_p, C.POINTER(_lib.MatmulDesc)]
    lib.sf_record_sparse_failure.argtypes = [C.c_char_p, C.POINTER(_lib.MatmulDesc), C.POINTER(_lib.GpuInfo)]
    return lib


def test_sf_api_follows_reference_test_c_api(lib, tmp_path):
    """The sequence of tests/test_c_api.cpp: dense-typed desc, repeat, then M=513 (next bucket)."""
    sf = _sf(lib)
    db = str(tmp_path / "test_c_api.db").encode()
    sf.sf_cache_clear(db)
    d = _desc()
    g = _lib.GpuInfo(86, 82, 100)
    k1 = sf.sf_select_kernel(db, C.byref(d), C.byref(g))
    assert k1 == 0                                   # dense-typed desc is cached as dense
    assert sf.sf_cache_size(db) == 1
    k2 = sf.sf_select_kernel(db, C.byref(d), C.byref(g))
    assert k2 == k1 and sf.sf_cache_size(db) == 1    # cache hit, no new row
    d.M = 513
    sf.sf_select_kernel(db, C.byref(d), C.byref(g))
    assert sf.sf_cache_size(db) == 2                 # 513 buckets to 1024: a second row
    # the table is the reference's schema and key format
    con = sqlite3.connect(db.decode())
    rows = dict(con.execute("SELECT key_hash, best_kernel FROM kernel_cache").fetchall())
    assert "M=512;N=512;K=512;dtype=0;layout=0;sp=0;sm=86" in rows
    assert "M=1024;N=512;K=512;dtype=0;layout=0;sp=0;sm=86" in rows
    cols = [r[1] for r in con.execute("PRAGMA table_info(kernel_cache)")]
    assert cols == ["key_hash", "best_kernel", "best_gflops", "sparse_failed", "failure_count",
                    "last_failure_code", "last_failure_ts"]
    con.close()
    sf.sf_cache_clear(db)
    assert sf.sf_cache_size(db) == 0


def test_sf_bucketing(lib):
    sf = _sf(lib)
    assert [sf.sf_bucket_dimension(v) for v in (0, 1, 32, 33, 512, 513, 2048, 40000, 70000)] == \
        [0, 32, 32, 64, 512, 1024, 2048, 65535, 65535]


def test_sf_eligibility_rules_without_gpu(lib, tmp_path):
    sf = _sf(lib)
    db = str(tmp_path / "elig.db").encode()
    g = _lib.GpuInfo(100, 148, 227)
    small = _desc(64, 64, 64, 1, 1, 0.5)             # 2:4 but under 512^3 flops -> dense, cached
    assert sf.sf_select_kernel(db, C.byref(small), C.byref(g)) == 0
    assert sf.sf_cache_size(db) == 1
    big = _desc(4096, 4096, 4096, 1, 1, 0.5)         # eligible size, compression not cached -> dense, cached
    assert sf.sf_select_kernel(db, C.byref(big), C.byref(g)) == 0
    assert sf.sf_cache_size(db) == 2
    # quarantine bookkeeping lands in the table
    other = _desc(8192, 4096, 4096, 1, 1, 0.5)
    for _ in range(3):
        sf.sf_record_sparse_failure(db, C.byref(other), C.byref(g))
    con = sqlite3.connect(db.decode())
    row = con.execute("SELECT sparse_failed, failure_count FROM kernel_cache WHERE key_hash LIKE 'M=8192;%'").fetchone()
    con.close()
    assert row == (1, 3)


def test_sf_null_path_uses_default_name(lib, tmp_path, monkeypatch):
    sf = _sf(lib)
    monkeypatch.chdir(tmp_path)
    d, g = _desc(), _lib.GpuInfo(100, 148, 227)
    sf.sf_select_kernel(None, C.byref(d), C.byref(g))
    assert os.path.exists(tmp_path / "kernel_cache.db")
    assert sf.sf_cache_size(None) == 1


def _counters(sf, db):
    out = (C.c_int64 * 8)()
    assert sf.sf_get_counters(db, out, 8) == 8
    return dict(zip(("calls", "hits", "misses", "benchmarks", "dense", "sparse", "failures", "forced"), out))


def test_sf_failure_report_does_not_pin_dense(lib, tmp_path):
    """One failure report before the first selection leaves a row with kernel 0 and 0 GFLOPS; that
    row must not be served as a cache hit (the shape would never be measured).  Below three failures
    the selector goes on to eligibility and measurement; from three on the shape is quarantined
    (experiments/old_structure/runtime/dispatch/eligibility_policy.cpp:72-84)."""
    sf = _sf(lib)
    db = str(tmp_path / "stub.db").encode()
    g = _lib.GpuInfo(100, 148, 227)
    d = _desc(4096, 4096, 4096, 1, 1, 0.5)
    sf.sf_note_compressed(db, C.byref(d))
    sf.sf_record_sparse_failure(db, C.byref(d), C.byref(g))
    assert sf.sf_cache_size(db) == 1
    sf.sf_select_kernel(db, C.byref(d), C.byref(g))
    c = _counters(sf, db)
    assert c["hits"] == 0 and c["misses"] == 1 and c["benchmarks"] == 1, c   # measured (or tried to), not a hit
    for _ in range(2):
        sf.sf_record_sparse_failure(db, C.byref(d), C.byref(g))
    con = sqlite3.connect(db.decode())
    con.execute("UPDATE kernel_cache SET best_kernel=0, best_gflops=0")      # back to a bare failure row
    con.commit()
    con.close()
    assert sf.sf_select_kernel(db, C.byref(d), C.byref(g)) == 0
    c2 = _counters(sf, db)
    assert c2["benchmarks"] == c["benchmarks"], c2                           # quarantined: no measurement
    assert c2["failures"] == 3
    # clearing forgets the quarantine as well as the rows
    sf.sf_cache_clear(db)
    assert sf.sf_cache_size(db) == 0
    sf.sf_note_compressed(db, C.byref(d))
    sf.sf_select_kernel(db, C.byref(d), C.byref(g))
    assert _counters(sf, db)["benchmarks"] == c["benchmarks"] + 1


def test_sf_env_overrides(lib, tmp_path, monkeypatch):
    sf = _sf(lib)
    g = _lib.GpuInfo(100, 148, 227)
    monkeypatch.setenv("SPARSEFLOW_CACHE_DB", str(tmp_path / "from_env.db"))
    d = _desc()
    sf.sf_select_kernel(None, C.byref(d), C.byref(g))
    assert os.path.exists(tmp_path / "from_env.db") and sf.sf_cache_size(None) == 1
    db = str(tmp_path / "force.db").encode()
    sp = _desc(4096, 4096, 4096, 1, 1, 0.5)
    odd = _desc(4096, 4096, 4000, 1, 1, 0.5)          # K % 64 != 0: no sparse kernel for it
    monkeypatch.setenv("SPARSEFLOW_FORCE", "sparse")
    assert sf.sf_select_kernel(db, C.byref(sp), C.byref(g)) == 2
    assert sf.sf_select_kernel(db, C.byref(odd), C.byref(g)) == 0
    assert sf.sf_select_kernel(db, C.byref(d), C.byref(g)) == 0      # dense-typed desc stays dense
    monkeypatch.setenv("SPARSEFLOW_FORCE", "dense")
    assert sf.sf_select_kernel(db, C.byref(sp), C.byref(g)) == 0
    assert sf.sf_cache_size(db) == 0                                  # forced decisions are not persisted
    assert _counters(sf, db)["forced"] == 4
    monkeypatch.delenv("SPARSEFLOW_FORCE")


def test_sf_compressed_store_refuses_without_device_or_bad_shape(lib):
    lib.sf_compress_weight.restype = C.c_int32
    d = _desc(4096, 4096, 4096, 2, 1, 0.5)           # fp32: no sparse kernel
    assert lib.sf_compress_weight(C.byref(d), C.c_void_p(16), None, None) == 0
    d = _desc(4096, 4096, 4096, 1, 1, 0.5)
    assert lib.sf_compress_weight(C.byref(d), None, None, None) == 0
    assert lib.sf_compressed_cache_count() >= 0


class _Version(C.Structure):
    _fields_ = [("major", C.c_int), ("minor", C.c_int), ("patch", C.c_int)]


def test_abi_v1_host_behaviour(lib):
    """tests/abi/test_abi_stability.c: version/compat, NULL ctx -> INVALID_ARGUMENT, strings."""
    lib.sparseflow_get_version.restype = _Version
    v = lib.sparseflow_get_version()
    assert (v.major, v.minor) == (1, 1)
    assert lib.sparseflow_is_abi_compatible(1, 0) == 1
    assert lib.sparseflow_is_abi_compatible(1, 7) == 1
    assert lib.sparseflow_is_abi_compatible(2, 0) == 0
    lib.sparseflow_get_error_string.restype = C.c_char_p
    lib.sparseflow_get_last_error.restype = C.c_char_p
    assert lib.sparseflow_get_error_string(0) == b"Success"
    assert lib.sparseflow_get_error_string(5) == b"Invalid handle"
    assert lib.sparseflow_create_context(None, 0) == 1            # NULL out-pointer
    assert b"NULL" in lib.sparseflow_get_last_error()
    assert lib.sparseflow_destroy_context(None) == 5              # NULL handle
    assert lib.sparseflow_destroy_kernel(None) == 5
    is_valid = C.c_int(-1)
    assert lib.sparseflow_validate_2_4(None, 4, 4, 0, C.byref(is_valid)) == 1
    assert lib.sparseflow_sparse_gemm(None, None, None, None, 1, 1, 1, 0, None) == 5
    lib.sparseflow_compressed_meta_offset.restype = C.c_size_t
    assert lib.sparseflow_compressed_meta_offset(128, 128) == 16384
    assert lib.sparseflow_compressed_meta_offset(8, 72) % 256 == 0


def test_compute_calls_fail_loudly_without_a_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    rc = lib.sfb200_prune_compress_24(None, 4, 16, 16, 0, 0, None, None, None, None, None)
    assert rc == 3                                             # SFB200_ERROR_CUDA, not a silent fallback
    ctx = C.c_void_p()
    assert lib.sparseflow_create_context(C.byref(ctx), 0) == 3


def test_package_has_no_oracle_dependency():
    """The product path must not import the oracle."""
    pkg = os.path.join(ROOT, "sparseflow_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cpp", ".h", ".cuh")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(import|from)\s+oracle\b", src, re.M), f


def test_host_pipeline_chunk_plan_covers_every_token():
    """Chunks are multiples of 8 rows (16-byte aligned row offsets for TMA) except the last, at most 8,
    and sum to M for any M and any tuning override."""
    import ctypes as C
    from sparseflow_b200 import _lib
    L = _lib.lib()
    out = (C.c_int * 8)()
    for M in (1, 7, 8, 511, 512, 1000, 1024, 1025, 4096, 5000, 16384, 100000, 1 << 20):
        for main, tail in ((0, 0), (1024, 256), (2048, 512), (512, 128), (64, 8), (4096, 4096)):
            n = L.sfb200_debug_host_chunk_plan(M, main, tail, out)
            plan = list(out[:n])
            assert 1 <= n <= 8 and sum(plan) == M and min(plan) > 0, (M, main, tail, plan)
            assert all(r % 8 == 0 for r in plan[:-1]), (M, main, tail, plan)
    n = L.sfb200_debug_host_chunk_plan(4096, 0, 0, out)
    assert list(out[:n]) == [1024] * 4
    assert L.sfb200_debug_host_chunk_plan(0, 0, 0, out) == 0 and L.sfb200_debug_host_chunk_plan(8, 0, 0, None) == 0


def test_kernel_plan_per_shape():
    """Which kernel the dispatcher runs for the benchmark shapes on a 148-SM GPU (host-only planning call)."""
    from sparseflow_b200 import _lib
    plan = lambda M, N, K, sw=0: _lib.lib().sfb200_debug_plan_gemm(M, N, K, sw, 148)
    # decode: many row tiles -> warp-level kernel up to 4 tokens; few row tiles -> it keeps only 1-2 tokens
    assert plan(1, 28672, 4096) == 8 and plan(4, 28672, 4096) == 8 and plan(4, 22016, 4096, 1) == 8
    assert plan(5, 28672, 4096) == 32 and plan(8, 22016, 4096, 1) == 32
    assert plan(2, 4096, 14336) == 8 and plan(4, 4096, 14336) == 4032
    # few row tiles, below the prefill threshold: split-K over a cluster, 4 slices for 32 tiles, 2 for 64
    assert plan(32, 4096, 11008) == 4032 and plan(64, 4096, 11008) == 4064 and plan(128, 4096, 11008) == 4128
    assert plan(16, 8192, 8192) == 3032 and plan(64, 8192, 8192) == 3064
    # 65..128 tokens: two 64-token tiles where they need no more passes over the SMs than one 128-token tile
    assert plan(128, 8192, 8192) == 64 and plan(128, 4096, 4096) == 64 and plan(128, 22016, 4096) == 64
    assert plan(128, 11008, 4096) == 128 and plan(100, 28672, 4096) == 128
    assert plan(32, 512, 256) == 32                   # too little K to split (< 4 metadata tiles per slice)
    # many row tiles, up to 128 tokens: single-CTA kernel with the smallest covering token tile
    assert plan(9, 22016, 4096) == 32 and plan(33, 22016, 4096) == 64 and plan(100, 11008, 4096) == 128
    assert plan(64, 22016, 4096, 1) == 64             # the SwiGLU epilogue has no split-K form
    # from 129 tokens: the cheapest of single-CTA tiles and CTA-pair tiles by estimated time (passes over the SMs)
    assert plan(512, 14336, 4096) == 1192 and plan(512, 22016, 4096, 1) == 1192 and plan(1024, 22016, 4096, 1) == 5208
    assert plan(256, 4096, 4096) == 128 and plan(512, 4096, 14336) == 128 and plan(768, 4096, 11008) == 1192
    # the 256 x 256 pair tile where it covers the output in ONE pass over the 74 SM pairs and the others need two
    assert plan(1024, 4096, 4096) == 1256 and plan(1024, 4096, 11008) == 1256 and plan(512, 8192, 8192) == 1256
    assert plan(256, 14336, 4096) == 1256
    # prefill: 256-row tiles with two accumulator sets where K is short (the drain hides behind the next tile), 512-row
    # tiles (the token tile is read by two row sets) where K is long or the passes over the SM pairs come out fewer
    assert plan(4096, 22016, 4096, 1) == 1240 and plan(4096, 4096, 4096) == 1240 and plan(2048, 22016, 4096, 1) == 5208
    assert plan(4096, 4096, 11008) == 5240 and plan(4096, 4096, 14336) == 5240 and plan(2048, 4096, 11008) == 5240
    assert plan(8192, 57344, 8192, 1) == 5240 and plan(8192, 8192, 28672) == 5224 and plan(16384, 8192, 8192) == 5240
    assert plan(0, 4096, 4096) == 0


def test_kernel_plan_is_always_a_known_variant():
    """Every shape gets a variant the dispatcher knows, and the families keep to their token ranges: decode kernel up to
    4 tokens, split-K cluster kernel up to 128, 512-row pair tiles from 1024."""
    from sparseflow_b200 import _lib
    plan = _lib.lib().sfb200_debug_plan_gemm
    single = {32, 64, 128, 192, 256}
    pair = {1192, 1208, 1224, 1240, 1256}
    pair512 = {5192, 5208, 5224, 5240}
    splitk = {3032, 3064, 3128, 4032, 4064, 4128}
    for sms in (148, 132, 64):
        for (N, K) in ((4096, 4096), (22016, 4096), (4096, 11008), (28672, 4096), (4096, 14336), (8192, 8192), (57344, 8192),
                       (8192, 28672), (1024, 1024), (512, 256), (5504, 4096), (4096, 2752)):
            for M in (1, 2, 4, 5, 16, 33, 64, 100, 128, 129, 200, 256, 500, 512, 768, 1000, 1024, 1500, 2048, 3000, 4096,
                      8192, 16384, 40000):
                for sw in (0, 1):
                    if sw and N % 32:
                        continue
                    v = plan(M, N, K, sw, sms)
                    assert v == 8 or v in single | pair | pair512 | splitk, (M, N, K, sw, sms, v)
                    if v == 8:
                        assert M <= 4
                    if v in splitk:
                        assert M <= 128 and sw == 0
                    if v in pair512:
                        assert M >= 1024
                    if M >= 4096:
                        assert v in pair | pair512
