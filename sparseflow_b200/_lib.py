"""ctypes binding of libsparseflow_b200.so (the C ABI declared in include/sparseflow_b200.h).

There is no fallback: if the library is missing the import of any compute function raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsparseflow_b200.so")

_lib = None


class FFNWeights(C.Structure):
    _fields_ = [
        ("H", C.c_int), ("I", C.c_int), ("dtype", C.c_int),
        ("gu_values", C.c_void_p), ("gu_meta", C.c_void_p),
        ("down_values", C.c_void_p), ("down_meta", C.c_void_p),
        ("down_bias", C.c_void_p),
    ]


class MatmulDesc(C.Structure):
    _fields_ = [("M", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("dtype", C.c_int32),
                ("sparsity_type", C.c_int32), ("sparsity_ratio", C.c_float), ("layout", C.c_int32)]


class GpuInfo(C.Structure):
    _fields_ = [("sm_arch", C.c_int32), ("num_sms", C.c_int32), ("shared_mem_kb", C.c_uint64)]


class BlobInfo(C.Structure):
    _fields_ = [("layout_version", C.c_uint32), ("dtype", C.c_int32), ("rows", C.c_int32), ("K", C.c_int32),
                ("flags", C.c_uint32), ("values_offset", C.c_uint64), ("values_bytes", C.c_uint64),
                ("meta_offset", C.c_uint64), ("meta_bytes", C.c_uint64), ("total_bytes", C.c_uint64),
                ("checksum", C.c_uint64)]


class SfbError(RuntimeError):
    def __init__(self, fn: str, code: int):
        msg = lib().sfb200_status_string(code).decode()
        super().__init__(f"{fn} failed: {msg} (status {code})")
        self.code = code


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m sparseflow_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    L = C.CDLL(LIB_PATH)
    vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
    L.sfb200_status_string.restype = C.c_char_p
    L.sfb200_status_string.argtypes = [i]
    L.sfb200_version.restype = i
    L.sfb200_values_bytes.restype = sz
    L.sfb200_values_bytes.argtypes = [i, i]
    L.sfb200_meta_bytes.restype = sz
    L.sfb200_meta_bytes.argtypes = [i, i]
    L.sfb200_device_status.argtypes = [C.POINTER(C.c_int)]
    L.sfb200_prune_compress_24.argtypes = [vp, i, i, i, i, i, vp, vp, vp, vp, vp]
    L.sfb200_prune_compress_gate_up.argtypes = [vp, vp, i, i, i, i, i, vp, vp, vp]
    L.sfb200_validate_24.argtypes = [vp, i, i, i, vp, vp]
    L.sfb200_decompress_24.argtypes = [vp, vp, i, i, vp, i, vp]
    L.sfb200_sparse_gemm.argtypes = [vp, i, vp, vp, vp, i, i, i, i, i, vp, i, vp]
    L.sfb200_sparse_gemm_swiglu.argtypes = [vp, i, vp, vp, vp, i, i, i, i, i, vp]
    L.sfb200_silu_mul.argtypes = [vp, i, vp, i, vp, i, i, i, i, vp]
    L.sfb200_ffn_forward.argtypes = [C.POINTER(FFNWeights), vp, i, vp, vp, i, i, vp]
    L.sfb200_ffn_forward_host.argtypes = [C.POINTER(FFNWeights), vp, vp, i, vp]
    L.sfb200_sparse_gemm_scatter.argtypes = [vp, i, vp, vp, C.POINTER(vp), i, i, i, i, i, i, i, i, vp]
    L.sfb200_tp_reduce_slots.argtypes = [vp, i, i, vp, C.POINTER(vp), i, i, i, vp, C.POINTER(vp), i, i, C.c_uint, vp]
    L.sfb200_tp_push_reduce.argtypes = [vp, i, C.POINTER(C.c_int), C.POINTER(vp), vp, i, i, C.POINTER(vp), i, i, i, vp,
                                        C.POINTER(vp), i, i, C.c_uint, i, vp]
    L.sfb200_tp_allgather.argtypes = [vp, vp, C.POINTER(vp), i, i, C.POINTER(vp), i, i, C.c_uint, vp]
    L.sfb200_tp_allreduce_switch.argtypes = [vp, vp, i, i, i, i, vp, C.POINTER(vp), i, i, C.c_uint, vp]
    L.sfb200_sparse_gemm_f32out.argtypes = [vp, i, vp, vp, vp, i, i, i, i, i, vp, i, vp]
    L.sfb200_ffn_forward_noalloc.argtypes = [C.POINTER(FFNWeights), vp, i, vp, i, i, vp]
    L.sfb200_noalloc_device_status.argtypes = [C.POINTER(C.c_int)]
    L.sfb200_debug_wait_timeout.argtypes = [C.c_uint, i, i, vp]
    L.sf_select_kernel.restype = C.c_int32
    L.sf_select_kernel.argtypes = [C.c_char_p, C.POINTER(MatmulDesc), C.POINTER(GpuInfo)]
    L.sf_select_kernel_ex.restype = C.c_int32
    L.sf_select_kernel_ex.argtypes = [C.c_char_p, C.POINTER(MatmulDesc), C.POINTER(GpuInfo), vp, vp, vp]
    L.sf_cache_size.restype = C.c_int32
    L.sf_cache_size.argtypes = [C.c_char_p]
    L.sf_cache_clear.restype = None
    L.sf_cache_clear.argtypes = [C.c_char_p]
    L.sf_note_compressed.restype = None
    L.sf_note_compressed.argtypes = [C.c_char_p, C.POINTER(MatmulDesc)]
    L.sf_record_sparse_failure.restype = None
    L.sf_record_sparse_failure.argtypes = [C.c_char_p, C.POINTER(MatmulDesc), C.POINTER(GpuInfo)]
    L.sf_compress_weight.restype = C.c_int32
    L.sf_compress_weight.argtypes = [C.POINTER(MatmulDesc), vp, C.POINTER(vp), C.POINTER(vp)]
    L.sf_compressed_cache_count.restype = C.c_int32
    L.sf_compressed_cache_bytes.restype = C.c_uint64
    L.sf_compressed_cache_clear.restype = None
    L.sf_get_counters.restype = C.c_int32
    L.sf_get_counters.argtypes = [C.c_char_p, C.POINTER(C.c_int64), C.c_int32]
    L.sfb200_debug_force_token_tile.argtypes = [i]
    L.sfb200_debug_plan_gemm.argtypes = [i, i, i, i, i]
    L.sfb200_debug_pair_tuning.argtypes = [i, i]
    L.sfb200_debug_host_pipeline.argtypes = [i, i]
    L.sfb200_debug_host_chunk_plan.argtypes = [i, i, i, C.POINTER(C.c_int)]
    L.sfb200_blob_bytes.restype = sz
    L.sfb200_blob_bytes.argtypes = [i, i]
    L.sfb200_blob_checksum.restype = C.c_uint64
    L.sfb200_blob_checksum.argtypes = [vp, sz]
    L.sfb200_blob_write_header.argtypes = [vp, i, i, i, C.c_uint, C.c_uint64]
    L.sfb200_blob_read_header.argtypes = [vp, sz, C.POINTER(BlobInfo)]
    _lib = L
    return L


def check(fn: str, code: int) -> None:
    if code != 0:
        raise SfbError(fn, code)
