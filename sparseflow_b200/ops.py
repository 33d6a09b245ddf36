"""Torch-facing wrappers over the C ABI.  PyTorch supplies device memory and streams only; every
computation below is a call into libsparseflow_b200.so.

Replaces, on the reference side: ``prune_24_dense_weight`` (sparseflow/nn/sparseflow_linear.py:20-35),
``torch.sparse.to_sparse_semi_structured`` (sparseflow/fused_mlp.py:22,28), the sparse matmul call
sites (sparseflow/fused_mlp.py:54,60; sparseflow/nn/sparseflow_linear.py:123) and
``fused_silu_mul`` (sparseflow/kernels/fused_silu_mul.py:33-57).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

F16, BF16 = 0, 1
TIE_HIGH, TIE_LOW = 0, 1
ACT = {"none": 0, None: 0, "relu": 1, "silu": 2, "gelu": 3}


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.bfloat16:
        return BF16
    raise ValueError(f"expected torch.float16 or torch.bfloat16, got {t.dtype}")


def _tie(tie) -> int:
    if tie in ("high", TIE_HIGH):
        return TIE_HIGH
    if tie in ("low", TIE_LOW):
        return TIE_LOW
    raise ValueError(f"tie must be 'high' or 'low', got {tie!r}")


def _need_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw getter is ~10x cheaper than building a
    torch.cuda.Stream object; it matters for kernels of a few microseconds launched eagerly)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class _NoSwitch:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


_NO_SWITCH = _NoSwitch()


def _on(device: torch.device):
    """Context that makes `device` current; free when it already is."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def device_status() -> int:
    """Synchronise and return the device status word (0 = ok); raises on a device-side failure."""
    w = C.c_int(0)
    rc = _lib.lib().sfb200_device_status(C.byref(w))
    if rc != 0:
        raise _lib.SfbError(f"sfb200_device_status (word 0x{w.value:x})", rc)
    return w.value


@dataclass
class Compressed24:
    """A 2:4-compressed weight: values [rows, K/2] + tiled metadata (uint8 view of the tile array)."""
    values: torch.Tensor
    meta: torch.Tensor
    rows: int
    K: int
    gate_up: bool = False   # rows interleaved 16 gate / 16 up

    @property
    def dtype(self) -> torch.dtype:
        return self.values.dtype

    def nbytes(self) -> int:
        return self.values.numel() * 2 + self.meta.numel()


def prune_compress_24(w: torch.Tensor, tie="high", want_values=True, want_meta=True,
                      want_ref_codes=False, want_pruned=False) -> dict:
    """2:4 magnitude prune + compress of w[rows, K]; returns the requested outputs."""
    _need_cuda(w, "w")
    if w.dim() != 2:
        raise ValueError(f"w must be 2D, got {w.dim()}D")
    rows, K = w.shape
    if K % 4 != 0:
        raise ValueError(f"in_features must be multiple of 4 for 2:4 (got {K})")
    if w.stride(1) != 1:
        w = w.contiguous()
    L = _lib.lib()
    dev = w.device
    out = {}
    with _on(dev):
        if want_values:
            out["values"] = torch.empty((rows, K // 2), dtype=w.dtype, device=dev)
        if want_meta:
            out["meta"] = torch.empty(L.sfb200_meta_bytes(rows, K), dtype=torch.uint8, device=dev)
        if want_ref_codes:
            out["ref_codes"] = torch.empty((rows, K // 4), dtype=torch.uint8, device=dev)
        if want_pruned:
            out["pruned"] = torch.empty((rows, K), dtype=w.dtype, device=dev)
        rc = L.sfb200_prune_compress_24(w.data_ptr(), rows, K, w.stride(0), _dt(w), _tie(tie),
                                        _ptr(out.get("values")), _ptr(out.get("meta")),
                                        _ptr(out.get("ref_codes")), _ptr(out.get("pruned")), _stream())
    _lib.check("sfb200_prune_compress_24", rc)
    return out


def compress_weight(w: torch.Tensor, tie="high") -> Compressed24:
    o = prune_compress_24(w, tie=tie)
    return Compressed24(o["values"], o["meta"], w.shape[0], w.shape[1])


def compress_gate_up(gate: torch.Tensor, up: torch.Tensor, tie="high") -> Compressed24:
    """Fused gate|up weight (2*I rows, 16-row interleave) for ``sparse_gemm_swiglu``."""
    _need_cuda(gate, "gate")
    _need_cuda(up, "up")
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must have the same shape and dtype")
    gate = gate.contiguous()
    up = up.contiguous()
    I, K = gate.shape
    L = _lib.lib()
    with _on(gate.device):
        values = torch.empty((2 * I, K // 2), dtype=gate.dtype, device=gate.device)
        meta = torch.empty(L.sfb200_meta_bytes(2 * I, K), dtype=torch.uint8, device=gate.device)
        rc = L.sfb200_prune_compress_gate_up(gate.data_ptr(), up.data_ptr(), I, K, K, _dt(gate),
                                             _tie(tie), values.data_ptr(), meta.data_ptr(), _stream())
    _lib.check("sfb200_prune_compress_gate_up", rc)
    return Compressed24(values, meta, 2 * I, K, gate_up=True)


def validate_24(w: torch.Tensor) -> bool:
    _need_cuda(w, "w")
    if w.stride(1) != 1:
        w = w.contiguous()
    with _on(w.device):
        flag = torch.empty(1, dtype=torch.int32, device=w.device)
        rc = _lib.lib().sfb200_validate_24(w.data_ptr(), w.shape[0], w.shape[1], w.stride(0),
                                           flag.data_ptr(), _stream())
    _lib.check("sfb200_validate_24", rc)
    return bool(flag.item())


def decompress_24(cw: Compressed24) -> torch.Tensor:
    with _on(cw.values.device):
        out = torch.empty((cw.rows, cw.K), dtype=cw.dtype, device=cw.values.device)
        rc = _lib.lib().sfb200_decompress_24(cw.values.data_ptr(), cw.meta.data_ptr(), cw.rows, cw.K,
                                             out.data_ptr(), cw.K, _stream())
    _lib.check("sfb200_decompress_24", rc)
    return out


def _kernel_ready(x: torch.Tensor) -> torch.Tensor:
    """The kernels read activations through TMA: unit inner stride, row pitch a multiple of 8 elements,
    16-byte aligned base.  A view that breaks one of these (a column slice, an odd offset) is copied,
    as the reference's call sites do unconditionally (sparseflow/nn/sparseflow_linear.py:122-124)."""
    if x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) % 8 != 0) or x.data_ptr() % 16 != 0:
        return x.contiguous()
    return x


def _check_bias(bias: torch.Tensor, x: torch.Tensor, rows: int) -> torch.Tensor:
    """The epilogue reads `rows` bias values in the GEMM's own 16-bit type."""
    if not bias.is_cuda or bias.device != x.device:
        raise ValueError(f"bias must be a CUDA tensor on {x.device}, got {bias.device}")
    if bias.dtype != x.dtype:
        raise ValueError(f"bias dtype {bias.dtype} != activation dtype {x.dtype}")
    if bias.numel() != rows:
        raise ValueError(f"bias has {bias.numel()} elements, weight has {rows} rows")
    return bias.contiguous().view(-1)


def sparse_gemm(x: torch.Tensor, cw: Compressed24, bias: Optional[torch.Tensor] = None,
                act: Optional[str] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[M, N] = act(x[M, K] . W^T + bias)."""
    _need_cuda(x, "x")
    if x.dim() != 2 or x.shape[1] != cw.K:
        raise ValueError(f"Expected last dim {cw.K}, got {tuple(x.shape)}")
    if x.dtype != cw.dtype:
        raise ValueError(f"x dtype {x.dtype} != weight dtype {cw.dtype}")
    x = _kernel_ready(x)
    if bias is not None:
        bias = _check_bias(bias, x, cw.rows)
    M = x.shape[0]
    with _on(x.device):
        if out is None:
            out = torch.empty((M, cw.rows), dtype=x.dtype, device=x.device)
        if M == 0:                      # empty batch: nothing to launch
            return out
        rc = _lib.lib().sfb200_sparse_gemm(x.data_ptr(), x.stride(0), cw.values.data_ptr(),
                                           cw.meta.data_ptr(), out.data_ptr(), out.stride(0), M, cw.rows,
                                           cw.K, _dt(x), _ptr(bias), ACT[act], _stream())
    _lib.check("sfb200_sparse_gemm", rc)
    return out


def sparse_gemm_swiglu(x: torch.Tensor, cw_gu: Compressed24, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h[M, I] = silu(x . Wg^T) * (x . Wu^T) from the fused gate|up weight."""
    _need_cuda(x, "x")
    if not cw_gu.gate_up:
        raise ValueError("weight was not built with compress_gate_up")
    if x.dim() != 2 or x.shape[1] != cw_gu.K or x.dtype != cw_gu.dtype:
        raise ValueError("shape / dtype mismatch")
    x = _kernel_ready(x)
    M, I = x.shape[0], cw_gu.rows // 2
    with _on(x.device):
        if out is None:
            out = torch.empty((M, I), dtype=x.dtype, device=x.device)
        if M == 0:
            return out
        rc = _lib.lib().sfb200_sparse_gemm_swiglu(x.data_ptr(), x.stride(0), cw_gu.values.data_ptr(),
                                                  cw_gu.meta.data_ptr(), out.data_ptr(), out.stride(0),
                                                  M, I, cw_gu.K, _dt(x), _stream())
    _lib.check("sfb200_sparse_gemm_swiglu", rc)
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """out = silu(gate) * up for 2-D (possibly strided-row) tensors."""
    _need_cuda(gate, "gate")
    if gate.shape != up.shape or gate.dtype != up.dtype or gate.dim() != 2:
        raise ValueError("fused_silu_mul expects two 2D tensors of equal shape and dtype")
    if gate.stride(1) != 1:
        gate = gate.contiguous()
    if up.stride(1) != 1:
        up = up.contiguous()
    with _on(gate.device):
        out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
        if gate.numel() == 0:
            return out
        rc = _lib.lib().sfb200_silu_mul(gate.data_ptr(), gate.stride(0), up.data_ptr(), up.stride(0),
                                        out.data_ptr(), out.stride(0), gate.shape[0], gate.shape[1],
                                        _dt(gate), _stream())
    _lib.check("sfb200_silu_mul", rc)
    return out


def force_token_tile(bn: int) -> None:
    _lib.check("sfb200_debug_force_token_tile", _lib.lib().sfb200_debug_force_token_tile(bn))
