"""Persist a compressed 2:4 weight (packed values + metadata) so that loading needs no pruning.

The reference keeps only dense copies in its modules' state (``W_original`` / ``W_dense_pruned``,
sparseflow/nn/sparseflow_linear.py:60-66) and rebuilds the sparse form at every construction.  Here
a weight can be packed into one self-describing ``uint8`` blob -- header, values, metadata; format
and validation live in the C library (``sfb200_blob_*``) -- which a ``state_dict`` or a file can
carry.  ``unpack`` returns views into the blob: no copy, no kernel launch.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .ops import BF16, F16, Compressed24

GATE_UP, TIE_LOW = 1, 2
HEADER_BYTES = 256
_DT = {torch.float16: F16, torch.bfloat16: BF16}
_TD = {F16: torch.float16, BF16: torch.bfloat16}


def blob_bytes(rows: int, K: int) -> int:
    n = _lib.lib().sfb200_blob_bytes(rows, K)
    if n == 0:
        raise ValueError(f"no blob form for a {rows} x {K} weight (K must be a multiple of 16)")
    return n


def read_header(blob: torch.Tensor) -> _lib.BlobInfo:
    """Parse and validate the header of ``blob`` (1-D uint8, any device)."""
    if blob.dtype != torch.uint8 or blob.dim() != 1:
        raise ValueError("blob must be a 1-D uint8 tensor")
    if blob.numel() < HEADER_BYTES:
        raise ValueError("blob is shorter than its header")
    head = blob[:HEADER_BYTES].cpu().contiguous()
    info = _lib.BlobInfo()
    rc = _lib.lib().sfb200_blob_read_header(head.data_ptr(), blob.numel(), C.byref(info))
    _lib.check("sfb200_blob_read_header", rc)
    return info


def pack(cw: Compressed24, tie: str = "high", checksum: bool = False) -> torch.Tensor:
    """One uint8 tensor on ``cw``'s device holding header | values | pad | metadata."""
    if cw.dtype not in _DT:
        raise ValueError(f"unsupported dtype {cw.dtype}")
    L = _lib.lib()
    total = blob_bytes(cw.rows, cw.K)
    dev = cw.values.device
    blob = torch.zeros(total, dtype=torch.uint8, device=dev)
    vb = L.sfb200_values_bytes(cw.rows, cw.K)
    mb = L.sfb200_meta_bytes(cw.rows, cw.K)
    moff = total - mb
    blob[HEADER_BYTES:HEADER_BYTES + vb].copy_(cw.values.contiguous().view(torch.uint8).reshape(-1))
    blob[moff:].copy_(cw.meta.reshape(-1)[:mb])
    csum = 0
    if checksum:
        payload = blob[HEADER_BYTES:].cpu().contiguous()
        csum = L.sfb200_blob_checksum(payload.data_ptr(), payload.numel())
    flags = (GATE_UP if cw.gate_up else 0) | (TIE_LOW if tie == "low" else 0)
    head = torch.zeros(HEADER_BYTES, dtype=torch.uint8)
    rc = L.sfb200_blob_write_header(head.data_ptr(), cw.rows, cw.K, _DT[cw.dtype], flags, csum)
    _lib.check("sfb200_blob_write_header", rc)
    blob[:HEADER_BYTES].copy_(head)
    return blob


def unpack(blob: torch.Tensor, verify_checksum: bool = False) -> Compressed24:
    """Views of the values and the metadata inside ``blob``.  Raises on a foreign, truncated or
    corrupt blob and on a layout version this library does not read."""
    info = read_header(blob)
    if blob.data_ptr() % 16 != 0:
        raise ValueError("blob storage must be 16-byte aligned")
    if verify_checksum and info.checksum != 0:
        payload = blob[HEADER_BYTES:info.total_bytes].cpu().contiguous()
        got = _lib.lib().sfb200_blob_checksum(payload.data_ptr(), payload.numel())
        if got != info.checksum:
            raise ValueError(f"blob checksum mismatch: header {info.checksum:#x}, payload {got:#x}")
    vo, vb, mo, mb = info.values_offset, info.values_bytes, info.meta_offset, info.meta_bytes
    values = blob[vo:vo + vb].view(_TD[info.dtype]).view(info.rows, info.K // 2)
    meta = blob[mo:mo + mb]
    return Compressed24(values, meta, info.rows, info.K, gate_up=bool(info.flags & GATE_UP))


def save(path: str, cw: Compressed24, tie: str = "high") -> None:
    """Write the blob (with payload checksum) to ``path``."""
    blob = pack(cw, tie=tie, checksum=True).cpu()
    with open(path, "wb") as f:
        f.write(blob.numpy().tobytes())


def load(path: str, device="cuda") -> Compressed24:
    with open(path, "rb") as f:
        raw = bytearray(f.read())
    blob = torch.frombuffer(raw, dtype=torch.uint8)
    return unpack(blob.to(device), verify_checksum=True)
