"""Blob format of a compressed weight: header written and validated by the C library, payload equal
to `values | pad | metadata` as the oracle produces them.  Host-only (no GPU work)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as o
from sparseflow_b200 import _lib, serialize
from sparseflow_b200.ops import Compressed24
from tests.util import seeded_weight


def _oracle_compressed(rows, K, dt, seed=5, gate_up=False):
    w = seeded_weight(rows, K, dt, seed)
    oc = o.prune_24(w, dt)
    vals = torch.from_numpy(oc["values"].view(np.int16)).view(torch.float16 if dt == "f16" else torch.bfloat16)
    meta = torch.from_numpy(o.hw_meta_tiled(oc["idx0"], oc["idx1"]).view(np.uint8).reshape(-1).copy())
    return Compressed24(vals, meta, rows, K, gate_up=gate_up), oc


@pytest.mark.parametrize("rows,K,dt", [(128, 128, "f16"), (200, 192, "bf16"), (8, 16, "bf16"), (264, 4096, "f16")])
def test_pack_unpack_round_trip_and_payload_layout(rows, K, dt):
    L = _lib.lib()
    cw, oc = _oracle_compressed(rows, K, dt)
    assert cw.meta.numel() == L.sfb200_meta_bytes(rows, K)
    blob = serialize.pack(cw, checksum=True)
    assert blob.numel() == L.sfb200_blob_bytes(rows, K) and blob.numel() % 256 == 0
    info = serialize.read_header(blob)
    assert (info.rows, info.K, info.layout_version, info.flags) == (rows, K, 1, 0)
    assert info.values_offset == 256 and info.values_offset % 256 == 0 and info.meta_offset % 256 == 0
    raw = blob.numpy()
    vb = rows * (K // 2) * 2
    assert raw[256:256 + vb].tobytes() == oc["values"].tobytes()
    assert not raw[256 + vb:info.meta_offset].any()                     # zero padding
    assert raw[info.meta_offset:].tobytes() == cw.meta.numpy().tobytes()
    back = serialize.unpack(blob, verify_checksum=True)
    assert back.values.data_ptr() == blob.data_ptr() + 256               # views, not copies
    assert torch.equal(back.values.view(torch.int16), cw.values.view(torch.int16))
    assert torch.equal(back.meta, cw.meta) and (back.rows, back.K, back.gate_up) == (rows, K, False)


def test_flags_survive_and_are_validated():
    cw, _ = _oracle_compressed(64, 64, "bf16", gate_up=True)
    blob = serialize.pack(cw, tie="low")
    info = serialize.read_header(blob)
    assert info.flags == serialize.GATE_UP | serialize.TIE_LOW
    assert serialize.unpack(blob).gate_up
    head = (C.c_ubyte * 256)()
    L = _lib.lib()
    assert L.sfb200_blob_write_header(head, 48, 64, 1, serialize.GATE_UP, 0) == 1     # gate|up needs rows % 32 == 0
    assert L.sfb200_blob_write_header(head, 64, 64, 1, 8, 0) == 1                      # unknown flag
    assert L.sfb200_blob_write_header(head, 64, 60, 1, 0, 0) == 1                      # K % 16 != 0
    assert L.sfb200_blob_write_header(head, 64, 64, 2, 0, 0) == 1                      # dtype
    assert L.sfb200_blob_write_header(None, 64, 64, 1, 0, 0) == 1
    assert L.sfb200_blob_bytes(64, 60) == 0 and L.sfb200_blob_bytes(0, 64) == 0


def test_foreign_truncated_corrupt_and_future_blobs_are_rejected():
    cw, _ = _oracle_compressed(128, 128, "f16")
    blob = serialize.pack(cw, checksum=True)
    with pytest.raises(_lib.SfbError) as e:                 # bad magic
        bad = blob.clone(); bad[0] = ord("X"); serialize.unpack(bad)
    assert e.value.code == 1
    with pytest.raises(_lib.SfbError) as e:                 # a later layout version: caller must re-compress
        bad = blob.clone(); bad[8] = 2; serialize.unpack(bad)
    assert e.value.code == 4
    with pytest.raises(_lib.SfbError):                      # truncated payload
        serialize.unpack(blob[:blob.numel() - 256].clone())
    with pytest.raises(ValueError):                         # shorter than a header
        serialize.unpack(blob[:100].clone())
    with pytest.raises(_lib.SfbError):                      # rows edited: derived sizes no longer match
        bad = blob.clone(); bad[20] = 64; serialize.unpack(bad)
    with pytest.raises(ValueError, match="checksum"):       # payload bit flip
        bad = blob.clone(); bad[4096] ^= 1; serialize.unpack(bad, verify_checksum=True)
    with pytest.raises(ValueError):
        serialize.unpack(blob.view(torch.int8))


def test_file_round_trip(tmp_path):
    cw, _ = _oracle_compressed(136, 256, "bf16")
    p = tmp_path / "w.sfb24"
    serialize.save(str(p), cw)
    assert p.stat().st_size == serialize.blob_bytes(136, 256)
    back = serialize.load(str(p), device="cpu")
    assert torch.equal(back.values.view(torch.int16), cw.values.view(torch.int16)) and torch.equal(back.meta, cw.meta)
    raw = bytearray(p.read_bytes()); raw[1000] ^= 0x10; p.write_bytes(bytes(raw))
    with pytest.raises(ValueError, match="checksum"):
        serialize.load(str(p), device="cpu")


def test_checksum_is_fnv1a64():
    data = np.frombuffer(b"hello", dtype=np.uint8).copy()
    h = 1469598103934665603
    for b in b"hello":
        h = ((h ^ b) * 1099511628211) % (1 << 64)
    assert _lib.lib().sfb200_blob_checksum(data.ctypes.data, 5) == h
