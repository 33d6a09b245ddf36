"""Conversions between the metadata encodings found in the reference tree.

The prune kernel emits two of them itself: the sm_100 tile layout the GEMMs consume, and (on request)
one PAIR_TO_CODE byte per group, the format of ``dE.bin`` (experiments/prune_24_cpu.py:12-28).  The
reference's experiment harnesses use three more, all functions of the kept index pair per group; they
are offered here so that data can be exchanged with those harnesses:

* ``enum_kmajor``      enum 0..5 in uint16, stored K-major ``E[g * rows + row]``
                       (experiments/sparse_harness/data/generate_test_data.py:25-38)
* ``nibble_words``     ``idx0 | idx1 << 2`` per group, eight groups per 32-bit word, row-major [rows, K/32]
                       (experiments/wmma_sparse_24/compress_24.py:31-44)
* ``packed_code_bytes``  PAIR_TO_CODE nibbles, two groups per byte, even group low: [rows, K/8]
                       (experiments/gen_test_artifacts.py:20-53)

Integer index arithmetic on torch tensors of any device; nothing here is on the FFN hot path.
"""
from __future__ import annotations

import torch

PAIR_TO_CODE = {(0, 1): 9, (0, 2): 4, (0, 3): 8, (1, 2): 12, (1, 3): 14, (2, 3): 13}
PAIR_TO_ENUM = {(0, 1): 0, (0, 2): 1, (0, 3): 2, (1, 2): 3, (1, 3): 4, (2, 3): 5}


def _table_by_nibble(pairs: dict, dev) -> torch.Tensor:
    """16-entry table: hardware nibble (idx0 | idx1 << 2) -> the value `pairs` gives that index pair; 255 = invalid."""
    t = torch.full((16,), 255, dtype=torch.uint8)
    for (a, b), c in pairs.items():
        t[a | (b << 2)] = c
    return t.to(dev)


def _nibble_by_code(dev) -> torch.Tensor:
    """16-entry table: PAIR_TO_CODE value -> hardware nibble; 255 = not a code."""
    t = torch.full((16,), 255, dtype=torch.uint8)
    for (a, b), c in PAIR_TO_CODE.items():
        t[c] = a | (b << 2)
    return t.to(dev)


def codes_to_nibbles(ref_codes: torch.Tensor) -> torch.Tensor:
    """PAIR_TO_CODE bytes [rows, K/4] -> hardware nibbles ``idx0 | idx1 << 2`` (uint8, same shape)."""
    if ref_codes.dtype != torch.uint8:
        raise ValueError("ref_codes must be uint8")
    lut = _nibble_by_code(ref_codes.device)
    nib = lut[ref_codes.long().clamp_(max=15)]
    if bool((nib == 255).any()) or bool((ref_codes > 15).any()):
        raise ValueError("not a PAIR_TO_CODE byte")
    return nib


def nibbles_to_codes(nib: torch.Tensor) -> torch.Tensor:
    lut = _table_by_nibble(PAIR_TO_CODE, nib.device)
    out = lut[nib.long()]
    if bool((out == 255).any()):
        raise ValueError("nibble does not name two distinct positions in increasing order")
    return out


def enum_kmajor(nib: torch.Tensor) -> torch.Tensor:
    """Nibbles [rows, G] -> enum 0..5 as int16 (uint16 bit patterns), flattened K-major: E[g * rows + row]."""
    lut = _table_by_nibble(PAIR_TO_ENUM, nib.device)
    e = lut[nib.long()]
    if bool((e == 255).any()):
        raise ValueError("invalid nibble")
    return e.t().contiguous().reshape(-1).to(torch.int16)


def nibble_words(nib: torch.Tensor) -> torch.Tensor:
    """Nibbles [rows, G] (G % 8 == 0) -> int32 words [rows, G/8], group j of a word at bits 4j."""
    rows, G = nib.shape
    if G % 8 != 0:
        raise ValueError("needs a multiple of 8 groups per row (K % 32 == 0)")
    n = nib.to(torch.int64).reshape(rows, G // 8, 8)
    sh = 4 * torch.arange(8, device=nib.device, dtype=torch.int64)
    w = (n << sh).sum(-1)
    return torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)     # uint32 bit pattern in an int32 tensor


def packed_code_bytes(ref_codes: torch.Tensor) -> torch.Tensor:
    """PAIR_TO_CODE bytes [rows, G] (G even) -> [rows, G/2] uint8, even group in the low nibble."""
    if ref_codes.shape[1] % 2 != 0:
        raise ValueError("needs an even number of groups per row (K % 8 == 0)")
    c = ref_codes.to(torch.int32)
    return ((c[:, 0::2] & 0xF) | ((c[:, 1::2] & 0xF) << 4)).to(torch.uint8)


def tiled_meta_to_nibbles(meta: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """The sm_100 tile layout (uint8 view, as ``Compressed24.meta``) -> row-major nibbles [rows, K/4].
    Tile = 128 rows x 128 K, 128 lanes x 4 words; row m = m0 + 8*m1 + 16*m2, lane = m0 + 8*kh + 16*m2,
    word = kb, bits [16*m1, +16) = four nibbles of the 16-wide half kh of 32-wide block kb."""
    RT, KT = (rows + 127) // 128, (K + 127) // 128
    w = meta.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    w = w.reshape(RT, KT, 8, 2, 8, 4)                          # [rt, kt, m2, kh, m0, kb]
    halves = torch.stack([w & 0xFFFF, w >> 16], 0)             # [m1, rt, kt, m2, kh, m0, kb]
    sh = 4 * torch.arange(4, device=meta.device, dtype=torch.int64)
    nib = (halves.unsqueeze(-1) >> sh) & 0xF                   # [m1, rt, kt, m2, kh, m0, kb, j]
    nib = nib.permute(1, 3, 0, 5, 2, 6, 4, 7)                  # [rt, m2, m1, m0, kt, kb, kh, j]
    nib = nib.reshape(RT * 128, KT * 32).to(torch.uint8)
    return nib[:rows, :K // 4].contiguous()
