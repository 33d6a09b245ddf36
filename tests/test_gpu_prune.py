"""Prune + compress on the GPU through the C ABI, bit-exact against the oracle and against the
reference script's own outputs."""
import os

import numpy as np
import pytest
import torch

import oracle as o
from sparseflow_b200 import ops
from sparseflow_b200.nn.sparseflow_linear import prune_24_dense_weight
from tests.util import bits_of, seeded_weight, to_dev

pytestmark = pytest.mark.gpu


def _check(bits, dtype, tie="high"):
    r = ops.prune_compress_24(to_dev(bits, dtype), tie=tie, want_ref_codes=True, want_pruned=True)
    oc = o.prune_24(bits, dtype, tie)
    assert (bits_of(r["values"]) == oc["values"]).all()
    assert (r["ref_codes"].cpu().numpy() == oc["ref_codes"]).all()
    assert (bits_of(r["pruned"]) == oc["pruned"]).all()
    meta = r["meta"].cpu().numpy().view(np.uint32)
    assert (meta == o.hw_meta_tiled(oc["idx0"], oc["idx1"]).reshape(-1)).all()
    assert ops.device_status() == 0
    return r, oc


def test_reference_fixture_bit_exact(golden_dir):
    A = np.fromfile(os.path.join(golden_dir, "A_dense.bin"), np.uint16).reshape(128, 128)
    r = ops.prune_compress_24(to_dev(A, "f16"), want_ref_codes=True, want_pruned=True)
    assert (bits_of(r["values"]) == np.fromfile(os.path.join(golden_dir, "dA.bin"), np.uint16).reshape(128, 64)).all()
    assert (r["ref_codes"].cpu().numpy() == np.fromfile(os.path.join(golden_dir, "dE.bin"), np.uint8).reshape(128, 32)).all()
    assert (bits_of(r["pruned"]) == np.fromfile(os.path.join(golden_dir, "A_pruned_dense.bin"), np.uint16).reshape(128, 128)).all()


def test_tie_and_special_patterns(golden_dir):
    t = np.load(os.path.join(golden_dir, "tie_patterns.npz"))
    pats = np.tile(t["patterns"], (1, 4))            # K = 16 so the vector kernel runs too
    r = ops.prune_compress_24(to_dev(pats, "f16"), want_ref_codes=True)
    i0, i1 = o.ref_codes_to_pairs(r["ref_codes"].cpu().numpy())
    assert (i0[:, 0] == t["kept"][:, 0]).all() and (i1[:, 0] == t["kept"][:, 1]).all()
    assert (i0 == i0[:, :1]).all()


@pytest.mark.parametrize("R,K,dtype,tie", [
    (128, 128, "f16", "high"), (256, 512, "bf16", "high"), (200, 1024, "f16", "low"),
    (48, 192, "bf16", "high"), (1, 64, "bf16", "low"), (130, 16, "f16", "high"),
    (1000, 4096, "bf16", "high"),
])
def test_random_with_specials(R, K, dtype, tie):
    rng = np.random.default_rng(R * 7 + K)
    bits = o.from_f32((rng.standard_normal((R, K)) * 0.02).astype(np.float32), dtype)
    n = max(4, R * K // 50)
    bits[rng.integers(0, R, n), rng.integers(0, K, n)] = bits[0, 0]                  # ties
    bits[rng.integers(0, R, n), rng.integers(0, K, n)] = 0x8000                       # -0
    bits[rng.integers(0, R, n), rng.integers(0, K, n)] = 0x0000
    bits[rng.integers(0, R, 8), rng.integers(0, K, 8)] = 0x7E00 if dtype == "f16" else 0x7FC0   # NaN
    bits[rng.integers(0, R, 8), rng.integers(0, K, 8)] = 0xFC00 if dtype == "f16" else 0xFF80   # -inf
    bits[rng.integers(0, R, 8), rng.integers(0, K, 8)] = 0x0001                       # denormal
    _check(bits, dtype, tie)


def test_config1_weight_and_ffn_weights_full_size():
    """Config-1 W (4096 x 4096 fp16) and a Llama-7B projection (11008 x 4096 bf16), N(0, 0.02)."""
    _check(seeded_weight(4096, 4096, "f16", 1), "f16")
    r, oc = _check(seeded_weight(11008, 4096, "bf16", 2), "bf16")
    # idempotence at full size: pruning the pruned matrix changes nothing
    r2 = ops.prune_compress_24(r["pruned"], want_pruned=True)
    assert torch.equal(r2["pruned"], r["pruned"]) and torch.equal(r2["values"], r["values"])
    assert torch.equal(r2["meta"], r["meta"])


def test_generic_path_k_multiple_of_4_only():
    rng = np.random.default_rng(11)
    bits = o.from_f32(rng.standard_normal((37, 20)).astype(np.float32), "bf16")
    r = ops.prune_compress_24(to_dev(bits, "bf16"), want_meta=False, want_ref_codes=True, want_pruned=True)
    oc = o.prune_24(bits, "bf16")
    assert (bits_of(r["values"]) == oc["values"]).all()
    assert (r["ref_codes"].cpu().numpy() == oc["ref_codes"]).all()
    assert (bits_of(r["pruned"]) == oc["pruned"]).all()


def test_gate_up_interleave():
    I, H, dt = 352, 256, "bf16"
    wg, wu = seeded_weight(I, H, dt, 5), seeded_weight(I, H, dt, 6)
    cw = ops.compress_gate_up(to_dev(wg, dt), to_dev(wu, dt))
    pg, pu = o.prune_24(wg, dt), o.prune_24(wu, dt)
    src = o.interleave_gate_up_rows(I, 16)
    assert (bits_of(cw.values) == np.concatenate([pg["values"], pu["values"]], 0)[src]).all()
    i0 = np.concatenate([pg["idx0"], pu["idx0"]], 0)[src]
    i1 = np.concatenate([pg["idx1"], pu["idx1"]], 0)[src]
    assert (cw.meta.cpu().numpy().view(np.uint32) == o.hw_meta_tiled(i0, i1).reshape(-1)).all()


def test_validate_and_decompress_round_trip():
    dt = "f16"
    w = seeded_weight(300, 448, dt, 9)
    wd = to_dev(w, dt)
    assert not ops.validate_24(wd)
    cw = ops.compress_weight(wd)
    dense = ops.decompress_24(cw)
    assert (bits_of(dense) == o.prune_24(w, dt)["pruned"]).all()
    assert ops.validate_24(dense)


def test_prune_24_dense_weight_api():
    w = seeded_weight(64, 128, "f16", 3)
    p = prune_24_dense_weight(to_dev(w, "f16"))
    assert (bits_of(p) == o.prune_24(w, "f16")["pruned"]).all()
    with pytest.raises(ValueError):
        prune_24_dense_weight(torch.zeros(4, 8, dtype=torch.float16))             # not CUDA
    with pytest.raises(ValueError):
        prune_24_dense_weight(torch.zeros(4, 6, dtype=torch.float16, device="cuda"))  # K % 4
    with pytest.raises(ValueError):
        prune_24_dense_weight(torch.zeros(4, 8, dtype=torch.float32, device="cuda"))
    with pytest.raises(ValueError):
        prune_24_dense_weight(torch.zeros(8, dtype=torch.float16, device="cuda"))


def test_full_size_tiled_metadata_equals_code_bytes_llama_gate():
    """Size-independent consistency at the benchmark's weight size (11008 x 4096): the sm_100 tile layout,
    un-tiled on the device, names the same index pairs as the per-group code bytes of the same launch, and
    the three harness encodings round-trip through them."""
    from sparseflow_b200 import encodings as enc
    g = torch.Generator(device="cuda").manual_seed(11)
    w = (torch.randn(11008, 4096, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    out = ops.prune_compress_24(w, want_ref_codes=True)
    nib = enc.tiled_meta_to_nibbles(out["meta"], 11008, 4096)
    assert torch.equal(nib, enc.codes_to_nibbles(out["ref_codes"]))
    assert torch.equal(enc.nibbles_to_codes(nib), out["ref_codes"])
    words = enc.nibble_words(nib)
    assert words.shape == (11008, 128)
    back = (words.to(torch.int64).unsqueeze(-1) >> (4 * torch.arange(8, device="cuda"))) & 0xF
    assert torch.equal(back.reshape(11008, 1024).to(torch.uint8), nib)
    assert enc.enum_kmajor(nib).shape == (11008 * 1024,) and int(enc.enum_kmajor(nib).max()) == 5
    assert enc.packed_code_bytes(out["ref_codes"]).shape == (11008, 512)
