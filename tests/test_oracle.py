"""The CPU oracle against the reference's own outputs (golden fixtures) and against its literal
loop form.  No GPU needed."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle as o


def test_manifest_matches_files(golden_dir):
    man = json.load(open(os.path.join(golden_dir, "manifest.json")))
    for name, digest in man["files"].items():
        with open(os.path.join(golden_dir, name), "rb") as fh:
            assert hashlib.sha256(fh.read()).hexdigest() == digest, name


def test_prune_matches_reference_script_outputs(golden_dir):
    A = np.fromfile(os.path.join(golden_dir, "A_dense.bin"), np.uint16).reshape(128, 128)
    r = o.prune_24(A, "f16")
    assert (r["pruned"] == np.fromfile(os.path.join(golden_dir, "A_pruned_dense.bin"), np.uint16).reshape(128, 128)).all()
    assert (r["values"] == np.fromfile(os.path.join(golden_dir, "dA.bin"), np.uint16).reshape(128, 64)).all()
    assert (r["ref_codes"] == np.fromfile(os.path.join(golden_dir, "dE.bin"), np.uint8).reshape(128, 32)).all()


def test_gemm_oracle_matches_reference_product(golden_dir):
    Ap = np.fromfile(os.path.join(golden_dir, "A_pruned_dense.bin"), np.uint16).reshape(128, 128)
    B = np.fromfile(os.path.join(golden_dir, "B_dense.bin"), np.float16).reshape(128, 128, order="F")
    D = np.fromfile(os.path.join(golden_dir, "D_pruned_ref.bin"), np.float32).reshape(128, 128)
    # reference: D = A_pruned @ B; oracle convention: Y = X . W^T with X = B^T, W = A_pruned
    y = o.gemm_ref(np.ascontiguousarray(B.T).view(np.uint16), Ap, "f16")
    np.testing.assert_allclose(y.T, D, rtol=1e-5, atol=1e-4)


def test_tie_and_special_value_patterns(golden_dir):
    t = np.load(os.path.join(golden_dir, "tie_patterns.npz"))
    r = o.prune_24(t["patterns"], "f16")
    assert (r["idx0"][:, 0] == t["kept"][:, 0]).all()
    assert (r["idx1"][:, 0] == t["kept"][:, 1]).all()
    low = o.prune_24(t["patterns"][80:81], "f16", tie="low")   # all-equal ranks -> (0, 1) under tie=low
    assert (low["idx0"][0, 0], low["idx1"][0, 0]) == (0, 1)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_vectorised_equals_loop_form(dtype):
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((24, 64)) * 0.02).astype(np.float32)
    bits = o.from_f32(w, dtype)
    # force many ties, zeros of both signs, NaN, inf, denormals
    bits[rng.integers(0, 24, 200), rng.integers(0, 64, 200)] = bits[0, 0]
    bits[rng.integers(0, 24, 40), rng.integers(0, 64, 40)] = 0x0000
    bits[rng.integers(0, 24, 40), rng.integers(0, 64, 40)] = 0x8000
    bits[rng.integers(0, 24, 10), rng.integers(0, 64, 10)] = 0x7E00 if dtype == "f16" else 0x7FC0
    bits[rng.integers(0, 24, 10), rng.integers(0, 64, 10)] = 0x7C00 if dtype == "f16" else 0x7F80
    bits[rng.integers(0, 24, 10), rng.integers(0, 64, 10)] = 0x0001
    a, b = o.prune_24(bits, dtype), o.prune_24_loop(bits, dtype)
    for k in a:
        assert (a[k] == b[k]).all(), k


def test_metadata_layouts_round_trip():
    rng = np.random.default_rng(3)
    bits = o.from_f32(rng.standard_normal((200, 320)).astype(np.float32), "bf16")
    r = o.prune_24(bits, "bf16")
    meta = o.hw_meta_tiled(r["idx0"], r["idx1"])
    assert meta.shape == (2, 3, 128, 4)
    nib = o.hw_meta_tiled_to_nibbles(meta, 200, 320)
    assert (nib == o.hw_nibbles(r["idx0"], r["idx1"])).all()
    assert (o.decompress(r["values"], r["idx0"], r["idx1"]) == r["pruned"]).all()
    i0, i1 = o.ref_codes_to_pairs(r["ref_codes"])
    assert (i0 == r["idx0"]).all() and (i1 == r["idx1"]).all()
    words = o.nibble_words_rowmajor(r["idx0"], r["idx1"])
    assert words.shape == (200, 10)
    assert o.enum_codes_kmajor(r["idx0"], r["idx1"]).shape == (200 * 80,)
    assert o.validate_24(r["pruned"]) and not o.validate_24(bits)


def test_metadata_word_definition_on_a_hand_case():
    # one tile; row 9 (m0=1, m1=1, m2=0), k block 2, upper half, group 3 -> lane 1+8, word 2, bits 28..31
    idx0 = np.zeros((128, 32), np.uint8)
    idx1 = np.ones((128, 32), np.uint8)
    g = (2 * 32 + 16) // 4 + 3
    idx0[9, g], idx1[9, g] = 2, 3
    meta = o.hw_meta_tiled(idx0, idx1)
    assert (meta[0, 0, 9, 2] >> 28) & 0xF == (2 | (3 << 2))
    assert (meta[0, 0, 9, 2] >> 12) & 0xF == 0x4       # row 1 (m1 = 0), same lane: default (0,1)


def test_bf16_conversion_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.3895314e38, 1e-40], np.float32)
    b = o.from_f32(x, "bf16")
    import torch
    tb = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert (b == tb).all()
    assert (o.to_f32(b, "bf16") == torch.from_numpy(x).to(torch.bfloat16).float().numpy()).all()


def test_ffn_oracle_composition():
    rng = np.random.default_rng(5)
    dt = "bf16"
    H, I, M = 64, 128, 8
    wg, wu = (o.from_f32((rng.standard_normal((I, H)) * 0.1).astype(np.float32), dt) for _ in range(2))
    wd = o.from_f32((rng.standard_normal((H, I)) * 0.1).astype(np.float32), dt)
    x = o.from_f32(rng.standard_normal((M, H)).astype(np.float32), dt)
    pg, pu, pd = (o.prune_24(w, dt)["pruned"] for w in (wg, wu, wd))
    r = o.ffn_ref(x, pg, pu, pd, dt)
    import torch
    xt, g, u, d = (torch.from_numpy(o.to_f32(a, dt)) for a in (x, pg, pu, pd))
    gt, ut = (xt @ g.T).bfloat16().float(), (xt @ u.T).bfloat16().float()
    ht = (torch.nn.functional.silu(gt) * ut).bfloat16().float()
    out = ht @ d.T
    np.testing.assert_allclose(r["out_f32"], out.numpy(), rtol=2e-2, atol=2e-2)
    src = o.interleave_gate_up_rows(I, 16)
    assert src[:16].tolist() == list(range(16)) and src[16:32].tolist() == list(range(I, I + 16))


def test_packed_code_bytes_match_reference_artifact():
    """The reference's gen_test_artifacts.py (run unmodified by make_golden.py) packs the code nibbles two
    groups per byte; same seed-0 matrix as the main fixture."""
    import os
    g = os.path.join(os.path.dirname(__file__), "golden")
    codes = np.fromfile(os.path.join(g, "dE.bin"), dtype=np.uint8).reshape(128, 32)
    want = np.fromfile(os.path.join(g, "dE_case_0.bin"), dtype=np.uint8).reshape(128, 16)
    assert np.array_equal(o.ref_codes_packed_bytes(codes), want)


def test_product_side_encoding_converters_agree_with_the_oracle():
    """sparseflow_b200.encodings (torch index arithmetic, any device) against the numpy oracle."""
    import os
    import torch
    from sparseflow_b200 import encodings as enc
    rng = np.random.default_rng(3)
    w = rng.standard_normal((200, 320)).astype(np.float16).view(np.uint16)
    r = o.prune_24(w, "f16")
    codes = torch.from_numpy(r["ref_codes"])
    nib = enc.codes_to_nibbles(codes)
    assert np.array_equal(nib.numpy(), o.hw_nibbles(r["idx0"], r["idx1"]))
    assert torch.equal(enc.nibbles_to_codes(nib), codes)
    assert np.array_equal(enc.enum_kmajor(nib).numpy().view(np.uint16), o.enum_codes_kmajor(r["idx0"], r["idx1"]))
    assert np.array_equal(enc.nibble_words(nib).numpy().view(np.uint32), o.nibble_words_rowmajor(r["idx0"], r["idx1"]))
    assert np.array_equal(enc.packed_code_bytes(codes).numpy(), o.ref_codes_packed_bytes(r["ref_codes"]))
    tiled = torch.from_numpy(o.hw_meta_tiled(r["idx0"], r["idx1"]).view(np.uint8).reshape(-1).copy())
    assert torch.equal(enc.tiled_meta_to_nibbles(tiled, 200, 320), nib)
    g = os.path.join(os.path.dirname(__file__), "golden")
    gold = torch.from_numpy(np.fromfile(os.path.join(g, "dE.bin"), dtype=np.uint8).reshape(128, 32))
    want = np.fromfile(os.path.join(g, "dE_case_0.bin"), dtype=np.uint8).reshape(128, 16)
    assert np.array_equal(enc.packed_code_bytes(gold).numpy(), want)
    import pytest
    with pytest.raises(ValueError):
        enc.codes_to_nibbles(torch.tensor([[7]], dtype=torch.uint8))
    with pytest.raises(ValueError):
        enc.nibbles_to_codes(torch.tensor([[5]], dtype=torch.uint8))      # idx0 == idx1
