"""The reference's older convenience API (experiments/old_structure/python/sparseflow/core.py, nn.py)
and the packed-weight persistence, on the GPU against the oracle.

Tolerance: max |d| / max(|ref|, 1e-2 * rms(ref)) <= 1e-2 against the fp32-accumulated oracle."""
import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle as o
import sparseflow_b200 as sf
from sparseflow_b200 import ops, serialize
from sparseflow_b200.fused_mlp import SparseFlowFusedMLP
from tests.util import bits_of, seeded_act, seeded_weight, to_dev

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2


def test_support_probe():
    ok, msg = sf.check_sparse_support()
    assert ok and "SM10" in msg and sf.is_sparse_available()


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_prune_validate_compress_match_oracle(dt):
    R, K = 256, 512
    w = seeded_weight(R, K, dt, 11)
    oc = o.prune_24(w, dt)
    wd = to_dev(w, dt)
    assert not sf.validate_2_4(wd)
    p = sf.prune_2_4(wd)
    assert np.array_equal(bits_of(p), oc["pruned"]) and sf.validate_2_4(p)
    p3 = sf.prune_2_4(wd.reshape(4, 64, K))                      # leading dims are flattened
    assert p3.shape == (4, 64, K) and np.array_equal(bits_of(p3).reshape(R, K), oc["pruned"])
    blob = sf.compress_2_4(p)
    cw = serialize.unpack(blob)
    assert np.array_equal(bits_of(cw.values), oc["values"])
    want_meta = o.hw_meta_tiled(oc["idx0"], oc["idx1"]).view(np.uint8).reshape(-1)
    assert np.array_equal(cw.meta.cpu().numpy(), want_meta)
    with pytest.raises(ValueError, match="valid 2:4"):
        sf.compress_2_4(wd)
    with pytest.raises(NotImplementedError):
        sf.prune_2_4(wd, method="random")
    with pytest.raises(ValueError, match="Unknown pruning method"):
        sf.prune_2_4(wd, method="l1")


@pytest.mark.parametrize("epilogue,bias", [("none", False), ("relu", False), ("silu", True), ("gelu", False),
                                           ("none", True), ("relu", True)])
def test_sparse_mm_epilogues(epilogue, bias):
    dt, M, K, N = "f16", 160, 256, 384
    w = seeded_weight(N, K, dt, 2)
    x = seeded_act(M, K, dt, 9)
    oc = o.prune_24(w, dt)
    ref = o.gemm_ref(x, oc["pruned"], dt)
    bt = None
    if bias:
        b = seeded_act(1, N, dt, 77)[0]
        bt = to_dev(b, dt)
        ref = ref + o.to_f32(b, dt)[None, :]
    if epilogue == "relu":
        ref = np.maximum(ref, 0)
    elif epilogue == "silu":
        ref = ref / (1 + np.exp(-ref))
    elif epilogue == "gelu":
        ref = torch.nn.functional.gelu(torch.from_numpy(ref)).numpy()
    Bc = sf.compress_2_4(sf.prune_2_4(to_dev(w, dt)))
    y = sf.sparse_mm(to_dev(x, dt), Bc.t(), epilogue=epilogue, bias=bt)
    assert ops.device_status() == 0
    m = o.rel_err_metrics(o.to_f32(bits_of(y), dt), ref)
    assert m["floor"] <= REL_TOL, m
    with pytest.raises(ValueError, match="Unknown epilogue"):
        sf.sparse_mm(to_dev(x, dt), Bc, epilogue="tanh")


def test_sparse_linear_from_dense_and_state_dict():
    torch.manual_seed(0)
    dense = nn.Linear(512, 768, bias=True, device="cuda", dtype=torch.bfloat16)
    sl, diff = sf.SparseLinear.from_dense(dense, return_diff=True)
    assert set(diff) == {"max_error", "mean_error", "relative_error"} and diff["max_error"] > 0
    x = torch.randn(3, 40, 512, device="cuda", dtype=torch.bfloat16)
    y = sl(x)
    assert y.shape == (3, 40, 768)
    wp = bits_of(sf.prune_2_4(dense.weight.detach()))
    ref = o.gemm_ref(bits_of(x.reshape(-1, 512)), wp, "bf16") + dense.bias.detach().float().cpu().numpy()[None, :]
    m = o.rel_err_metrics(o.to_f32(bits_of(y.reshape(-1, 768)), "bf16"), ref)
    assert m["floor"] <= REL_TOL, m

    sd = sl.state_dict()
    assert set(sd) == {"weight_compressed", "bias"} and sd["weight_compressed"].dtype == torch.uint8
    fresh = sf.SparseLinear.empty(512, 768, dtype=torch.bfloat16, bias=True)
    assert not torch.equal(fresh(x), y)
    fresh.load_state_dict(sd)
    assert torch.equal(fresh(x), y)                    # same packed bits -> same kernel -> same output bits


def test_fused_mlp_rebuilt_from_packed_state_gives_identical_bits(tmp_path):
    H, I, M, dt = 512, 1408, 300, "bf16"
    mk = lambda r, k, s: ops.prune_compress_24(to_dev(seeded_weight(r, k, dt, s), dt), want_values=False,
                                               want_meta=False, want_pruned=True)["pruned"]
    g, u, d = (nn.Linear(H, I, bias=False), nn.Linear(H, I, bias=False), nn.Linear(I, H, bias=False))
    g.weight.data, u.weight.data, d.weight.data = mk(I, H, 1), mk(I, H, 2), mk(H, I, 3)
    mlp = SparseFlowFusedMLP(g, u, d, force_mode="sparse")
    x = to_dev(seeded_act(M, H, dt, 5), dt)
    want = mlp(x)
    st = mlp.compressed_state()
    assert set(st) == {"gate_up", "down"}
    torch.save(st, tmp_path / "ffn.pt")
    st2 = torch.load(tmp_path / "ffn.pt", map_location="cuda")
    again = SparseFlowFusedMLP.from_compressed_state(st2)
    assert torch.equal(again(x), want)
    assert ops.device_status() == 0
    with pytest.raises(ValueError):
        SparseFlowFusedMLP.from_compressed_state({"gate_up": st["gate_up"]})
    with pytest.raises(ValueError):
        SparseFlowFusedMLP.from_compressed_state(st, force_mode="auto")


def test_blob_payload_is_the_abi_v1_compressed_block():
    """`blob + 256` is what sparseflow_sparse_gemm takes as Bc: values, then metadata at
    sparseflow_compressed_meta_offset(N, K)."""
    from sparseflow_b200 import _lib
    L = _lib.lib()
    L.sparseflow_compressed_meta_offset.restype = __import__("ctypes").c_size_t
    N, K = 200, 192
    cw = ops.compress_weight(to_dev(seeded_weight(N, K, "f16", 4), "f16"))
    info = serialize.read_header(serialize.pack(cw))
    assert info.meta_offset - info.values_offset == L.sparseflow_compressed_meta_offset(N, K)
