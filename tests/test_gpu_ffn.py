"""Gated FFN and the nn modules on the GPU against the oracle."""
import ctypes as C

import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle as o
from sparseflow_b200 import _lib, ops
from sparseflow_b200.fused_mlp import SparseFlowFusedMLP
from sparseflow_b200.kernels.fused_silu_mul import fused_silu_mul
from sparseflow_b200.nn.policy import SparseFlowPolicy
from sparseflow_b200.nn.sparseflow_linear import SparseFlowLinear, make_sparseflow_linear
from sparseflow_b200.nn.sparseflow_mlp import SparseFlowMLP, make_sparseflow_mlp
from tests.util import bits_of, seeded_act, seeded_weight, to_dev

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2


@pytest.fixture(autouse=True)
def _auto_tile():
    ops.force_token_tile(0)
    yield
    ops.force_token_tile(0)


def _weights(H, I, dt):
    wg, wu, wd = seeded_weight(I, H, dt, 1), seeded_weight(I, H, dt, 2), seeded_weight(H, I, dt, 3)
    return wg, wu, wd, [o.prune_24(w, dt)["pruned"] for w in (wg, wu, wd)]


@pytest.mark.parametrize("bn", [0, 64, 192, 1256, 1240, 1224, 1208, 1192, 2192, 2208, 2224, 2240, 5240, 5224, 5208, 5192])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_swiglu_epilogue(bn, dt):
    H, I, M = 512, 352, 300
    wg, wu, _, (pg, pu, _) = _weights(H, I, dt)
    x = seeded_act(M, H, dt, 1234)
    cw = ops.compress_gate_up(to_dev(wg, dt), to_dev(wu, dt))
    ops.force_token_tile(bn)
    h = ops.sparse_gemm_swiglu(to_dev(x, dt), cw)
    assert ops.device_status() == 0
    ref = o.silu_mul_ref(o.gemm_ref(x, pg, dt), o.gemm_ref(x, pu, dt))
    assert o.rel_err_metrics(o.to_f32(bits_of(h), dt), ref)["floor"] <= REL_TOL


@pytest.mark.parametrize("M", [1, 8, 13, 32])
def test_swiglu_small_m_kernel(M):
    dt, H, I = "bf16", 1024, 2752
    wg, wu, _, (pg, pu, _) = _weights(H, I, dt)
    x = seeded_act(M, H, dt, 4321)
    cw = ops.compress_gate_up(to_dev(wg, dt), to_dev(wu, dt))
    ops.force_token_tile(8)
    h = ops.sparse_gemm_swiglu(to_dev(x, dt), cw)
    assert ops.device_status() == 0
    ref = o.silu_mul_ref(o.gemm_ref(x, pg, dt), o.gemm_ref(x, pu, dt))
    assert o.rel_err_metrics(o.to_f32(bits_of(h), dt), ref)["floor"] <= REL_TOL


@pytest.mark.parametrize("H,I,M", [(512, 1408, 100), (4096, 11008, 512)])
def test_ffn_forward_c_abi_device_and_host(H, I, M):
    """sfb200_ffn_forward / sfb200_ffn_forward_host against the oracle; (4096, 11008, 512) is the
    Llama-7B shape at its smallest token count."""
    dt = "bf16"
    wg, wu, wd, (pg, pu, pd) = _weights(H, I, dt)
    x = seeded_act(M, H, dt, 1235)
    gu = ops.compress_gate_up(to_dev(wg, dt), to_dev(wu, dt))
    dn = ops.compress_weight(to_dev(wd, dt))
    W = _lib.FFNWeights(H, I, ops.BF16, gu.values.data_ptr(), gu.meta.data_ptr(), dn.values.data_ptr(),
                        dn.meta.data_ptr(), None)
    xd = to_dev(x, dt)
    hidden = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    L = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    assert L.sfb200_ffn_forward(C.byref(W), xd.data_ptr(), H, hidden.data_ptr(), out.data_ptr(), H, M, st) == 0
    assert ops.device_status() == 0
    fused = o.ffn_ref(x, pg, pu, pd, dt, round_gate_up=False)     # the dataflow the kernels implement
    unfused = o.ffn_ref(x, pg, pu, pd, dt, round_gate_up=True)    # the reference's unfused dataflow
    y = o.to_f32(bits_of(out), dt)
    mh = o.rel_err_metrics(o.to_f32(bits_of(hidden), dt), o.to_f32(fused["hidden"], dt))
    md = o.rel_err_metrics(y, o.gemm_ref(bits_of(hidden), pd, dt))     # down GEMM alone, same input bits
    mf = o.rel_err_metrics(y, fused["out_f32"])
    mu = o.rel_err_metrics(y, unfused["out_f32"])
    assert mh["floor"] <= REL_TOL, mh
    assert md["floor"] <= REL_TOL, md
    assert mf["chain"] <= REL_TOL and mf["norm"] <= REL_TOL, mf
    # informative: the reference's unfused dataflow also rounds gate and up to the 16-bit type;
    # those extra roundings (and their 1-ulp flips) show as noise of a few percent of the rms
    assert mu["chain"] <= 3 * REL_TOL and mu["norm"] <= REL_TOL, mu
    # host-buffer entry point: same bits as the device path
    xh = torch.from_numpy(x.view(np.int16)).pin_memory()
    oh = torch.empty(M, H, dtype=torch.int16).pin_memory()
    assert L.sfb200_ffn_forward_host(C.byref(W), xh.data_ptr(), oh.data_ptr(), M, st) == 0
    assert (oh.numpy().view(np.uint16) == bits_of(out)).all()


def test_fused_silu_mul_kernel():
    dt = "f16"
    g, u = seeded_act(300, 1000, dt, 1), seeded_act(300, 1000, dt, 2)
    gu = torch.cat([to_dev(g, dt), to_dev(u, dt)], 1)                  # strided rows, like chunk(2)
    out = fused_silu_mul(*gu.chunk(2, dim=-1))
    ref = o.silu_mul_ref(o.to_f32(g, dt), o.to_f32(u, dt))
    assert o.rel_err_metrics(o.to_f32(bits_of(out), dt), ref)["floor"] <= 2e-3
    odd = fused_silu_mul(to_dev(g, dt)[:, :999], to_dev(u, dt)[:, :999])  # scalar path
    assert o.rel_err_metrics(o.to_f32(bits_of(odd), dt), ref[:, :999])["floor"] <= 2e-3


def _linears(H, I, dt, prune):
    tdt = torch.bfloat16 if dt == "bf16" else torch.float16
    wg, wu, wd, pr = _weights(H, I, dt)
    src = pr if prune else (wg, wu, wd)
    mods = []
    for w, (o_f, i_f) in zip(src, [(I, H), (I, H), (H, I)]):
        lin = nn.Linear(i_f, o_f, bias=False, device="cuda", dtype=tdt)
        lin.weight.data.copy_(to_dev(w, dt))
        mods.append(lin)
    return mods, pr


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_fused_mlp_module_force_modes(dt):
    H, I, M = 512, 1408, 320
    (gp, up, dp), (pg, pu, pd) = _linears(H, I, dt, prune=True)
    x = seeded_act(M, H, dt, 99)
    ref = o.ffn_ref(x, pg, pu, pd, dt, round_gate_up=False)["out_f32"]
    xs = to_dev(x, dt).view(4, 80, H)
    for mode in ("sparse", "dense", "auto"):
        mlp = SparseFlowFusedMLP(gp, up, dp, force_mode=mode)
        assert mlp._gate_up_sparse is not None and mlp._down_sparse is not None
        y = mlp(xs)
        assert y.shape == (4, 80, H)
        m = o.rel_err_metrics(o.to_f32(bits_of(y), dt).reshape(M, H), ref)
        # the dense branch (library GEMM) stores gate and up in the 16-bit type before SiLU.mul:
        # those roundings show as noise of up to a few percent of the rms on cancelling outputs.
        # (The reference's own smoke bound is 0.5 absolute, tools/smoke_dispatch.py:83.)
        tol = REL_TOL if mode == "sparse" else 3 * REL_TOL
        assert m["chain"] <= tol and m["norm"] <= REL_TOL, (mode, m)
    assert ops.device_status() == 0
    # a weight that is not 2:4 leaves the module dense, as upstream
    (gd, ud, dd), _ = _linears(H, I, dt, prune=False)
    dense_mlp = SparseFlowFusedMLP(gd, ud, dd)
    assert dense_mlp._gate_up_sparse is None and dense_mlp._down_sparse is None
    dense_mlp(xs)
    with pytest.raises(RuntimeError):
        SparseFlowFusedMLP(gd, ud, dd, force_mode="sparse")(xs)


def test_sparseflow_linear_module():
    dt = "bf16"
    w = seeded_weight(1024, 512, dt, 4)
    b = seeded_act(1, 1024, dt, 8)[0]
    pol = SparseFlowPolicy(min_M_default=64)
    lin = SparseFlowLinear(to_dev(w, dt), to_dev(b, dt), policy=pol, op_name="default", dense_uses_pruned=True)
    x = seeded_act(200, 512, dt, 5)
    y = lin(to_dev(x, dt).view(2, 100, 512))
    assert lin._sparse_count == 1 and y.shape == (2, 100, 1024)
    ref = o.gemm_ref(x, o.prune_24(w, dt)["pruned"], dt) + o.to_f32(b, dt)[None]
    assert o.rel_err_metrics(o.to_f32(bits_of(y), dt).reshape(200, 1024), ref)["floor"] <= REL_TOL
    y_small = lin(to_dev(x, dt)[:8])                         # below min_M: dense branch, pruned weight
    assert lin._dense_count == 1
    assert o.rel_err_metrics(o.to_f32(bits_of(y_small), dt), ref[:8])["floor"] <= REL_TOL
    assert (bits_of(lin.W_dense_pruned) == o.prune_24(w, dt)["pruned"]).all()
    sd = lin.state_dict()
    assert set(sd) == {"W_original", "W_dense_pruned", "bias"}
    m = make_sparseflow_linear(nn.Linear(512, 64, device="cuda", dtype=torch.float16), name="q_proj")
    assert m.op_name == "q_proj"
    with pytest.raises(ValueError):
        lin(torch.zeros(2, 100, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(TypeError):
        make_sparseflow_linear(nn.ReLU())


def test_sparseflow_mlp_module():
    dt = "f16"
    H, I = 512, 704
    wg, wu, wd, (pg, pu, pd) = _weights(H, I, dt)
    x = seeded_act(96, H, dt, 6)
    xs = to_dev(x, dt).view(2, 48, H)
    mlp = SparseFlowMLP(H, I, to_dev(wg, dt), to_dev(wu, dt), to_dev(wd, dt))
    y = mlp(xs)
    # reference function: sparse gate/up on pruned weights, DENSE down on the unpruned weight
    hid = o.from_f32(o.silu_mul_ref(o.gemm_ref(x, pg, dt), o.gemm_ref(x, pu, dt)), dt)
    ref = o.to_f32(hid, dt) @ o.to_f32(wd, dt).T
    assert o.rel_err_metrics(o.to_f32(bits_of(y), dt).reshape(96, H), ref)["chain"] <= REL_TOL
    mlp_s = SparseFlowMLP(H, I, to_dev(wg, dt), to_dev(wu, dt), to_dev(wd, dt), down_mode="sparse")
    ref_s = o.ffn_ref(x, pg, pu, pd, dt, round_gate_up=False)["out_f32"]
    assert o.rel_err_metrics(o.to_f32(bits_of(mlp_s(xs)), dt).reshape(96, H), ref_s)["chain"] <= REL_TOL
    # biases on gate/up take the unfused path
    bg, bu = seeded_act(1, I, dt, 11)[0], seeded_act(1, I, dt, 12)[0]
    mlp_b = SparseFlowMLP(H, I, to_dev(wg, dt), to_dev(wu, dt), to_dev(wd, dt), to_dev(bg, dt), to_dev(bu, dt),
                          down_mode="sparse")
    g = o.to_f32(o.from_f32(o.gemm_ref(x, pg, dt) + o.to_f32(bg, dt)[None], dt), dt)
    u = o.to_f32(o.from_f32(o.gemm_ref(x, pu, dt) + o.to_f32(bu, dt)[None], dt), dt)
    ref_b = o.gemm_ref(o.from_f32(o.silu_mul_ref(g, u), dt), pd, dt)
    assert o.rel_err_metrics(o.to_f32(bits_of(mlp_b(xs)), dt).reshape(96, H), ref_b)["chain"] <= REL_TOL

    class Gated(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = nn.Linear(H, I, bias=False, device="cuda", dtype=torch.float16)
            self.up_proj = nn.Linear(H, I, bias=False, device="cuda", dtype=torch.float16)
            self.down_proj = nn.Linear(I, H, bias=False, device="cuda", dtype=torch.float16)
    assert isinstance(make_sparseflow_mlp(Gated()), SparseFlowMLP)
    assert ops.device_status() == 0


def test_model_surgery_replaces_every_mlp():
    """A two-layer Llama-shaped stack with random weights (no checkpoints exist offline)."""
    from sparseflow_b200.nn.surgery import replace_llama_mlp_module
    H, I = 512, 1408

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = nn.Linear(H, I, bias=False, device="cuda", dtype=torch.bfloat16)
            self.up_proj = nn.Linear(H, I, bias=False, device="cuda", dtype=torch.bfloat16)
            self.down_proj = nn.Linear(I, H, bias=False, device="cuda", dtype=torch.bfloat16)

        def forward(self, x):
            return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = MLP()

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Layer(), Layer()])

    torch.manual_seed(0)
    m = Model()
    for layer in m.layers:                      # make the weights 2:4 so dense and sparse agree
        for lin in (layer.mlp.gate_proj, layer.mlp.up_proj, layer.mlp.down_proj):
            lin.weight.data = ops.prune_compress_24(lin.weight.data, want_values=False, want_meta=False,
                                                    want_pruned=True)["pruned"]
    x = torch.randn(2, 64, H, device="cuda", dtype=torch.bfloat16)
    want = [layer.mlp(x) for layer in m.layers]
    assert replace_llama_mlp_module(m, SparseFlowPolicy(), down_mode="sparse") == 2
    for layer, w in zip(m.layers, want):
        assert isinstance(layer.mlp, SparseFlowMLP)
        got = layer.mlp(x)
        err = (got.float() - w.float()).abs().max().item()
        assert err <= 3e-2 * w.float().pow(2).mean().sqrt().item() + 2.0 ** -8 * w.float().abs().max().item()
    assert ops.device_status() == 0


def test_empty_batch_returns_empty_outputs():
    """Zero tokens: every entry of the Python surface returns an empty tensor of the right shape and
    launches nothing (the C ABI itself rejects M <= 0 as an invalid argument)."""
    dt, H, I = "bf16", 256, 512
    (gp, up, dp), _ = _linears(H, I, dt, prune=True)
    x0 = torch.zeros(0, H, device="cuda", dtype=torch.bfloat16)
    cw = ops.compress_weight(gp.weight.data)
    assert ops.sparse_gemm(x0, cw).shape == (0, I)
    assert ops.sparse_gemm_swiglu(x0, ops.compress_gate_up(gp.weight.data, up.weight.data)).shape == (0, I)
    assert ops.silu_mul(torch.zeros(0, I, device="cuda", dtype=torch.bfloat16),
                        torch.zeros(0, I, device="cuda", dtype=torch.bfloat16)).shape == (0, I)
    for mode in ("sparse", "dense", "auto"):
        assert SparseFlowFusedMLP(gp, up, dp, force_mode=mode)(x0).shape == (0, H)
        assert SparseFlowFusedMLP(gp, up, dp, force_mode=mode)(x0.view(0, 7, H)[:0]).shape[-1] == H
    lin = SparseFlowLinear(gp.weight.data, None, policy=SparseFlowPolicy(min_M_default=1), dense_uses_pruned=True)
    assert lin(x0).shape == (0, I)
    from sparseflow_b200 import _lib
    rc = _lib.lib().sfb200_sparse_gemm(x0.data_ptr(), H, cw.values.data_ptr(), cw.meta.data_ptr(), x0.data_ptr(), I,
                                       0, I, H, 1, None, 0, None)
    assert rc == 1
    assert ops.device_status() == 0


def test_linear_level_surgery_mlp_and_attention():
    """replace_llama_mlp / replace_llama_full (tools/llama_surgery.py, tools/llama_surgery_full.py): every projection of
    every layer becomes a SparseFlowLinear carrying its op name; outputs match the dense layers on the pruned weights."""
    from sparseflow_b200.nn.replace_llama import replace_llama_attention, replace_llama_full, replace_llama_mlp
    H, I = 256, 512

    def lin(i, o):
        l = nn.Linear(i, o, bias=False, device="cuda", dtype=torch.bfloat16)
        l.weight.data = ops.prune_compress_24(l.weight.data, want_values=False, want_meta=False, want_pruned=True)["pruned"]
        return l

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = nn.Module()
            self.mlp.gate_proj, self.mlp.up_proj, self.mlp.down_proj = lin(H, I), lin(H, I), lin(I, H)
            self.self_attn = nn.Module()
            for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
                setattr(self.self_attn, n, lin(H, H))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.model = nn.Module()
            self.model.layers = nn.ModuleList([Block(), Block()])

    torch.manual_seed(1)
    m = Model()
    x = torch.randn(96, H, device="cuda", dtype=torch.bfloat16)
    want = {(li, n): getattr(b.self_attn, n)(x) for li, b in enumerate(m.model.layers) for n in ("q_proj", "o_proj")}
    want_g = m.model.layers[1].mlp.gate_proj(x)
    pol = SparseFlowPolicy(min_M_gate_up=1, min_M_down=1, min_M_qkv=1, min_M_o=1)
    assert replace_llama_mlp(m, pol, verbose=False) == 6
    assert replace_llama_full(m, pol, verbose=False) == 8            # MLP already swapped: only the attention is left
    assert replace_llama_attention(m, pol, verbose=False) == 0
    b1 = m.model.layers[1]
    assert isinstance(b1.mlp.gate_proj, SparseFlowLinear) and b1.mlp.gate_proj.op_name == "gate_proj"
    assert b1.self_attn.k_proj.op_name == "k_proj"
    for (li, n), ref in want.items():
        got = getattr(m.model.layers[li].self_attn, n)(x)
        assert (got.float() - ref.float()).abs().max() <= 1e-2 * ref.float().abs().max()
    got_g = b1.mlp.gate_proj(x)
    assert b1.mlp.gate_proj._sparse_count == 1
    assert (got_g.float() - want_g.float()).abs().max() <= 1e-2 * want_g.float().abs().max()
    assert ops.device_status() == 0


def test_random_ffn_shapes_through_the_c_abi():
    """Seeded random (tokens, hidden, intermediate) triples through sfb200_ffn_forward (whatever kernels the
    dispatcher picks for each GEMM) against fp32 math on the decompressed weights with the same rounding points
    (hidden stored in the 16-bit type)."""
    import ctypes as C
    from sparseflow_b200 import _lib
    rng = np.random.default_rng(7)
    L = _lib.lib()
    for case in range(24):
        M = int(rng.choice([1, 3, 8, 20, 64, 100, 130, 300, 512, 1025, 1400]))
        H = int(rng.choice([64, 256, 320, 1024, 2048]))
        I = int(rng.choice([64, 192, 1408, 2752, 4096]))      # I % 64 == 0: it is the K of the down GEMM
        g = torch.Generator(device="cuda").manual_seed(100 + case)
        rnd = lambda *s, sigma: (torch.randn(*s, generator=g, device="cuda") * sigma).to(torch.bfloat16)
        wg, wu, wd, x = rnd(I, H, sigma=0.05), rnd(I, H, sigma=0.05), rnd(H, I, sigma=0.05), rnd(M, H, sigma=1.0)
        gu, dn = ops.compress_gate_up(wg, wu), ops.compress_weight(wd)
        W = _lib.FFNWeights(H, I, ops.BF16, gu.values.data_ptr(), gu.meta.data_ptr(), dn.values.data_ptr(),
                            dn.meta.data_ptr(), None)
        hid = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
        rc = L.sfb200_ffn_forward(C.byref(W), x.data_ptr(), H, hid.data_ptr(), out.data_ptr(), H, M,
                                  torch.cuda.current_stream().cuda_stream)
        assert rc == 0, (M, H, I, rc)
        pg = ops.prune_compress_24(wg, want_values=False, want_meta=False, want_pruned=True)["pruned"].float()
        pu = ops.prune_compress_24(wu, want_values=False, want_meta=False, want_pruned=True)["pruned"].float()
        gg, uu = x.float() @ pg.t(), x.float() @ pu.t()
        h_ref = (gg * torch.sigmoid(gg) * uu)
        rms_h = h_ref.pow(2).mean().sqrt()
        rel_h = ((hid.float() - h_ref).abs() / torch.maximum(h_ref.abs(), 1e-2 * rms_h)).max().item()
        assert rel_h <= REL_TOL, (M, H, I, "hidden", rel_h)
        o_ref = hid.float() @ ops.decompress_24(dn).float().t()          # down GEMM on the GPU's own hidden bits
        rms_o = o_ref.pow(2).mean().sqrt()
        rel_o = ((out.float() - o_ref).abs() / torch.maximum(o_ref.abs(), 1e-2 * rms_o)).max().item()
        assert rel_o <= REL_TOL, (M, H, I, "out", rel_o)
    assert ops.device_status() == 0
