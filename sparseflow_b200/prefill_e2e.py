"""End-to-end prefill of a Llama-shaped decoder stack: dense vs pruned-dense vs sparse MLP (vs sparse
MLP + sparse attention projections), with the MLP's share of the forward time.

Stands in for the reference's ``tools/bench_prefill_e2e.py`` (three arms, same speed-up lines) and
``tools/llama_surgery_mlp.py`` (surgery + timing).  Those load a checkpoint and a tokenizer from a
model hub; here the stack is built from its SHAPE with seeded random weights and random token ids
(no checkpoint is needed to time a forward pass, and none is available offline).  The module tree
follows the usual decoder layout (``model.layers[i].self_attn.{q,k,v,o}_proj``,
``model.layers[i].mlp.{gate,up,down}_proj``) so ``replace_llama_mlp_module`` applies unchanged.

    python -m sparseflow_b200.prefill_e2e --layers 4 --batch 2 --seq 2048 [--json out.json]
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch
import torch.nn as nn
import torch.nn.functional as F

from .nn import SparseFlowPolicy, prune_24_dense_weight, replace_llama_mlp_module


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5, **kw):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, **kw))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class Attention(nn.Module):
    def __init__(self, hidden, heads, **kw):
        super().__init__()
        self.heads, self.head_dim = heads, hidden // heads
        self.q_proj = nn.Linear(hidden, hidden, bias=False, **kw)
        self.k_proj = nn.Linear(hidden, hidden, bias=False, **kw)
        self.v_proj = nn.Linear(hidden, hidden, bias=False, **kw)
        self.o_proj = nn.Linear(hidden, hidden, bias=False, **kw)

    def forward(self, x, rope):
        B, T, H = x.shape
        shp = (B, T, self.heads, self.head_dim)
        q, k, v = (p(x).view(shp).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        cos, sin = rope
        rot = lambda t: torch.cat([-t[..., self.head_dim // 2:], t[..., :self.head_dim // 2]], -1)
        q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.o_proj(a.transpose(1, 2).reshape(B, T, H))


class GatedMLP(nn.Module):
    def __init__(self, hidden, inter, **kw):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False, **kw)
        self.up_proj = nn.Linear(hidden, inter, bias=False, **kw)
        self.down_proj = nn.Linear(inter, hidden, bias=False, **kw)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class DecoderLayer(nn.Module):
    def __init__(self, hidden, inter, heads, **kw):
        super().__init__()
        self.input_layernorm = RMSNorm(hidden, **kw)
        self.self_attn = Attention(hidden, heads, **kw)
        self.post_attention_layernorm = RMSNorm(hidden, **kw)
        self.mlp = GatedMLP(hidden, inter, **kw)

    def forward(self, x, rope):
        x = x + self.self_attn(self.input_layernorm(x), rope)
        return x + self.mlp(self.post_attention_layernorm(x))


class LlamaShapedStack(nn.Module):
    """Embedding -> N decoder layers -> norm.  (No LM head: prefill cost is the layers'.)"""

    def __init__(self, layers, hidden, inter, heads, vocab=32000, device="cuda", dtype=torch.bfloat16, seed=0):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        torch.manual_seed(seed)
        self.embed_tokens = nn.Embedding(vocab, hidden, **kw)
        self.layers = nn.ModuleList([DecoderLayer(hidden, inter, heads, **kw) for _ in range(layers)])
        self.norm = RMSNorm(hidden, **kw)
        self.head_dim = hidden // heads
        for p in self.parameters():
            if p.dim() == 2:
                p.data.normal_(0, 0.02)

    def rope(self, T, device, dtype):
        inv = 1.0 / (10000 ** (torch.arange(0, self.head_dim, 2, device=device).float() / self.head_dim))
        f = torch.outer(torch.arange(T, device=device).float(), inv)
        emb = torch.cat([f, f], -1)
        return emb.cos().to(dtype)[None, None], emb.sin().to(dtype)[None, None]

    @torch.no_grad()
    def forward(self, ids):
        x = self.embed_tokens(ids)
        rope = self.rope(ids.shape[1], ids.device, x.dtype)
        for layer in self.layers:
            x = layer(x, rope)
        return self.norm(x)


class _MlpTimer:
    """CUDA events around every ``layer.mlp`` call."""

    def __init__(self, model):
        self.pairs, self.handles = [], []
        for layer in model.layers:
            self.handles.append(layer.mlp.register_forward_pre_hook(self._pre))
            self.handles.append(layer.mlp.register_forward_hook(self._post))

    def _pre(self, mod, args):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self._open = e

    def _post(self, mod, args, out):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.pairs.append((self._open, e))

    def total_ms(self):
        torch.cuda.synchronize()
        t = sum(a.elapsed_time(b) for a, b in self.pairs)
        self.pairs.clear()
        return t

    def remove(self):
        for h in self.handles:
            h.remove()


@torch.no_grad()
def time_arm(model, ids, iters, warmup):
    for _ in range(warmup):
        model(ids)
    timer = _MlpTimer(model)
    whole, mlp = [], []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        model(ids)
        b.record()
        mlp.append(timer.total_ms())
        whole.append(a.elapsed_time(b))
    timer.remove()
    return statistics.median(whole), statistics.median(mlp)


def sparsify_attention(model, policy) -> int:
    """q/k/v/o of every layer through ``SparseFlowLinear`` (the MLPs were already swapped as whole modules)."""
    from .nn.replace_llama import replace_llama_full
    return replace_llama_full(model, policy, verbose=False, dense_uses_pruned=True)


def run(layers=4, hidden=4096, inter=11008, heads=32, batch=2, seq=2048, dtype="bf16", iters=10, warmup=3,
        attention=True) -> dict:
    td = torch.bfloat16 if dtype == "bf16" else torch.float16
    model = LlamaShapedStack(layers, hidden, inter, heads, dtype=td).eval()
    g = torch.Generator(device="cpu").manual_seed(1234)
    ids = torch.randint(0, 32000, (batch, seq), generator=g).cuda()
    res = {"config": dict(layers=layers, hidden=hidden, inter=inter, heads=heads, batch=batch, seq=seq,
                          tokens=batch * seq, dtype=dtype, weights="seeded random N(0, 0.02), no checkpoint",
                          iters=iters, warmup=warmup), "arms": {}}

    def arm(name):
        ms, mlp_ms = time_arm(model, ids, iters, warmup)
        res["arms"][name] = dict(ms=ms, mlp_ms=mlp_ms, mlp_share=mlp_ms / ms, tokens_per_s=batch * seq / ms * 1e3)

    arm("dense")
    for m in model.modules():                       # every Linear, as the reference's pruned-dense arm does
        if isinstance(m, nn.Linear):
            m.weight.data.copy_(prune_24_dense_weight(m.weight.data))
    ref_out = model(ids)
    arm("pruned_dense")
    M = batch * seq
    policy = SparseFlowPolicy()
    n = replace_llama_mlp_module(model, policy, down_mode="sparse")
    res["mlp_layers_replaced"] = n
    out = model(ids)
    err = (out.float() - ref_out.float()).abs().max().item() / ref_out.float().abs().max().item()
    res["sparse_vs_pruned_dense_max_err_over_max"] = err        # demo/demo_harness.py:187 metric
    arm("sparse_mlp")
    if attention:
        res["attn_linears_replaced"] = sparsify_attention(model, policy)
        res["attn_uses_sparse_at_this_M"] = policy.should_use_sparse("q_proj", M)
        arm("sparse_mlp_attn")
    a = res["arms"]
    res["speedup_sparse_vs_pruned_dense"] = a["pruned_dense"]["ms"] / a["sparse_mlp"]["ms"]
    res["speedup_sparse_vs_dense"] = a["dense"]["ms"] / a["sparse_mlp"]["ms"]
    res["mlp_speedup"] = a["pruned_dense"]["mlp_ms"] / a["sparse_mlp"]["mlp_ms"]
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=11008)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-attention", action="store_true")
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    assert torch.cuda.is_available(), "CUDA required"
    r = run(a.layers, a.hidden, a.inter, a.heads, a.batch, a.seq, a.dtype, a.iters, a.warmup, not a.no_attention)
    for name, v in r["arms"].items():
        print(f"{name:16s} {v['ms']:8.3f} ms   MLP {v['mlp_ms']:8.3f} ms ({100 * v['mlp_share']:.1f} %)   "
              f"{v['tokens_per_s']:.0f} tok/s")
    print(f"Speedup (sparse vs pruned-dense): {r['speedup_sparse_vs_pruned_dense']:.2f}x   "
          f"(sparse vs dense): {r['speedup_sparse_vs_dense']:.2f}x   MLP alone: {r['mlp_speedup']:.2f}x   "
          f"max err / max: {r['sparse_vs_pruned_dense_max_err_over_max']:.2e}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump(r, f, indent=1)


if __name__ == "__main__":
    main()
