"""Linear-level model surgery: swap the projections of every decoder layer for ``SparseFlowLinear``.

Names of the reference's ``sparseflow/nn/replace_llama.py`` (``replace_llama_mlp``, ``replace_llama_attention``)
and of the tools it forwards to: ``tools/llama_surgery.py:25-52`` (``replace_llama_mlp``: gate/up/down, each with its
own ``op_name`` so the policy can tell them apart) and ``tools/llama_surgery_full.py:20-50`` (``replace_llama_full``:
the MLP projections plus q/k/v/o).  Each returns the number of Linear layers replaced.  (For a whole-MLP swap with
the fused gate|up kernel use ``replace_llama_mlp_module`` from ``surgery.py``.)
"""
from __future__ import annotations

import torch.nn as nn

from .sparseflow_linear import make_sparseflow_linear
from .surgery import _layers_of

_MLP = ("gate_proj", "up_proj", "down_proj")
_ATTN = ("q_proj", "k_proj", "v_proj", "o_proj")


def _swap(parent: nn.Module, names, policy, li: int, verbose: bool, **kw) -> int:
    n = 0
    for proj_name in names:
        lin = getattr(parent, proj_name, None)
        if lin is None or not isinstance(lin, nn.Linear):
            continue
        setattr(parent, proj_name, make_sparseflow_linear(lin, policy=policy, op_name=proj_name, **kw))
        n += 1
        if verbose:
            print(f"  [ok] Layer {li:02d} {proj_name:10s} -> SparseFlowLinear (op_name={proj_name})")
    return n


def replace_llama_mlp(model: nn.Module, policy, verbose: bool = True, **kw) -> int:
    replaced = 0
    for li, layer in enumerate(_layers_of(model)):
        mlp = getattr(layer, "mlp", None)
        if mlp is not None:
            replaced += _swap(mlp, _MLP, policy, li, verbose, **kw)
    return replaced


def replace_llama_full(model: nn.Module, policy, verbose: bool = True, **kw) -> int:
    replaced = 0
    for li, layer in enumerate(_layers_of(model)):
        mlp = getattr(layer, "mlp", None)
        if mlp is not None:
            replaced += _swap(mlp, _MLP, policy, li, verbose, **kw)
        attn = getattr(layer, "self_attn", None)
        if attn is not None:
            replaced += _swap(attn, _ATTN, policy, li, verbose, **kw)
    return replaced


def replace_llama_attention(model: nn.Module, policy, verbose: bool = True, **kw) -> int:
    """Entry point older scripts expect; as upstream it delegates to the full swap."""
    return replace_llama_full(model, policy, verbose=verbose, **kw)
