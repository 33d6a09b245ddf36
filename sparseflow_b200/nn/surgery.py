"""Swap the gated MLP of every decoder layer for ``SparseFlowMLP``.

Interface of the reference's ``sparseflow/nn/surgery.py:22-99`` (``replace_llama_mlp_module(model,
policy, verbose)`` -> number of layers replaced): walks ``model.model.layers`` or ``model.layers``,
accepts the ``gate_proj/up_proj/down_proj`` and ``w1/w3/w2`` layouts, and builds the replacement from
the layer's own weights.  ``down_mode`` is passed through (default "dense", the reference's function).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .sparseflow_mlp import SparseFlowMLP


def _get_mlp_projections(mlp: nn.Module):
    if all(hasattr(mlp, n) for n in ("gate_proj", "up_proj", "down_proj")):
        return mlp.gate_proj, mlp.up_proj, mlp.down_proj
    if all(hasattr(mlp, n) for n in ("w1", "w3", "w2")):      # w1 = gate, w3 = up, w2 = down
        return mlp.w1, mlp.w3, mlp.w2
    raise RuntimeError(f"Unsupported MLP layout: {type(mlp)}")


def _layers_of(model: nn.Module):
    if hasattr(model, "model") and hasattr(model.model, "layers"):
        return model.model.layers
    if hasattr(model, "layers"):
        return model.layers
    raise RuntimeError("Could not locate transformer layers (expected model.model.layers or model.layers).")


def replace_llama_mlp_module(model: nn.Module, policy, verbose: bool = False, down_mode: str = "dense") -> int:
    replaced = 0
    for i, layer in enumerate(_layers_of(model)):
        if not hasattr(layer, "mlp"):
            continue
        gate, up, down = _get_mlp_projections(layer.mlp)
        bias = lambda m: None if getattr(m, "bias", None) is None else m.bias.detach()
        with torch.inference_mode(False):
            layer.mlp = SparseFlowMLP(
                hidden_size=gate.in_features, intermediate_size=gate.out_features,
                gate_weight=gate.weight.detach(), up_weight=up.weight.detach(), down_weight=down.weight.detach(),
                gate_bias=bias(gate), up_bias=bias(up), down_bias=bias(down), policy=policy,
                device=str(gate.weight.device), dtype=gate.weight.dtype, down_mode=down_mode)
        replaced += 1
        if verbose:
            print(f"  layer {i:02d} mlp -> SparseFlowMLP")
    return replaced
