"""``SparseFlowMLP``: gated-MLP replacement built on the fused sm_100a kernels.

Constructor and forward signature of the reference's ``sparseflow/nn/sparseflow_mlp.py:15-130``.
The reference runs a transposed [I, B*T] dataflow with two sparse GEMMs, a Triton SiLU.mul and a
DENSE down projection on the unpruned weight (:124).  Here gate and up are one sparse GEMM whose
epilogue applies SiLU.mul; ``down_mode`` picks the down projection: ``"dense"`` (default, the
reference's function: unpruned weight through the library GEMM) or ``"sparse"`` (pruned weight
through the sparse kernel).  Biases on gate/up select the unfused path (two GEMMs with a bias
epilogue + the standalone SiLU.mul kernel).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .policy import SparseFlowPolicy


class SparseFlowMLP(nn.Module):
    def __init__(
        self,
        hidden_size: int,
        intermediate_size: int,
        gate_weight: torch.Tensor,
        up_weight: torch.Tensor,
        down_weight: torch.Tensor,
        gate_bias: Optional[torch.Tensor] = None,
        up_bias: Optional[torch.Tensor] = None,
        down_bias: Optional[torch.Tensor] = None,
        policy: SparseFlowPolicy = SparseFlowPolicy(),
        device: str = "cuda",
        dtype: torch.dtype = torch.float16,
        down_mode: str = "dense",
    ):
        super().__init__()
        if down_mode not in ("dense", "sparse"):
            raise ValueError("down_mode must be 'dense' or 'sparse'")
        with torch.inference_mode(False):
            gate_weight = gate_weight.detach().clone().contiguous()
            up_weight = up_weight.detach().clone().contiguous()
            down_weight = down_weight.detach().clone().contiguous()
            gate_bias = None if gate_bias is None else gate_bias.detach().clone().contiguous()
            up_bias = None if up_bias is None else up_bias.detach().clone().contiguous()
            down_bias = None if down_bias is None else down_bias.detach().clone().contiguous()

        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.policy = policy
        self.down_mode = down_mode
        if gate_weight.shape != (self.intermediate_size, self.hidden_size):
            raise ValueError("gate_weight must be [intermediate_size, hidden_size]")

        self.register_buffer("down_weight", down_weight, persistent=False)
        self._fused = gate_bias is None and up_bias is None
        if self._fused:
            gu = ops.compress_gate_up(gate_weight, up_weight)
            self.register_buffer("gu_values", gu.values, persistent=False)
            self.register_buffer("gu_meta", gu.meta, persistent=False)
        else:
            g, u = ops.compress_weight(gate_weight), ops.compress_weight(up_weight)
            self.register_buffer("gate_values", g.values, persistent=False)
            self.register_buffer("gate_meta", g.meta, persistent=False)
            self.register_buffer("up_values", u.values, persistent=False)
            self.register_buffer("up_meta", u.meta, persistent=False)
        d = ops.compress_weight(down_weight)
        self.register_buffer("down_values", d.values, persistent=False)
        self.register_buffer("down_meta", d.meta, persistent=False)
        self.register_buffer("gate_bias", gate_bias, persistent=False)
        self.register_buffer("up_bias", up_bias, persistent=False)
        self.register_buffer("down_bias", down_bias, persistent=False)

    def _cw(self, which: str) -> ops.Compressed24:
        H, I = self.hidden_size, self.intermediate_size
        if which == "gu":
            return ops.Compressed24(self.gu_values, self.gu_meta, 2 * I, H, gate_up=True)
        if which == "down":
            return ops.Compressed24(self.down_values, self.down_meta, H, I)
        return ops.Compressed24(getattr(self, which + "_values"), getattr(self, which + "_meta"), I, H)

    @torch.no_grad()
    def forward(self, x):
        B, T, H = x.shape
        x2d = x.reshape(B * T, H)
        if self._fused:
            hidden = ops.sparse_gemm_swiglu(x2d, self._cw("gu"))
        else:
            gate = ops.sparse_gemm(x2d, self._cw("gate"), bias=self.gate_bias)
            up = ops.sparse_gemm(x2d, self._cw("up"), bias=self.up_bias)
            hidden = ops.silu_mul(gate, up)
        if self.down_mode == "sparse":
            out2d = ops.sparse_gemm(hidden, self._cw("down"), bias=self.down_bias)
        else:
            out2d = F.linear(hidden, self.down_weight, self.down_bias)
        return out2d.view(B, T, H)


def make_sparseflow_mlp(*args, **kwargs):
    """Factory.  Accepts the constructor arguments, or (as the reference's tools call it,
    tools/llama_surgery_mlp.py:44) a gated-MLP module with gate_proj / up_proj / down_proj."""
    if len(args) == 1 and isinstance(args[0], nn.Module):
        m = args[0]
        g, u, d = m.gate_proj, m.up_proj, m.down_proj
        return SparseFlowMLP(g.in_features, g.out_features, g.weight, u.weight, d.weight,
                             g.bias, u.bias, d.bias, **kwargs)
    return SparseFlowMLP(*args, **kwargs)
