"""``SparseFlowFusedMLP``: the gated FFN hot path, out = down(act(gate(x)) * up(x)).

Constructor and forward of the reference's ``sparseflow/fused_mlp.py:9-98``: takes the three
``nn.Linear`` projections, assumes their weights are ALREADY 2:4 (it does not prune; a weight that
is not 2:4 leaves that GEMM dense for good, as upstream :21-30), gates each GEMM with
``should_use_sparse`` unless ``force_mode`` is "sparse" or "dense".

What changed underneath: gate|up is one tcgen05 sparse GEMM whose epilogue applies SiLU.mul and
writes only ``hidden`` (upstream: GEMM, chunk, act, mul as separate kernels, :77-83); no M padding
buffers (:38-61) because ragged token tiles are zero-filled by TMA; fp16 and bf16.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops
from .dispatch import get_padded_M, should_use_sparse  # noqa: F401  (same names as upstream)


class SparseFlowFusedMLP(nn.Module):
    def __init__(self, gate_proj, up_proj, down_proj, act_fn=nn.SiLU(), force_mode="auto", debug=False):
        super().__init__()
        if force_mode not in ("auto", "sparse", "dense"):
            raise ValueError("force_mode must be 'auto', 'sparse' or 'dense'")
        self.act_fn = act_fn
        self.force_mode = force_mode
        self.debug = debug
        self.hidden_size = gate_proj.in_features
        self.intermediate_size = gate_proj.out_features

        fused_weight = torch.cat([gate_proj.weight.data, up_proj.weight.data], dim=0).contiguous()
        self.fused_gate_up_weight = nn.Parameter(fused_weight, requires_grad=False)
        self.down_weight = nn.Parameter(down_proj.weight.data.contiguous(), requires_grad=False)
        self.down_bias = down_proj.bias
        self._silu = isinstance(act_fn, nn.SiLU) or act_fn is torch.nn.functional.silu

        H, I = self.hidden_size, self.intermediate_size
        self._gate_up_sparse = None   # fused, 16-row interleaved (SiLU epilogue)
        self._gate_up_plain = None    # [gate; up] row order (other activations)
        self._down_sparse = None
        w = self.fused_gate_up_weight
        ok16 = w.is_cuda and w.dtype in (torch.float16, torch.bfloat16)
        if ok16 and H % 64 == 0 and I % 16 == 0 and ops.validate_24(w):
            if self._silu:
                self._gate_up_sparse = ops.compress_gate_up(w[:I], w[I:])
            else:
                self._gate_up_plain = ops.compress_weight(w)
        if ok16 and I % 64 == 0 and H % 8 == 0 and ops.validate_24(self.down_weight):
            self._down_sparse = ops.compress_weight(self.down_weight)

    def compressed_state(self) -> dict:
        """The packed weights as ``uint8`` blobs (plus the bias): what a checkpoint needs to rebuild the
        sparse path without pruning, validating or compressing again.  Keys absent = that GEMM is dense."""
        from . import serialize
        st = {}
        gu = self._gate_up_sparse if self._gate_up_sparse is not None else self._gate_up_plain
        if gu is not None:
            st["gate_up"] = serialize.pack(gu)
        if self._down_sparse is not None:
            st["down"] = serialize.pack(self._down_sparse)
        if self.down_bias is not None:
            st["down_bias"] = self.down_bias.detach()
        return st

    @classmethod
    def from_compressed_state(cls, state: dict, act_fn=nn.SiLU(), force_mode: str = "sparse") -> "SparseFlowFusedMLP":
        """Rebuild from ``compressed_state()``.  Both GEMMs must be present in packed form; the module
        holds no dense weights, so only ``force_mode="sparse"`` is possible."""
        from . import serialize
        if force_mode != "sparse":
            raise ValueError("a module rebuilt from packed weights has no dense copy: force_mode must be 'sparse'")
        if "gate_up" not in state or "down" not in state:
            raise ValueError("state needs both 'gate_up' and 'down' blobs")
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        gu, down = serialize.unpack(state["gate_up"]), serialize.unpack(state["down"])
        if gu.rows != 2 * down.K or gu.K != down.rows:
            raise ValueError(f"gate_up {gu.rows}x{gu.K} and down {down.rows}x{down.K} do not form a gated FFN")
        self.act_fn, self.force_mode, self.debug = act_fn, force_mode, False
        self.hidden_size, self.intermediate_size = gu.K, down.K
        self._silu = isinstance(act_fn, nn.SiLU) or act_fn is torch.nn.functional.silu
        if gu.gate_up != self._silu:
            raise ValueError("the gate|up blob's row order does not match the activation it was packed for")
        self.fused_gate_up_weight = None
        self.down_weight = None
        self.down_bias = state.get("down_bias")
        self._gate_up_sparse = gu if gu.gate_up else None
        self._gate_up_plain = None if gu.gate_up else gu
        self._down_sparse = down
        self._shape_gu = (gu.rows, gu.K)
        self._shape_d = (down.rows, down.K)
        return self

    def _has_gu_sparse(self) -> bool:
        return self._gate_up_sparse is not None or self._gate_up_plain is not None

    @torch.no_grad()
    def forward(self, x):
        orig_shape = x.shape
        x_2d = x.reshape(-1, self.hidden_size)
        M_eff = x_2d.shape[0]
        out_gu, in_gu = self._shape_gu if self.fused_gate_up_weight is None else self.fused_gate_up_weight.shape
        out_d, in_d = self._shape_d if self.down_weight is None else self.down_weight.shape

        use_sparse_gu = self._has_gu_sparse() and (
            self.force_mode == "sparse"
            or (self.force_mode == "auto" and should_use_sparse(M_eff, in_gu, out_gu))
        )
        if self.force_mode == "sparse" and not self._has_gu_sparse():
            raise RuntimeError("force_mode='sparse' but the gate/up weight is not 2:4 or not a supported shape")
        if use_sparse_gu and self._gate_up_sparse is not None:
            hidden = ops.sparse_gemm_swiglu(x_2d, self._gate_up_sparse)
        else:
            if use_sparse_gu:
                fused_out = ops.sparse_gemm(x_2d, self._gate_up_plain)
            else:
                fused_out = nn.functional.linear(x_2d, self.fused_gate_up_weight)
            gate, up = fused_out.chunk(2, dim=-1)
            hidden = ops.silu_mul(gate, up) if self._silu else self.act_fn(gate) * up

        use_sparse_d = self._down_sparse is not None and (
            self.force_mode == "sparse"
            or (self.force_mode == "auto" and should_use_sparse(M_eff, in_d, out_d))
        )
        if self.force_mode == "sparse" and self._down_sparse is None:
            raise RuntimeError("force_mode='sparse' but the down weight is not 2:4 or not a supported shape")
        if use_sparse_d:
            out = ops.sparse_gemm(hidden, self._down_sparse, bias=self.down_bias)
        else:
            out = nn.functional.linear(hidden, self.down_weight, self.down_bias)
        return out.view(*orig_shape[:-1], out.shape[-1])
