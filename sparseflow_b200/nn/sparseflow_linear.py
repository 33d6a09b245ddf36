"""``SparseFlowLinear``: Linear layer with a per-op sparse / dense policy, sparse path on the
sm_100a tcgen05 kernels.

Interface of the reference's ``sparseflow/nn/sparseflow_linear.py``: ``prune_24_dense_weight``
(:20-35), ``SparseFlowLinear(weight, bias, policy, op_name)`` (:38-137) and
``make_sparseflow_linear`` (:140-152).  Differences:

* fp16 AND bf16 are accepted (the reference rejects bf16, :13-17);
* pruning ties are deterministic and equal to the reference CPU script (higher index wins), where
  the reference's ``torch.topk`` leaves tie order unspecified;
* bias is applied in the GEMM epilogue, and no transpose / ``.contiguous()`` copy of the output is
  needed (the reference computes Y^T and copies, :121-124);
* the dense branch uses the ORIGINAL weight, as upstream does (:128-130); pass
  ``dense_uses_pruned=True`` to make both branches compute the same function.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .policy import SparseFlowPolicy

_OK_DTYPES = (torch.float16, torch.bfloat16)


def _require_cuda_16bit(x: torch.Tensor, name: str) -> None:
    if not x.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if x.dtype not in _OK_DTYPES:
        raise ValueError(f"{name} must be torch.float16 or torch.bfloat16 (got {x.dtype})")


@torch.no_grad()
def prune_24_dense_weight(W: torch.Tensor, tie: str = "high") -> torch.Tensor:
    """Prune to 2:4 semi-structured sparsity (keep the two largest |w| of every four along in_features)."""
    _require_cuda_16bit(W, "W")
    if W.dim() != 2:
        raise ValueError(f"W must be 2D, got {W.dim()}D")
    out_f, in_f = W.shape
    if in_f % 4 != 0:
        raise ValueError(f"in_features must be multiple of 4 for 2:4 (got {in_f})")
    return ops.prune_compress_24(W, tie=tie, want_values=False, want_meta=False, want_pruned=True)["pruned"]


class SparseFlowLinear(nn.Module):
    def __init__(
        self,
        weight_fp16: torch.Tensor,
        bias_fp16: Optional[torch.Tensor],
        policy: SparseFlowPolicy = SparseFlowPolicy(),
        op_name: str = "default",
        dense_uses_pruned: bool = False,
    ):
        super().__init__()
        self.op_name = op_name
        self.policy = policy
        self.dense_uses_pruned = dense_uses_pruned

        _require_cuda_16bit(weight_fp16, "weight_fp16")
        if bias_fp16 is not None:
            _require_cuda_16bit(bias_fp16, "bias_fp16")
            if bias_fp16.dtype != weight_fp16.dtype:
                raise ValueError(f"bias dtype {bias_fp16.dtype} != weight dtype {weight_fp16.dtype}")
            if bias_fp16.numel() != weight_fp16.shape[0]:
                raise ValueError(f"bias has {bias_fp16.numel()} elements, weight has {weight_fp16.shape[0]} rows")

        W = weight_fp16.contiguous()
        self.register_buffer("W_original", W, persistent=True)
        self.out_features, self.in_features = W.shape

        # one pass: pruned dense copy + compressed values + metadata
        self._supports_sparse_weight = self.in_features % 64 == 0 and self.out_features % 8 == 0
        o = ops.prune_compress_24(W, want_values=self._supports_sparse_weight,
                                  want_meta=self._supports_sparse_weight, want_pruned=True)
        self.register_buffer("W_dense_pruned", o["pruned"], persistent=True)
        if self._supports_sparse_weight:
            self.register_buffer("W_values", o["values"], persistent=False)
            self.register_buffer("W_meta", o["meta"], persistent=False)
        else:
            self.W_values = None
            self.W_meta = None

        if bias_fp16 is not None:
            self.register_buffer("bias", bias_fp16.contiguous(), persistent=True)
        else:
            self.bias = None

        self._sparse_count = 0
        self._dense_count = 0

    @property
    def W_sparse(self) -> Optional[ops.Compressed24]:
        if self.W_values is None:
            return None
        return ops.Compressed24(self.W_values, self.W_meta, self.out_features, self.in_features)

    def extra_repr(self) -> str:
        return (
            f"op_name={self.op_name}, in={self.in_features}, out={self.out_features}, "
            f"sparse_weight={self._supports_sparse_weight}"
        )

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _require_cuda_16bit(x, "x")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"Expected last dim {self.in_features}, got {x.shape[-1]}")
        leading = x.shape[:-1]
        M = 1
        for d in leading:
            M *= int(d)
        use_sparse = (
            self.policy.supports_sm100()
            and self._supports_sparse_weight
            and self.policy.should_use_sparse(self.op_name, M)
        )
        x2d = x.reshape(M, self.in_features)
        if use_sparse:
            self._sparse_count += 1
            y2d = ops.sparse_gemm(x2d, self.W_sparse, bias=self.bias)
        else:
            self._dense_count += 1
            W = self.W_dense_pruned if self.dense_uses_pruned else self.W_original
            y2d = F.linear(x2d, W, self.bias)
        return y2d.reshape(*leading, self.out_features)

    @property
    def supports_sparse_weight(self) -> bool:
        return self._supports_sparse_weight


@torch.no_grad()
def make_sparseflow_linear(
    dense_linear: nn.Linear,
    policy: SparseFlowPolicy = SparseFlowPolicy(),
    op_name: str = "default",
    name: Optional[str] = None,
    **kw,
) -> SparseFlowLinear:
    """Convert nn.Linear to SparseFlowLinear.  ``name`` is accepted as an alias of ``op_name``
    (the reference's tools spell it that way, tools/compare_dense_pruned_sparse.py:54)."""
    if not isinstance(dense_linear, nn.Linear):
        raise TypeError("dense_linear must be torch.nn.Linear")
    W = dense_linear.weight.detach()
    b = dense_linear.bias.detach() if dense_linear.bias is not None else None
    return SparseFlowLinear(W, b, policy=policy, op_name=name or op_name, **kw)
