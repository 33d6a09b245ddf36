"""``SparseLinear``: the reference's older drop-in for ``nn.Linear``
(experiments/old_structure/python/sparseflow/nn.py:7-137).

``SparseLinear(weight_compressed, metadata, bias)`` and ``SparseLinear.from_dense(dense_linear,
method, validate, return_diff)`` as upstream.  ``weight_compressed`` is the blob of
``sparseflow_b200.core.compress_2_4`` and is a persistent buffer: ``state_dict()`` carries the packed
weight, ``load_state_dict()`` restores it, and neither prunes or compresses again.  The bias is
added in the GEMM epilogue (upstream adds it with a separate kernel, nn.py:135-136).
"""
from __future__ import annotations

import torch
from torch import nn

from .. import core as sf
from .. import serialize


class SparseLinear(nn.Module):
    def __init__(self, weight_compressed: torch.Tensor, metadata=None, bias=None):
        super().__init__()
        info = serialize.read_header(weight_compressed)
        self.in_features, self.out_features = info.K, info.rows
        self.register_buffer("weight_compressed", weight_compressed, persistent=True)
        self.metadata = metadata  # unused, kept for signature compatibility: the blob carries its metadata
        if bias is not None:
            self.bias = nn.Parameter(bias, requires_grad=False)
        else:
            self.register_parameter("bias", None)

    @staticmethod
    def empty(in_features: int, out_features: int, dtype=torch.float16, bias: bool = False, device="cuda"):
        """A module of the right shape with an all-zero weight, to be filled by ``load_state_dict``."""
        from .. import _lib
        blob = torch.zeros(serialize.blob_bytes(out_features, in_features), dtype=torch.uint8)
        rc = _lib.lib().sfb200_blob_write_header(blob.data_ptr(), out_features, in_features,
                                                 serialize._DT[dtype], 0, 0)
        _lib.check("sfb200_blob_write_header", rc)
        b = torch.zeros(out_features, dtype=dtype, device=device) if bias else None
        return SparseLinear(blob.to(device), bias=b)

    @staticmethod
    def from_dense(dense_linear: nn.Linear, method: str = "magnitude", validate: bool = True,
                   return_diff: bool = False):
        weight = dense_linear.weight.detach()
        weight_sparse = sf.prune_2_4(weight, method=method)
        if validate and not sf.validate_2_4(weight_sparse):
            raise ValueError("Failed to create valid 2:4 pattern")
        weight_compressed = sf.compress_2_4(weight_sparse)
        sparse_linear = SparseLinear(
            weight_compressed, metadata=None,
            bias=dense_linear.bias.detach() if dense_linear.bias is not None else None)
        if not return_diff:
            return sparse_linear
        with torch.no_grad():     # accuracy impact of pruning on a random probe batch (nn.py:84-108)
            x = torch.randn(128, dense_linear.in_features, device=weight.device, dtype=weight.dtype)
            dense_out = dense_linear(x)
            err = (dense_out - sparse_linear(x)).abs().float()
            diff = {
                "max_error": err.max().item(),
                "mean_error": err.mean().item(),
                "relative_error": (err / (dense_out.abs().float() + 1e-8)).mean().item(),
            }
        return sparse_linear, diff

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x_2d = x.reshape(-1, x.shape[-1])
        out = sf.sparse_mm(x_2d, self.weight_compressed.t(), epilogue="none", bias=self.bias)
        return out.view(*x.shape[:-1], -1)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"
