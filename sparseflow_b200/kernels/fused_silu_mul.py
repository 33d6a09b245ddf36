"""``fused_silu_mul(gate, up)``: same call as the reference's Triton wrapper
(sparseflow/kernels/fused_silu_mul.py:33-57), backed by the CUDA kernel in csrc/elementwise.cu.
Accepts 2-D tensors whose rows may be strided; fp16 or bf16."""
from __future__ import annotations

import torch

from .. import ops


def fused_silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    assert gate.is_cuda and up.is_cuda
    assert gate.dtype == up.dtype
    assert gate.ndim == 2 and up.ndim == 2, "fused_silu_mul expects 2D tensors"
    return ops.silu_mul(gate, up)
