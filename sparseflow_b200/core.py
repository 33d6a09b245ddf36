"""The reference's older convenience API on top of the sm_100a library.

Names, arguments and error behaviour of ``experiments/old_structure/python/sparseflow/core.py:18-116``
(documented in docs/API.md:24-127): ``check_sparse_support``, ``is_sparse_available``,
``validate_2_4``, ``prune_2_4``, ``compress_2_4`` and ``sparse_mm(A, Bc, epilogue, bias)``.

Differences a caller sees: bf16 is accepted beside fp16; the compressed form is one self-describing
``uint8`` tensor (header + values + metadata, see ``sparseflow_b200.serialize``) instead of a bare
half-size tensor, so it can be stored in a ``state_dict``; the activation and the bias run in the
GEMM epilogue rather than as separate kernels.  As upstream there is no fallback: without the
library or an sm_100 device the compute calls raise ``RuntimeError``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops, serialize

_EPILOGUES = ("none", "relu", "silu", "gelu")


def check_sparse_support() -> Tuple[bool, str]:
    """(supported, message) for the current CUDA device.  core.py:18-28."""
    try:
        from . import _lib
        _lib.lib()
    except (ImportError, OSError) as e:
        return False, f"C++ extension not available: {e}"
    if not torch.cuda.is_available():
        return False, "CUDA is not available"
    major, minor = torch.cuda.get_device_capability()
    name = torch.cuda.get_device_name()
    if major != 10:
        return False, f"{name} (SM{major}{minor}) is not supported: this build targets sm_100a only"
    return True, f"{name} (SM{major}{minor}) supports 2:4 sparse tensor cores (tcgen05)"


def is_sparse_available() -> bool:
    """core.py:30-36."""
    return check_sparse_support()[0]


def _require_lib() -> None:
    try:
        from . import _lib
        _lib.lib()
    except (ImportError, OSError) as e:
        raise RuntimeError(f"C++ extension required: {e}") from e


def validate_2_4(tensor: torch.Tensor) -> bool:
    """True iff every group of four along the last dimension has at most two non-zeros.  core.py:38-51."""
    _require_lib()
    return ops.validate_24(tensor.reshape(-1, tensor.shape[-1]))


def prune_2_4(tensor: torch.Tensor, method: str = "magnitude") -> torch.Tensor:
    """Dense tensor -> same shape with the two smallest |w| of every four zeroed.  core.py:53-73."""
    _require_lib()
    if method == "magnitude":
        w2 = tensor.reshape(-1, tensor.shape[-1])
        out = ops.prune_compress_24(w2, want_values=False, want_meta=False, want_pruned=True)["pruned"]
        return out.reshape(tensor.shape)
    if method == "random":
        raise NotImplementedError("Random pruning not yet implemented")
    raise ValueError(f"Unknown pruning method: {method}")


def compress_2_4(tensor: torch.Tensor) -> torch.Tensor:
    """Tensor with a valid 2:4 pattern -> compressed blob (uint8).  Raises ``ValueError`` on a tensor
    that is not 2:4, as core.py:75-93 does."""
    _require_lib()
    if tensor.dim() != 2:
        raise ValueError(f"expected a 2-D weight, got {tensor.dim()}-D")
    if not validate_2_4(tensor):
        raise ValueError("Tensor does not have valid 2:4 sparsity pattern")
    return serialize.pack(ops.compress_weight(tensor))


def sparse_mm(A: torch.Tensor, Bc: torch.Tensor, epilogue: str = "none",
              bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[M, N] = epilogue(A[M, K] @ B + bias) with B = W^T, W the [N, K] weight ``Bc`` was compressed
    from (upstream callers pass ``weight_compressed.t()``, nn.py:128-132; the blob is 1-D so ``.t()``
    returns it unchanged).  core.py:95-116."""
    _require_lib()
    if not is_sparse_available():
        raise RuntimeError("2:4 sparse not available on this GPU. Requires NVIDIA Blackwell (SM100).")
    if epilogue not in _EPILOGUES:
        raise ValueError(f"Unknown epilogue: {epilogue} (expected one of {_EPILOGUES})")
    cw = Bc if isinstance(Bc, ops.Compressed24) else serialize.unpack(Bc)
    if bias is not None and bias.numel() != cw.rows:
        raise ValueError(f"bias must have {cw.rows} elements, got {bias.numel()}")
    return ops.sparse_gemm(A, cw, bias=bias, act=epilogue)
