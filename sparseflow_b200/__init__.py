"""sparseflow_b200: Blackwell-native 2:4-sparse FFN path behind SparseFlow's API surface.

Same best-effort re-export scheme as the reference's ``sparseflow/__init__.py:12-31``: importing
the package never raises; the compute entry points raise when the CUDA library is missing.
"""
from importlib import import_module

__version__ = "0.1.0"
__all__ = []


def _safe_export(mod: str, names: list) -> None:
    try:
        m = import_module(mod)
        g = globals()
        for n in names:
            if hasattr(m, n):
                g[n] = getattr(m, n)
                __all__.append(n)
    except Exception:
        pass


_safe_export("sparseflow_b200.dispatch", ["should_use_sparse", "classify_projection"])
_safe_export("sparseflow_b200.fused_mlp", ["SparseFlowFusedMLP"])
_safe_export("sparseflow_b200.nn.policy", ["SparseFlowPolicy"])
_safe_export("sparseflow_b200.nn.sparseflow_linear", ["SparseFlowLinear", "make_sparseflow_linear", "prune_24_dense_weight"])
_safe_export("sparseflow_b200.nn.sparseflow_mlp", ["SparseFlowMLP", "make_sparseflow_mlp"])
_safe_export("sparseflow_b200.nn.surgery", ["replace_llama_mlp_module"])
_safe_export("sparseflow_b200.core", ["compress_2_4", "validate_2_4", "prune_2_4", "sparse_mm", "check_sparse_support",
                                      "is_sparse_available"])
_safe_export("sparseflow_b200.nn.sparse_linear", ["SparseLinear"])
