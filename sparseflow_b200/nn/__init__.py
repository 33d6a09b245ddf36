"""sparseflow_b200.nn -- same lazy, never-raising re-export scheme as the reference's
sparseflow/nn/__init__.py:12-27."""
from importlib import import_module

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


_safe_export("sparseflow_b200.nn.policy", ["SparseFlowPolicy"])
_safe_export("sparseflow_b200.nn.surgery", ["replace_llama_mlp_module"])
_safe_export("sparseflow_b200.nn.sparseflow_linear", ["SparseFlowLinear", "make_sparseflow_linear", "prune_24_dense_weight"])
_safe_export("sparseflow_b200.nn.sparseflow_mlp", ["SparseFlowMLP", "make_sparseflow_mlp"])
_safe_export("sparseflow_b200.nn.sparse_linear", ["SparseLinear"])
_safe_export("sparseflow_b200.nn.replace_llama", ["replace_llama_mlp", "replace_llama_full", "replace_llama_attention"])
