"""sparseflow_b200.nn: the module-level surface of the reference's ``sparseflow.nn`` (its ``__init__`` exports
``SparseFlowPolicy``, ``replace_llama_mlp_module``, the Linear and MLP classes and their ``make_*`` helpers,
sparseflow/nn/__init__.py:12-27) plus ``SparseLinear`` and the ``replace_llama*`` helpers.

Like upstream, importing the package must never fail because one submodule cannot be imported (torch missing, the CUDA
library not built yet): each name is bound only if its module imports and defines it.
"""
import importlib

_EXPORTS = {
    "policy": ("SparseFlowPolicy",),
    "surgery": ("replace_llama_mlp_module",),
    "sparseflow_linear": ("SparseFlowLinear", "make_sparseflow_linear", "prune_24_dense_weight"),
    "sparseflow_mlp": ("SparseFlowMLP", "make_sparseflow_mlp"),
    "sparse_linear": ("SparseLinear",),
    "replace_llama": ("replace_llama_mlp", "replace_llama_full", "replace_llama_attention"),
}

__all__ = []
for _module, _names in _EXPORTS.items():
    try:
        _m = importlib.import_module(f"{__name__}.{_module}")
    except Exception:          # keep going: the other modules are still usable
        continue
    for _n in _names:
        if hasattr(_m, _n):
            globals()[_n] = getattr(_m, _n)
            __all__.append(_n)
del _module, _names
