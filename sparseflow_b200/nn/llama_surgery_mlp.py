"""Module name the reference's tooling imports (``sparseflow/nn/llama_surgery_mlp.py``): re-exports
``replace_llama_mlp_module``."""
from .surgery import replace_llama_mlp_module

__all__ = ["replace_llama_mlp_module"]
