"""sparseflow_b200: Blackwell-native 2:4-sparse FFN path behind SparseFlow's API surface."""
__version__ = "0.1.0"
