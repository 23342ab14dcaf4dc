"""Alias of supergrok15_b200.optim.cuda_graph_optimizer (same import path as the reference package)."""
from supergrok15_b200.optim.cuda_graph_optimizer import CUDAGraphOptimizer, List, Optional  # noqa: F401
