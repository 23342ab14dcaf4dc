"""Alias of supergrok15_b200.optim.neuralgrok (same import path as the reference package)."""
from supergrok15_b200.optim.neuralgrok import List, NeuralGrok, Optimizer, Tuple  # noqa: F401
