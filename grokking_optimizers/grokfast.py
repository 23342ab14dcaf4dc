"""Alias of supergrok15_b200.optim.grokfast (same import path as the reference package)."""
from supergrok15_b200.optim.grokfast import Grokfast, Optimizer  # noqa: F401
