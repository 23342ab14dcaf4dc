"""Alias of supergrok15_b200.optim.grokadamw (same import path as the reference package)."""
from supergrok15_b200.optim.grokadamw import GrokAdamW, Optimizer  # noqa: F401
