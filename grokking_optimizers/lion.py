"""Alias of supergrok15_b200.optim.lion (same import path as the reference package)."""
from supergrok15_b200.optim.lion import Lion, Optimizer  # noqa: F401
