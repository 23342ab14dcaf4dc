"""Alias of supergrok15_b200.optim.prodigy (same import path as the reference package)."""
from supergrok15_b200.optim.prodigy import Optimizer, Prodigy  # noqa: F401
