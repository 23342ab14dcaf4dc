"""Alias of supergrok15_b200.optim.looksam (same import path as the reference package)."""
from supergrok15_b200.optim.looksam import LookSAM, Optimizer, adamw_step_multi  # noqa: F401
