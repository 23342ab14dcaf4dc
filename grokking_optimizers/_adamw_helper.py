"""Alias of supergrok15_b200.optim._adamw_helper (same import path as the reference package)."""
from supergrok15_b200.optim._adamw_helper import adamw_step, adamw_step_multi  # noqa: F401
