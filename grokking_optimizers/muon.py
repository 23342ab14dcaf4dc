"""Alias of supergrok15_b200.optim.muon (same import path as the reference package)."""
from supergrok15_b200.optim.muon import Iterable, Muon, Optimizer, Optional, Tuple, adamw_step_multi  # noqa: F401
