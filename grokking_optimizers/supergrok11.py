"""Alias of supergrok15_b200.optim.supergrok11 (same import path as the reference package)."""
from supergrok15_b200.optim.supergrok11 import Optional, SharpnessMetaNet, SuperGrok11, SuperGrokBase  # noqa: F401
