"""Alias of supergrok15_b200.optim.supergrok15 (same import path as the reference package)."""
from supergrok15_b200.optim.supergrok15 import Dict, Optional, SharpnessMetaNet, SuperGrok15, SuperGrokBase  # noqa: F401
