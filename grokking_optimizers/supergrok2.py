"""Alias of supergrok15_b200.optim.supergrok2 (same import path as the reference package)."""
from supergrok15_b200.optim.supergrok2 import Dict, Mamba3PEERMetaNet, Optional, SuperGrok15, SuperGrok2  # noqa: F401
