"""Drop-in alias of the reference's import surface (reference grokking_optimizers/__init__.py:22-47)."""
from supergrok15_b200 import _build as _build
from supergrok15_b200.optim import (AdamW, CUDAGraphOptimizer, GrokAdamW, Grokfast, Lion, LookSAM, Mamba3PEERMetaNet,
                                    Mamba3ScanBlock, MiniGRU, Muon, NeuralGrok, Prodigy, SharpnessMetaNet, SuperGrok11,
                                    SuperGrok15, SuperGrok2)

__version__ = "2.0.0"
from supergrok15_b200.ops import ref_api as _ref_api
import sys as _sys
# the reference's 22 entry points by name (adapters over the multi-tensor kernels); other attributes resolve to the native extension
_ops = _ref_api.module(__name__ + "._ops")
_sys.modules[__name__ + "._ops"] = _ops
__all__ = ["AdamW", "CUDAGraphOptimizer", "GrokAdamW", "Grokfast", "Lion", "LookSAM", "Mamba3PEERMetaNet", "Mamba3ScanBlock",
           "MiniGRU", "Muon", "NeuralGrok", "Prodigy", "SharpnessMetaNet", "SuperGrok11", "SuperGrok15", "SuperGrok2"]
