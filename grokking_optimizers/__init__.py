"""Drop-in alias of the reference's import surface (reference grokking_optimizers/__init__.py:22-47)."""
from supergrok15_b200 import _build as _build
from supergrok15_b200.optim import (AdamW, CUDAGraphOptimizer, GrokAdamW, Grokfast, Lion, LookSAM, Mamba3PEERMetaNet,
                                    Mamba3ScanBlock, MiniGRU, Muon, NeuralGrok, Prodigy, SharpnessMetaNet, SuperGrok11,
                                    SuperGrok15, SuperGrok2)

__version__ = "2.0.0"
_ops = _build.load()            # native extension module (None when it has not been built); CUDA steps require it
__all__ = ["AdamW", "CUDAGraphOptimizer", "GrokAdamW", "Grokfast", "Lion", "LookSAM", "Mamba3PEERMetaNet", "Mamba3ScanBlock",
           "MiniGRU", "Muon", "NeuralGrok", "Prodigy", "SharpnessMetaNet", "SuperGrok11", "SuperGrok15", "SuperGrok2"]
