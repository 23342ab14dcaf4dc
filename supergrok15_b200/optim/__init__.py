"""The eleven optimizers, their meta-networks and the CUDA-graph wrapper."""
from .adamw import AdamW
from .cuda_graph_optimizer import CUDAGraphOptimizer
from .grokadamw import GrokAdamW
from .grokfast import Grokfast
from .lion import Lion
from .looksam import LookSAM
from .metanet import Mamba3PEERMetaNet, Mamba3ScanBlock, MiniGRU, SharpnessMetaNet
from .muon import Muon
from .neuralgrok import NeuralGrok
from .prodigy import Prodigy
from .supergrok11 import SuperGrok11
from .supergrok15 import SuperGrok15
from .supergrok2 import SuperGrok2

__all__ = ["AdamW", "CUDAGraphOptimizer", "GrokAdamW", "Grokfast", "Lion", "LookSAM", "Mamba3PEERMetaNet",
           "Mamba3ScanBlock", "MiniGRU", "SharpnessMetaNet", "Muon", "NeuralGrok", "Prodigy", "SuperGrok11",
           "SuperGrok15", "SuperGrok2"]
