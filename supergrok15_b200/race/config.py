"""Configuration of the grokking race: flat dictionaries with the reference's key names
(reference grokking_race_v2.py:213-228, 1554-1623) plus a typed front end for the command line."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Dict, List, Optional

MODEL_SCALES = {
    "small": {"dim_model": 128, "num_heads": 4, "num_layers": 2},
    "medium": {"dim_model": 256, "num_heads": 8, "num_layers": 4},
    "large": {"dim_model": 512, "num_heads": 8, "num_layers": 6},
}

DEFAULT_CONFIG: Dict = {
    "p": 97, "operation": "x/y", "frac_train": 0.5,
    "num_layers": 2, "dim_model": 128, "num_heads": 4, "num_tokens": 99,
    "lr": 1e-3, "weight_decay": 1.0, "beta1": 0.9, "beta2": 0.98,
    "max_steps": 100_000, "early_stop_threshold": 0.95,
    "early_stop_patience": 500, "log_every": 10, "seed": 42,
    "compile_model": False, "use_amp": False, "model_type": "decoder",
    "patch_dim": 49, "num_patches": 16, "chain_length": 3, "seq_len": 8,
    "use_cuda_graph": False, "reference_compat": False,
}

# per-optimizer overrides as shipped by the reference's __main__ (the supergrok2 block keeps its stale keys: only
# sg2_expert_hidden and sg2_meta_rescale are read, so the race runs v2 with expert_hidden = 4)
OPTIMIZER_CONFIGS: Dict[str, Dict] = {
    "adamw": {"weight_decay": 1.0},
    "grokadamw": {"weight_decay": 1.0, "grokadamw_alpha": 0.98, "grokadamw_lamb": 5.0, "grokadamw_grad_clip": 1.0},
    "neuralgrok": {"weight_decay": 1.0, "neural_alpha": 10.0, "neural_beta": 4.0, "neural_layers": 3, "neural_hidden": 128,
                   "inner_steps": 1},
    "supergrok11": {"weight_decay": 1.0, "supergrok11_lamb": 5.0, "supergrok11_gate_temperature": 5.0,
                    "supergrok11_alpha_update_freq": 50, "supergrok11_meta_freq": 5, "supergrok11_sam_freq": 10},
    "supergrok15": {"weight_decay": 1.0, "supergrok15_lamb": 2.0, "supergrok15_alpha_update_freq": 50},
    "supergrok2": {"weight_decay": 1.0, "sg2_num_inducing": 16, "sg2_num_peer_experts": 1024, "sg2_expert_hidden": 4,
                   "sg2_meta_rescale": 0.1, "sg2_alpha_update_freq": 50},
    "grokfast": {"weight_decay": 1.0, "grokfast_alpha": 0.98, "grokfast_lamb": 2.0},
    "muon": {"weight_decay": 1.0, "muon_lr": 0.02, "muon_momentum": 0.95},
    "lion": {"lion_lr": 3e-4, "lion_wd": 3.0, "lion_beta2": 0.99},
    "looksam": {"weight_decay": 1.0, "looksam_rho": 0.05, "looksam_k": 5, "looksam_alpha": 0.7},
    "prodigy": {"weight_decay": 1.0, "prodigy_lr": 1.0},
}
ALL_OPTIMIZERS = ["adamw", "grokadamw", "neuralgrok", "supergrok11", "supergrok15", "supergrok2", "grokfast", "muon", "lion",
                  "looksam", "prodigy"]
COMMON = {"max_steps": 20_000, "early_stop_threshold": 0.95, "early_stop_patience": 500, "log_every": 10}
SEEDS = [42, 137, 256, 512, 1024]
TRAIN_SPLITS = [0.1, 0.25, 0.5, 0.8]

DISPLAY_NAMES = {"adamw": "AdamW", "grokadamw": "GrokAdamW", "neuralgrok": "NeuralGrok", "supergrok11": "SuperGrok1.1",
                 "supergrok15": "SuperGrok1.5", "supergrok2": "SuperGrok2", "grokfast": "Grokfast", "muon": "Muon", "lion": "Lion",
                 "looksam": "LookSAM", "prodigy": "Prodigy"}
MODEL_LABELS = {"decoder": "Decoder Transformer", "decoder_preln": "Pre-LN Decoder", "vit": "ViT (MNIST addition)",
                "mamba": "Mamba (chained division)"}


@dataclass
class RaceConfig:
    """Typed view of a race run; ``flat()`` yields the dictionary the training loops read."""
    optimizers: List[str] = field(default_factory=lambda: list(ALL_OPTIMIZERS))
    seeds: List[int] = field(default_factory=lambda: [42])
    model_scale: str = "small"
    model_type: str = "decoder"
    task: str = "division"            # division | addition
    frac_train: float = 0.5
    max_steps: int = 20_000
    dtype: str = "fp32"
    device: str = "auto"
    gpus: Optional[List[int]] = None
    reference_compat: bool = False
    save_dir: str = "results"
    overrides: Dict = field(default_factory=dict)

    def flat(self) -> Dict:
        c = copy.deepcopy(DEFAULT_CONFIG)
        c.update(COMMON)
        c.update(MODEL_SCALES[self.model_scale])
        c.update(model_type=self.model_type, frac_train=self.frac_train, max_steps=self.max_steps, task=self.task,
                 use_amp=self.dtype in ("bf16", "fp16"), amp_dtype=self.dtype, reference_compat=self.reference_compat)
        c.update(self.overrides)
        return c


def merged(base: Dict, name: str, extra: Optional[Dict] = None) -> Dict:
    c = dict(base)
    c.update(OPTIMIZER_CONFIGS.get("supergrok11" if name == "supergrok" else name, {}))
    if extra:
        c.update(extra)
    return c
