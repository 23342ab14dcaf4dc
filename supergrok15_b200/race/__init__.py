"""The grokking race: data, models, one training loop with per-optimizer specs, pipelines, status server, plots."""
from .config import ALL_OPTIMIZERS, DEFAULT_CONFIG, MODEL_SCALES, OPTIMIZER_CONFIGS, RaceConfig
from .data import (make_addition_data, make_data, make_data_for_task, make_mnist_addition_data,
                   make_sequential_division_data)
from .runner import (main, print_summary, run_architecture_comparison, run_full_sweep, run_multi_split, run_pipeline,
                     run_scale_comparison, save_json)
from .train import OPTIMIZER_REGISTRY, EarlyStopper, TrainResult, evaluate, get_init_state, train
