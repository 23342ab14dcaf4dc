"""Per-tensor AdamW used by Grokfast, LookSAM and Muon's non-matrix group.

Same contract as the reference helper (grokking_optimizers/_adamw_helper.py:12-22): decoupled
weight decay ``p *= 1 - lr*wd`` first, then ``p -= lr/bc1 * m / (sqrt(v/bc2) + eps)``.
``adamw_step_multi`` does a whole group in one fused multi-tensor launch on CUDA.
"""
from __future__ import annotations

from ..ops import elementwise as ew


def adamw_step(p, grad, exp_avg, exp_avg_sq, step, lr, beta1, beta2, eps, weight_decay):
    ew.adamw([p], [grad], [exp_avg], [exp_avg_sq], [step], lr, beta1, beta2, eps, weight_decay)


def adamw_step_multi(params, grads, exp_avgs, exp_avg_sqs, steps, lr, beta1, beta2, eps, weight_decay):
    if params:
        ew.adamw(params, grads, exp_avgs, exp_avg_sqs, steps, lr, beta1, beta2, eps, weight_decay)
