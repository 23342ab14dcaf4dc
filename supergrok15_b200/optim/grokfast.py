"""Grokfast: EMA low-pass filter added to the gradient, then AdamW
(reference grokking_optimizers/grokfast.py:76-145).  The gradient is amplified in place, as in
the reference; on CUDA the filter and the AdamW update are one fused kernel.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from ..ops import elementwise as ew
from ._common import run_closure, zeros_state


class Grokfast(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.98), eps=1e-8, weight_decay=1.0, grokfast_alpha=0.98,
                 grokfast_lamb=2.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      grokfast_alpha=grokfast_alpha, grokfast_lamb=grokfast_lamb))

    @torch.no_grad()
    def step(self, closure=None):
        loss = run_closure(closure)
        for group in self.param_groups:
            ps, gs, ms, vs, es, steps = [], [], [], [], [], []
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["ema"] = zeros_state(p)
                    st["exp_avg"] = zeros_state(p)
                    st["exp_avg_sq"] = zeros_state(p)
                st["step"] += 1
                ps.append(p); gs.append(p.grad); ms.append(st["exp_avg"]); vs.append(st["exp_avg_sq"])
                es.append(st["ema"]); steps.append(st["step"])
            if ps:
                ew.grokfast_adamw(ps, gs, ms, vs, es, steps, group["lr"], group["betas"][0], group["betas"][1],
                                  group["eps"], group["weight_decay"], group["grokfast_alpha"], group["grokfast_lamb"])
        return loss
