"""AdamW with the fused multi-tensor sm_100a step (one launch per parameter group).

Numerically the same update as ``torch.optim.AdamW`` (the race driver's baseline optimizer,
reference grokking_race_v2.py:570), state layout ``step / exp_avg / exp_avg_sq``.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from ._common import run_closure, zeros_state
from ._adamw_helper import adamw_step_multi


class AdamW(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = run_closure(closure)
        for group in self.param_groups:
            ps, gs, ms, vs, steps = [], [], [], [], []
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = zeros_state(p)
                    st["exp_avg_sq"] = zeros_state(p)
                st["step"] += 1
                ps.append(p); gs.append(p.grad); ms.append(st["exp_avg"]); vs.append(st["exp_avg_sq"]); steps.append(st["step"])
            adamw_step_multi(ps, gs, ms, vs, steps, group["lr"], group["betas"][0], group["betas"][1], group["eps"],
                             group["weight_decay"])
        return loss
