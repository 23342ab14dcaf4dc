"""Lion: sign of an interpolated momentum (reference grokking_optimizers/lion.py:21-101).

State: ``exp_avg`` (fp32).  One fused multi-tensor launch per group on CUDA.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from ..ops import elementwise as ew
from ._common import run_closure, zeros_state


class Lion(Optimizer):
    def __init__(self, params, lr: float = 3e-4, betas=(0.9, 0.99), weight_decay: float = 3.0):
        if lr < 0:
            raise ValueError(f"Invalid learning rate: {lr}")
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = run_closure(closure)
        for group in self.param_groups:
            ps, gs, ms = [], [], []
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = zeros_state(p)
                ps.append(p); gs.append(p.grad); ms.append(st["exp_avg"])
            if ps:
                ew.lion(ps, gs, ms, group["lr"], group["betas"][0], group["betas"][1], group["weight_decay"])
        return loss
