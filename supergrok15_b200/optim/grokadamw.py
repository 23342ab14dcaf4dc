"""GrokAdamW: global clip, EMA filter, amplification and AdamW in one pass
(reference grokking_optimizers/grokadamw.py:80-144, csrc/grokadamw_kernels.cu:42).
``gamma`` and ``decay`` are accepted and stored but unused, as in the reference.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from ..ops import elementwise as ew
from ._common import run_closure, zeros_state


class GrokAdamW(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.98), eps=1e-8, weight_decay=1.0, alpha=0.98, lamb=5.0,
                 gamma=0.1, decay=0.1, grad_clip=1.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, alpha=alpha, lamb=lamb,
                                      gamma=gamma, decay=decay, grad_clip=grad_clip))

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
                    st["exp_avg"] = zeros_state(p)
                    st["exp_avg_sq"] = zeros_state(p)
                    st["ema"] = zeros_state(p)
                st["step"] += 1
                ps.append(p); gs.append(p.grad); ms.append(st["exp_avg"]); vs.append(st["exp_avg_sq"])
                es.append(st["ema"]); steps.append(st["step"])
            if ps:
                ew.grokadamw(ps, gs, ms, vs, es, steps, group["lr"], group["betas"][0], group["betas"][1],
                             group["eps"], group["weight_decay"], group["alpha"], group["lamb"], group["grad_clip"])
        return loss
