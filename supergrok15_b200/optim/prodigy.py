"""Prodigy: distance-aware self-tuning Adam (reference grokking_optimizers/prodigy.py:64-136,
csrc/ops.cpp:425-507).  The distance estimate ``d_lr`` is global over all parameter groups and
monotone non-decreasing.  On CUDA it lives in a one-element device tensor that the reduction
kernel updates and the step kernel reads, so a step does not synchronise the host; the ``d_lr``
property reads it back on demand.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from ..ops import elementwise as ew
from ._common import run_closure, zeros_state


class Prodigy(Optimizer):
    def __init__(self, params, lr=1.0, betas=(0.9, 0.999), eps=1e-8, weight_decay=1.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._d_lr = 1e-6
        self._d_lr_dev = None

    @property
    def d_lr(self) -> float:
        if self._d_lr_dev is not None:
            self._d_lr = float(self._d_lr_dev.item())
        return self._d_lr

    @torch.no_grad()
    def step(self, closure=None):
        loss = run_closure(closure)
        ps, gs, ms, vs, ss, p0s, steps = [], [], [], [], [], [], []
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = zeros_state(p)
                    st["exp_avg_sq"] = zeros_state(p)
                    st["s"] = zeros_state(p)
                    st["param_init"] = p.detach().clone().float()
                st["step"] += 1
                ps.append(p); gs.append(p.grad); ms.append(st["exp_avg"]); vs.append(st["exp_avg_sq"])
                ss.append(st["s"]); p0s.append(st["param_init"]); steps.append(st["step"])
        if not ps:
            return loss
        if ps[0].is_cuda and self._d_lr_dev is None:
            self._d_lr_dev = torch.full((1,), self._d_lr, dtype=torch.float32, device=ps[0].device)
        cuda = ps[0].is_cuda
        r = ew.prodigy_dlr(ps, gs, ss, p0s, self._d_lr_dev, self._d_lr)     # one reduction over every group
        if not cuda:
            self._d_lr = r
        d = self._d_lr_dev if cuda else self._d_lr
        k = 0
        for group in self.param_groups:
            n = sum(1 for p in group["params"] if p.grad is not None)
            if n:
                sl = slice(k, k + n)
                ew.prodigy_step(ps[sl], gs[sl], ms[sl], vs[sl], ss[sl], steps[sl], d, group["lr"], group["betas"][0],
                                group["betas"][1], group["eps"], group["weight_decay"])
            k += n
        return loss

    def state_dict(self):
        sd = super().state_dict()
        sd["extra"] = {"d_lr": self.d_lr}
        return sd

    def load_state_dict(self, state_dict):
        extra = state_dict.get("extra")
        super().load_state_dict({k: v for k, v in state_dict.items() if k != "extra"})
        if extra and "d_lr" in extra:
            self._d_lr = float(extra["d_lr"])
            if self._d_lr_dev is not None:
                self._d_lr_dev.fill_(self._d_lr)
