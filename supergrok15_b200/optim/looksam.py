"""LookSAM: AdamW whose gradient is nudged along a sharpness direction that is refreshed
every k-th step (reference grokking_optimizers/looksam.py:80-247, csrc/looksam_kernels.cu).

``sam_step``: p += rho*g/||g||_global (in place, with fp32 backups) -> forward/backward at the
perturbed point -> restore -> v = (g_sam-g)/||g_sam-g|| per tensor -> g += alpha*||g||*v.
All norms are reduced on the device; nothing is copied to the host.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from ..ops import elementwise as ew
from ._adamw_helper import adamw_step_multi
from ._common import run_closure, zeros_state


class LookSAM(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.98), eps=1e-8, weight_decay=1.0, rho=0.05, k=5, alpha=0.7):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, rho=rho, k=k,
                                      alpha=alpha))
        self._global_step = 0

    def _init_state(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = zeros_state(p)
            st["exp_avg_sq"] = zeros_state(p)
            st["sam_direction"] = zeros_state(p)
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = run_closure(closure)
        self._global_step += 1
        for group in self.param_groups:
            ps, gs, ms, vs, steps = [], [], [], [], []
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._init_state(p)
                st["step"] += 1
                ps.append(p); gs.append(p.grad); ms.append(st["exp_avg"]); vs.append(st["exp_avg_sq"]); steps.append(st["step"])
            adamw_step_multi(ps, gs, ms, vs, steps, group["lr"], group["betas"][0], group["betas"][1], group["eps"],
                             group["weight_decay"])
        return loss

    def sam_step(self, model, train_x, train_y, criterion) -> None:
        data = []
        with torch.no_grad():
            for group in self.param_groups:
                ps = [p for p in group["params"] if p.grad is not None]
                if not ps:
                    data.append(None)
                    continue
                dirs = [self._init_state(p)["sam_direction"] for p in ps]
                orig = [p.grad.clone() for p in ps]
                backups = [zeros_state(p) for p in ps]
                ew.perturb(ps, orig, backups, group["rho"])
                data.append((ps, orig, dirs, backups, group))
        model.zero_grad()
        with torch.enable_grad():
            criterion(model(train_x), train_y).backward()
        with torch.no_grad():
            for gd in data:
                if gd is None:
                    continue
                ps, orig, dirs, backups, group = gd
                sam_grads = [p.grad if p.grad is not None else torch.zeros_like(p) for p in ps]
                ew.restore(ps, backups)
                ew.looksam_direction_adjust(orig, sam_grads, dirs, group["alpha"])
                for p, g in zip(ps, orig):
                    if p.grad is None:
                        p.grad = g
                    else:
                        p.grad.copy_(g)

    @property
    def global_step(self) -> int:
        return self._global_step

    def should_sam_step(self) -> bool:
        return self._global_step % self.param_groups[0]["k"] == 0

    def state_dict(self):
        sd = super().state_dict()
        sd["extra"] = {"global_step": self._global_step}
        return sd

    def load_state_dict(self, state_dict):
        extra = state_dict.get("extra")
        super().load_state_dict({k: v for k, v in state_dict.items() if k != "extra"})
        if extra:
            self._global_step = int(extra.get("global_step", 0))
