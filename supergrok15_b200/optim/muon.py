"""Muon: momentum followed by 5 Newton-Schulz iterations on every 2-D weight; AdamW for the rest
(reference grokking_optimizers/muon.py:45-210, csrc/ops.cpp:663-746).

Update of a matrix:  buf = m*buf + g ;  X = buf/(||buf||+1e-7) ;  X <- NS_k(X) ;
p = (p - 0.2*lr*X) * (1 - lr*wd).  No Nesterov term and no (1-m) factor, as in the reference.
On CUDA the momentum/norm pass is one multi-tensor kernel, the norms stay on the device, and the
Newton-Schulz chain runs on the tcgen05 GEMM kernels (``ops/muon.py``).
"""
from __future__ import annotations

from typing import Iterable, Optional, Tuple

import torch
from torch.optim import Optimizer

from ..ops import muon as muon_ops
from ._adamw_helper import adamw_step_multi
from ._common import run_closure, zeros_state


class Muon(Optimizer):
    def __init__(self, params_2d: Iterable, params_1d: Optional[Iterable] = None, lr: float = 0.02,
                 momentum: float = 0.95, weight_decay: float = 1.0, adamw_lr: float = 1e-3,
                 adamw_betas: Tuple[float, float] = (0.9, 0.98), adamw_eps: float = 1e-8, ns_steps: int = 5):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if adamw_lr < 0.0:
            raise ValueError(f"Invalid AdamW learning rate: {adamw_lr}")
        if not 0.0 <= momentum < 1.0:
            raise ValueError(f"Invalid momentum: {momentum}")
        for i in (0, 1):
            if not 0.0 <= adamw_betas[i] < 1.0:
                raise ValueError(f"Invalid AdamW beta at index {i}: {adamw_betas[i]}")
        if ns_steps < 1:
            raise ValueError(f"Invalid ns_steps: {ns_steps}")
        p2, p1 = list(params_2d), (list(params_1d) if params_1d is not None else [])
        groups = [dict(params=p2, lr=lr, momentum=momentum, weight_decay=weight_decay, ns_steps=ns_steps,
                       group_type="muon")]
        if p1:
            groups.append(dict(params=p1, lr=adamw_lr, betas=adamw_betas, eps=adamw_eps, weight_decay=weight_decay,
                               group_type="adamw"))
        super().__init__(groups, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, ns_steps=ns_steps,
                                      group_type="muon"))

    @torch.no_grad()
    def step(self, closure=None):
        loss = run_closure(closure)
        for group in self.param_groups:
            if group.get("group_type", "muon") == "muon":
                self._step_muon(group)
            else:
                self._step_adamw(group)
        return loss

    def _step_muon(self, group):
        ps, gs, bufs = [], [], []
        for p in group["params"]:
            if p.grad is None:
                continue
            if p.dim() != 2:
                raise ValueError("Muon's matrix group got a parameter that is not 2-D; pass it in params_1d")
            st = self.state[p]
            if not st:
                st["momentum_buffer"] = zeros_state(p)
            ps.append(p); gs.append(p.grad); bufs.append(st["momentum_buffer"])
        if ps:
            muon_ops.muon_step(ps, gs, bufs, group["lr"], group["momentum"], group["weight_decay"], group["ns_steps"])

    def _step_adamw(self, group):
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
