"""NeuralGrok: Adam on gradients rescaled by a learned MLP amplifier
(reference grokking_optimizers/neuralgrok.py:22-243, csrc/neuralgrok_kernels.cu:244).

The fused kernel evaluates the amplifier's FIRST and LAST linear layers only (1 -> H ReLU -> 1),
which is the reference kernel's contract; with ``num_layers=2`` that is the whole amplifier.
The amplifier itself is trained by a separate Adam (``get_amplifier_optimizer``); call
``mark_amplifier_dirty()`` after that optimizer steps so the cached weights are refreshed.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.nn as nn
from torch.optim import Optimizer

from ..ops import elementwise as ew
from ._common import run_closure, zeros_state


class _Amplifier(nn.Module):
    def __init__(self, num_layers: int = 3, hidden_dim: int = 128) -> None:
        super().__init__()
        if num_layers < 2:
            raise ValueError("num_layers must be >= 2 (input + output layer)")
        self.hidden_dim = hidden_dim
        layers: List[nn.Module] = [nn.Linear(1, hidden_dim), nn.ReLU()]
        for _ in range(num_layers - 2):
            layers += [nn.Linear(hidden_dim, hidden_dim), nn.ReLU()]
        layers.append(nn.Linear(hidden_dim, 1))
        self.net = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)

    def get_weights(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        first, last = self.net[0], self.net[-1]
        c = lambda t: t.detach().float().contiguous()  # noqa: E731
        return c(first.weight), c(first.bias), c(last.weight), c(last.bias)


class NeuralGrok(Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.98), eps=1e-8, weight_decay=1.0, alpha=10.0, beta=4.0,
                 num_layers=3, hidden_dim=128, inner_steps=1, grad_clip=1.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, alpha=alpha, beta=beta,
                                      inner_steps=inner_steps, grad_clip=grad_clip))
        self.amplifier = _Amplifier(num_layers, hidden_dim)
        try:
            self.amplifier = self.amplifier.to(self.param_groups[0]["params"][0].device)
        except (IndexError, KeyError):
            pass
        self._cached_meta_weights = None
        self._meta_weights_dirty = True

    @torch.no_grad()
    def step(self, closure=None):
        loss = run_closure(closure)
        if self._meta_weights_dirty or self._cached_meta_weights is None:
            self._cached_meta_weights = self.amplifier.get_weights()
            self._meta_weights_dirty = False
        W1, b1, W2, b2 = self._cached_meta_weights
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
            if not ps:
                continue
            dev = ps[0].device
            ew.neuralgrok(ps, gs, ms, vs, steps, W1.to(dev), b1.to(dev), W2.to(dev), b2.to(dev), group["alpha"],
                          group["beta"], group["lr"], group["betas"][0], group["betas"][1], group["eps"],
                          group["weight_decay"], group["grad_clip"])
        return loss

    def mark_amplifier_dirty(self) -> None:
        self._meta_weights_dirty = True

    def get_amplifier(self) -> _Amplifier:
        return self.amplifier

    def get_amplifier_optimizer(self, lr: float = 1e-4) -> torch.optim.Adam:
        return torch.optim.Adam(self.amplifier.parameters(), lr=lr)

    def state_dict(self):
        sd = super().state_dict()
        sd["extra"] = {"amplifier": self.amplifier.state_dict()}
        return sd

    def load_state_dict(self, state_dict):
        extra = state_dict.get("extra")
        super().load_state_dict({k: v for k, v in state_dict.items() if k != "extra"})
        if extra and "amplifier" in extra:
            self.amplifier.load_state_dict(extra["amplifier"])
            self._meta_weights_dirty = True
