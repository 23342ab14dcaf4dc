"""SuperGrok v1.1: as v1.5 but with a per-tensor cosine gate sigmoid(T*cos(smart_grad, mu)) and
constant weight decay (reference grokking_optimizers/supergrok11.py:21-302,
csrc/supergrok11_kernels.cu:37,109,218, csrc/ops.cpp:211-291).

The reference copies three sums per tensor to the host between its two kernels.  Here kernel A
(mu + meta-net + partial sums), a tiny gate kernel and kernel B (Adam with the per-tensor gate
read from device memory) are queued back to back: the step never waits for the device.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import elementwise as ew
from ._common import run_closure
from ._supergrok_base import SuperGrokBase
from .metanet import SharpnessMetaNet


class SuperGrok11(SuperGrokBase):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1.0, alpha_init=0.98, lamb=5.0,
                 gamma=0.1, gamma_alpha=0.0, kappa=0.1, warmup_steps=100, warmup_ramp=100, gradient_clipping=1.0,
                 meta_net: Optional[nn.Module] = None, meta_hidden_dim=32, gate_temperature=5.0, alpha_update_freq=50,
                 meta_update_freq=5, zero_loss_threshold=1e-4, zero_acc_threshold=0.995, sam_rho=0.05,
                 sam_enable_threshold=0.0, reference_compat=False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._init_common(alpha_init=alpha_init, lamb=lamb, gamma=gamma, gamma_alpha=gamma_alpha, kappa=kappa,
                          warmup_steps=warmup_steps, warmup_ramp=warmup_ramp, gradient_clipping=gradient_clipping,
                          alpha_update_freq=alpha_update_freq, zero_loss_threshold=zero_loss_threshold,
                          zero_acc_threshold=zero_acc_threshold, sam_rho=sam_rho,
                          sam_enable_threshold=sam_enable_threshold, reference_compat=reference_compat)
        self.gate_temperature = gate_temperature
        self.meta_update_freq = meta_update_freq
        self.meta_hidden_dim = meta_hidden_dim
        self.meta_net = meta_net if meta_net is not None else SharpnessMetaNet(meta_hidden_dim)
        if hasattr(self.meta_net, "hidden_dim"):
            self.meta_hidden_dim = self.meta_net.hidden_dim
        try:
            self.meta_net = self.meta_net.to(self.param_groups[0]["params"][0].device)
        except (IndexError, KeyError):
            pass
        self.last_gates = None

    def _get_effective_sam_freq(self):
        return 999999 if self._cached_train_acc < self.sam_enable_threshold else 1

    @torch.no_grad()
    def step(self, closure=None, train_loss=None, val_loss=None, train_acc=None):
        loss = run_closure(closure)
        self._ensure_state()
        self._global_step += 1
        if train_acc is not None:
            self._cached_train_acc = train_acc
        if self._global_step % self.alpha_update_freq == 0 or self._global_step == 1:
            self._update_alpha(train_loss, val_loss, train_acc)
        ramp = self._get_ramp_factor()
        group = self.param_groups[0]
        lr, beta2, eps, wd = group["lr"], group["betas"][1], group["eps"], group["weight_decay"]
        if self._weights_dirty or self._cached_weights is None:
            self._cached_weights = self.meta_net.get_weights()
            self._weights_dirty = False
        W1, b1, W2, b2, rescale = self._cached_weights
        idx = [i for i, p in enumerate(self._flat_params) if p.grad is not None and p.numel() > 0]
        if not idx:
            return loss
        for i in idx:
            self._flat_steps[i] += 1
        bc_steps = [1 if self.reference_compat else self._flat_steps[i] for i in idx]
        pick = lambda l: [l[i] for i in idx]  # noqa: E731
        alphas = [max(0.0, min(1.0, self._cached_alpha * self._flat_layer_alphas[i])) for i in idx]
        dev = self._flat_params[idx[0]].device
        self.last_gates = ew.sg11(pick(self._flat_params), [self._flat_params[i].grad for i in idx],
                                  pick(self._flat_exp_avgs), pick(self._flat_exp_avg_sqs), pick(self._flat_mus),
                                  pick(self._flat_sharpness), bc_steps, alphas, pick(self._flat_layer_beta1s),
                                  W1.to(dev), b1.to(dev), W2.to(dev), b2.to(dev), rescale, beta2, lr, wd, eps,
                                  self.lamb, ramp, self.gate_temperature, self.gradient_clipping)
        return loss

    def meta_step(self, model, val_x, val_y, criterion, meta_optimizer):
        """Bilevel update of the meta-net against validation gradients (reference supergrok11.py:242-299).

        The reference runs this under ``torch.no_grad()``, so its meta-loss has no graph, ``backward()`` raises
        and the validation gradients are left in ``p.grad``; ``reference_compat=True`` reproduces that."""
        self._ensure_state()
        named = list(model.named_parameters())
        saved = {n: p.grad.detach().clone() for n, p in named if p.grad is not None}
        if self.reference_compat:
            model.zero_grad()
            with torch.enable_grad():
                criterion(model(val_x), val_y).backward()
            raise RuntimeError("element 0 of tensors does not require grad and does not have a grad_fn")
        try:
            names, gs, ss, sizes = [], [], [], []
            for n, p in named:
                if n in saved:
                    pidx = self._param_to_idx.get(id(p))
                    gs.append(saved[n].reshape(-1).float())
                    ss.append(self._flat_sharpness[pidx].reshape(-1))
                    names.append(n); sizes.append(p.numel())
            with torch.enable_grad():
                smart = dict(zip(names, torch.split(self.meta_net(torch.cat(gs), torch.cat(ss)), sizes))) if gs else {}
                model.zero_grad()
                val_loss = criterion(model(val_x), val_y)
                val_loss.backward()
                meta_optimizer.zero_grad()
                meta_loss = None
                for n, p in named:
                    if n in smart and p.grad is not None:
                        vg = p.grad.detach().reshape(-1).float()
                        vn = vg.norm()
                        vu = torch.where(vn > 1e-12, vg / vn.clamp_min(1e-30), vg)
                        t = -(smart[n] * vu).sum()
                        meta_loss = t if meta_loss is None else meta_loss + t
                if meta_loss is not None:
                    meta_loss.backward()
                    meta_optimizer.step()
                    self._weights_dirty = True
            return float(val_loss.item())
        finally:
            for n, p in named:
                p.grad = saved.get(n)
