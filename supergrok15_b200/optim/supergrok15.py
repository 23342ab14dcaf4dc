"""SuperGrok v1.5: AdamW + gradient EMA (mu) + 2->H->1 sharpness meta-net + sigmoid schedules
(reference grokking_optimizers/supergrok15.py:74-478, csrc/supergrok15_kernels.cu:323,
csrc/ops.cpp:83-152).

Per step: global clip -> mu = a_i*mu + (1-a_i)g -> sg = g + rescale*MLP(g, sharpness) ->
fg = sg + lamb_eff*mu -> Adam(fg; beta1_i, beta2) with progressive weight decay, where
lamb_eff = ramp*gate*lamb, gate = sigmoid(gate_scale*(train_acc-gate_thresh)).  On CUDA this is one
reduction launch plus one fused multi-tensor launch with the clip coefficient read on device.
"""
from __future__ import annotations

import warnings
from typing import Dict, Optional

import torch
import torch.nn as nn

from ..ops import elementwise as ew
from ._common import run_closure
from ._supergrok_base import SuperGrokBase
from .metanet import SharpnessMetaNet

__all__ = ["SuperGrok15", "SharpnessMetaNet"]


class SuperGrok15(SuperGrokBase):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1.0, alpha_init=0.98, lamb=2.0,
                 gamma=0.1, gamma_alpha=0.0, kappa=0.1, warmup_steps=100, warmup_ramp=100, gradient_clipping=1.0,
                 meta_net: Optional[nn.Module] = None, meta_hidden_dim=32, alpha_update_freq=100,
                 zero_loss_threshold=1e-4, zero_acc_threshold=0.995, sam_rho=0.05, gate_scale=20.0, gate_thresh=0.8,
                 sam_freq_min=3, sam_freq_max=20, sam_scale=20.0, sam_thresh=0.85, bilevel_freq_min=5,
                 bilevel_freq_max=30, bilevel_scale=20.0, bilevel_thresh=0.9, wd_ramp=4.0, wd_scale=20.0,
                 wd_thresh=0.9, sam_enable_threshold=0.0, reference_compat=False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._init_common(alpha_init=alpha_init, lamb=lamb, gamma=gamma, gamma_alpha=gamma_alpha, kappa=kappa,
                          warmup_steps=warmup_steps, warmup_ramp=warmup_ramp, gradient_clipping=gradient_clipping,
                          alpha_update_freq=alpha_update_freq, zero_loss_threshold=zero_loss_threshold,
                          zero_acc_threshold=zero_acc_threshold, sam_rho=sam_rho,
                          sam_enable_threshold=sam_enable_threshold, reference_compat=reference_compat)
        self.gate_scale, self.gate_thresh = gate_scale, gate_thresh
        self.sam_freq_min, self.sam_freq_max, self.sam_scale, self.sam_thresh = sam_freq_min, sam_freq_max, sam_scale, sam_thresh
        self.bilevel_freq_min, self.bilevel_freq_max = bilevel_freq_min, bilevel_freq_max
        self.bilevel_scale, self.bilevel_thresh = bilevel_scale, bilevel_thresh
        self.wd_ramp, self.wd_scale, self.wd_thresh = wd_ramp, wd_scale, wd_thresh
        self.meta_hidden_dim = meta_hidden_dim
        self.meta_net = meta_net if meta_net is not None else SharpnessMetaNet(meta_hidden_dim)
        if hasattr(self.meta_net, "hidden_dim"):
            self.meta_hidden_dim = self.meta_net.hidden_dim
        try:
            self.meta_net = self.meta_net.to(self.param_groups[0]["params"][0].device)
        except (IndexError, KeyError):
            pass

    # ------------------------------------------------------------------ schedules
    def _get_effective_wd(self, base_wd):
        return base_wd * (1.0 + self.wd_ramp * self._sigmoid(self.wd_scale, self._cached_train_acc, self.wd_thresh))

    def _get_gate_signal(self):
        return self._sigmoid(self.gate_scale, self._cached_train_acc, self.gate_thresh)

    def _get_effective_sam_freq(self):
        if self._cached_train_acc < self.sam_enable_threshold:
            return 999999
        heat = self._sigmoid(self.sam_scale, self._cached_train_acc, self.sam_thresh)
        return max(1, round(self.sam_freq_max - (self.sam_freq_max - self.sam_freq_min) * heat))

    def _get_effective_bilevel_freq(self):
        heat = self._sigmoid(self.bilevel_scale, self._cached_train_acc, self.bilevel_thresh)
        return max(1, round(self.bilevel_freq_max - (self.bilevel_freq_max - self.bilevel_freq_min) * heat))

    def get_effective_wd(self):
        return self._get_effective_wd(self.param_groups[0]["weight_decay"]) if self.param_groups else 0.0

    def _schedule_tick(self, train_loss, val_loss, train_acc, memorised_refresh=True):
        self._global_step += 1
        if train_acc is not None:
            self._cached_train_acc = train_acc
        if self._global_step % self.alpha_update_freq == 0 or self._global_step == 1:
            self._update_alpha(train_loss, val_loss, train_acc)
        elif memorised_refresh and ((train_acc is not None and train_acc >= self.zero_acc_threshold) or
                                    (train_loss is not None and train_loss < self.zero_loss_threshold)):
            self._update_alpha(train_loss, val_loss, train_acc)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None, train_loss=None, val_loss=None, train_acc=None):
        loss = run_closure(closure)
        self._ensure_state()
        self._schedule_tick(train_loss, val_loss, train_acc)
        ramp = self._get_ramp_factor()
        group = self.param_groups[0]                       # only the first group's hyper-parameters are read
        lr, beta2, eps = group["lr"], group["betas"][1], group["eps"]
        wd_eff = self._get_effective_wd(group["weight_decay"])
        gate = self._get_gate_signal()
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
        ew.sg15(pick(self._flat_params), [self._flat_params[i].grad for i in idx], pick(self._flat_exp_avgs),
                pick(self._flat_exp_avg_sqs), pick(self._flat_mus), pick(self._flat_sharpness), bc_steps, alphas,
                pick(self._flat_layer_beta1s), W1.to(dev), b1.to(dev), W2.to(dev), b2.to(dev), rescale, beta2, lr,
                wd_eff, eps, self.lamb, ramp, gate, self.gradient_clipping)
        return loss

    # ------------------------------------------------------------------ bilevel
    def bilevel_step(self, model, train_x, train_y, val_x, val_y, criterion, meta_optimizer):
        """One meta-learning update: meta_loss = -sum_i <meta_net(g_i, s_i), vg_i/||vg_i||> with vg the
        validation gradient (reference supergrok15.py:354-411).  Training gradients are restored."""
        self._ensure_state()
        named = list(model.named_parameters())
        saved = {n: p.grad.detach().clone() for n, p in named if p.grad is not None}
        try:
            names, gs, ss, sizes = [], [], [], []
            for n, p in named:
                if n in saved:
                    pidx = self._param_to_idx.get(id(p))
                    gs.append(saved[n].reshape(-1).float())
                    ss.append(self._flat_sharpness[pidx].reshape(-1) if pidx is not None
                              else torch.zeros(p.numel(), device=p.device))
                    names.append(n); sizes.append(p.numel())
            smart = {}
            with torch.enable_grad():
                if gs:
                    cat = self.meta_net(torch.cat(gs), torch.cat(ss))
                    for n, chunk in zip(names, torch.split(cat, sizes)):
                        smart[n] = chunk
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
                        term = -(smart[n] * vu).sum()
                        meta_loss = term if meta_loss is None else meta_loss + term
                if meta_loss is not None:
                    meta_loss.backward()
                    meta_optimizer.step()
                    self._weights_dirty = True
            return float(val_loss.item())
        finally:
            for n, p in named:
                p.grad = saved.get(n)

    def sam_meta_step(self, model, train_x, train_y, val_x, val_y, criterion, meta_optimizer):
        return (self.sam_step(model, train_x, train_y, criterion),
                self.bilevel_step(model, train_x, train_y, val_x, val_y, criterion, meta_optimizer))

    def step_full(self, model, train_x, train_y, val_x, val_y, criterion=None):
        """forward + backward + (scheduled) SAM + (scheduled) bilevel + step; returns a metrics dict.
        Failures of the SAM / bilevel sub-steps are reported as warnings, not swallowed."""
        criterion = criterion or nn.CrossEntropyLoss()
        if not hasattr(self, "_auto_meta_opt"):
            self._auto_meta_opt = torch.optim.Adam(self.meta_net.parameters(), lr=1e-4)
        model.zero_grad()
        logits = model(train_x)
        loss = criterion(logits, train_y)
        loss.backward()
        metrics: Dict[str, float] = {}
        step_num = self._global_step + 1
        if step_num % self._get_effective_sam_freq() == 0:
            try:
                metrics["sam_loss"] = self.sam_step(model, train_x, train_y, criterion)
            except Exception as e:  # noqa: BLE001
                warnings.warn(f"sam_step failed: {e}")
        if step_num % self._get_effective_bilevel_freq() == 0:
            try:
                metrics["val_loss"] = self.bilevel_step(model, train_x, train_y, val_x, val_y, criterion,
                                                        self._auto_meta_opt)
            except Exception as e:  # noqa: BLE001
                warnings.warn(f"bilevel_step failed: {e}")
        kw: Dict[str, float] = {}
        if step_num % self.alpha_update_freq == 0 or step_num == 1:
            with torch.no_grad():
                kw["train_loss"] = metrics["train_loss"] = float(loss.item())
                kw["train_acc"] = metrics["train_acc"] = float((logits.detach().argmax(-1) == train_y).float().mean().item())
                if step_num % self.alpha_update_freq == 0:
                    kw["val_loss"] = float(criterion(model(val_x), val_y).item())
                    metrics.setdefault("val_loss", kw["val_loss"])
        self.step(**kw)
        return metrics
