"""SuperGrok v2: AdamW whose gradient is rewritten by the Mamba-3 + PEER + GRU meta-network
(reference grokking_optimizers/supergrok2.py:49-1438).

Per step and per tensor: per-tensor clip and NaN scrub -> sort by |g| -> input projection ->
forward and reverse selective scans (states persist across optimizer steps) -> un-sort ->
per-element GRU -> 4-head product-key routing (top-1) over 144 tiny experts ->
smart = g + rescale*mean_heads -> mu EMA -> Adam with progressive weight decay.
On CUDA the whole list of tensors goes through one batched pipeline of sm_100a kernels
(``ops/sg2.py``); nothing is copied to the host during a step.

``bilevel_step`` trains the meta-net on validation gradients with soft top-4 routing; gradients of
the meta-net parameters are exact (autograd of the differentiable forward).
"""
from __future__ import annotations

import warnings
from typing import Dict, Optional

import torch
import torch.nn as nn

from ..ops import sg2 as sg2_ops
from ._common import run_closure
from .metanet import Mamba3PEERMetaNet
from .supergrok15 import SuperGrok15


class SuperGrok2(SuperGrok15):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1.0, alpha_init=0.98, lamb=2.0,
                 gamma=0.1, gamma_alpha=0.0, kappa=0.1, warmup_steps=100, warmup_ramp=100, gradient_clipping=1.0,
                 meta_net: Optional[nn.Module] = None, d_model=8, d_state=16, mamba_expand=2, num_peer_heads=4,
                 num_experts=144, expert_hidden=16, gru_hidden=4, meta_rescale=0.1, recycle_interval=100,
                 recycle_threshold=0.001, alpha_update_freq=100, zero_loss_threshold=1e-4, zero_acc_threshold=0.995,
                 sam_rho=0.05, gate_scale=20.0, gate_thresh=0.8, sam_freq_min=3, sam_freq_max=20, sam_scale=20.0,
                 sam_thresh=0.85, bilevel_freq_min=5, bilevel_freq_max=30, bilevel_scale=20.0, bilevel_thresh=0.9,
                 wd_ramp=4.0, wd_scale=20.0, wd_thresh=0.9, sam_enable_threshold=0.0, bilevel_checkpoint_interval=1,
                 reference_compat=False, recycle_seed: int = 0):
        if meta_net is None:
            meta_net = Mamba3PEERMetaNet(d_model=d_model, d_state=d_state, mamba_expand=mamba_expand,
                                         num_peer_heads=num_peer_heads, num_experts=num_experts,
                                         expert_hidden=expert_hidden, gru_hidden=gru_hidden, rescale=meta_rescale,
                                         recycle_interval=recycle_interval, recycle_threshold=recycle_threshold)
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, alpha_init=alpha_init,
                         lamb=lamb, gamma=gamma, gamma_alpha=gamma_alpha, kappa=kappa, warmup_steps=warmup_steps,
                         warmup_ramp=warmup_ramp, gradient_clipping=gradient_clipping, meta_net=meta_net,
                         alpha_update_freq=alpha_update_freq, zero_loss_threshold=zero_loss_threshold,
                         zero_acc_threshold=zero_acc_threshold, sam_rho=sam_rho, gate_scale=gate_scale,
                         gate_thresh=gate_thresh, sam_freq_min=sam_freq_min, sam_freq_max=sam_freq_max,
                         sam_scale=sam_scale, sam_thresh=sam_thresh, bilevel_freq_min=bilevel_freq_min,
                         bilevel_freq_max=bilevel_freq_max, bilevel_scale=bilevel_scale, bilevel_thresh=bilevel_thresh,
                         wd_ramp=wd_ramp, wd_scale=wd_scale, wd_thresh=wd_thresh,
                         sam_enable_threshold=sam_enable_threshold, reference_compat=reference_compat)
        self.d_model, self.d_state = d_model, d_state
        self.num_experts, self.expert_hidden, self.gru_hidden = num_experts, expert_hidden, gru_hidden
        self.meta_rescale = meta_rescale
        self.bilevel_checkpoint_interval = max(1, bilevel_checkpoint_interval)
        self._step_counter = 0
        self._flat_gru_states, self._flat_mamba_fwd_states, self._flat_mamba_bwd_states = [], [], []
        # recycling draws come from a private CPU generator so every data-parallel rank makes the same choice
        self._recycle_gen = torch.Generator(device="cpu")
        self._recycle_gen.manual_seed(recycle_seed)
        self._recycle_seed, self._recycle_calls, self._recycle_info = recycle_seed, 0, None
        self._native_plan = None

    # ------------------------------------------------------------------ state
    def _new_state(self, p):
        st = super()._new_state(p)
        di, ds = self.meta_net.mamba_fwd.d_inner, self.meta_net.d_state
        st["gru_state"] = torch.zeros(p.numel(), self.meta_net.gru_hidden, dtype=torch.float32, device=p.device)
        st["mamba_fwd_state"] = torch.zeros(di, ds, dtype=torch.float32, device=p.device)
        st["mamba_bwd_state"] = torch.zeros(di, ds, dtype=torch.float32, device=p.device)
        return st

    def _relink(self):
        super()._relink()
        self._flat_gru_states = [self.state[p]["gru_state"] for p in self._flat_params]
        self._flat_mamba_fwd_states = [self.state[p]["mamba_fwd_state"] for p in self._flat_params]
        self._flat_mamba_bwd_states = [self.state[p]["mamba_bwd_state"] for p in self._flat_params]
        self._native_plan = None

    # ------------------------------------------------------------------ step
    def _prepare_step(self, train_loss=None, val_loss=None, train_acc=None):
        """Host side of a step: schedules, step counters and the scalars every tensor needs.  Returns
        ``(idx, per, hyper)``: the tensors that take part, ``per[k] = (alpha, lamb_eff, beta1, bc1, bc2)`` and the keyword
        arguments of ``ops.sg2.step``.  The tensor lists are cached: they only change when gradients appear or disappear."""
        self._ensure_state()
        self._schedule_tick(train_loss, val_loss, train_acc)
        ramp, gate = self._get_ramp_factor(), self._get_gate_signal()
        group = self.param_groups[0]
        lr, beta2, eps = group["lr"], group["betas"][1], group["eps"]
        wd_eff = self._get_effective_wd(group["weight_decay"])
        lamb_eff = self.lamb * ramp * gate
        ext = getattr(self, "_grad_override", None) is not None or getattr(self, "_pull_grads", None) is not None
        if ext:                                            # the ZeRO engine hands in gradients for every tensor, every step
            idx = getattr(self, "_all_idx", None)
            if idx is None or len(idx) != sum(1 for p in self._flat_params if p.numel() > 0):
                self._all_idx = idx = [i for i, p in enumerate(self._flat_params) if p.numel() > 0]
        else:
            idx = [i for i, p in enumerate(self._flat_params) if p.numel() > 0 and p.grad is not None]
        per = []
        ca, steps, b1s, las = self._cached_alpha, self._flat_steps, self._flat_layer_beta1s, self._flat_layer_alphas
        for i in idx:
            steps[i] += 1
            s = steps[i]
            b1 = b1s[i]
            a = max(0.0, min(1.0, ca * las[i]))
            per.append((a, lamb_eff, b1, 1.0 - b1 ** s, 1.0 - beta2 ** s))
        return idx, per, dict(beta2=beta2, lr=lr, wd_eff=wd_eff, eps=eps, clip=self.gradient_clipping)

    def _after_step(self):
        self._step_counter += 1
        ri = self.meta_net.recycle_interval
        if ri > 0 and self._step_counter % ri == 0 and not getattr(self, "_external_recycle", False):
            self.recycle_dead_experts()

    @torch.no_grad()
    def step(self, closure=None, train_loss=None, val_loss=None, train_acc=None):
        loss = run_closure(closure)
        idx, per, hyper = self._prepare_step(train_loss, val_loss, train_acc)
        if not idx:
            return loss
        sg2_ops.step(self, idx, per, **hyper)
        self._after_step()
        return loss

    def recycle_dead_experts(self):
        """Expert recycling (reference mamba3_peer_metanet.py:437-491).  On CUDA the whole decision runs in one device kernel
        (Philox keyed by the recycle seed and the call number: identical on every data-parallel rank, no host read-back);
        on CPU a private generator makes the draw reproducible."""
        mn = self.meta_net
        # the device kernel is built for the default expert width (16 hidden units); other widths (the race driver's
        # expert_hidden = 4) take the seeded host routine, which reads the counts back once per recycle_interval steps
        if mn.expert_counts.is_cuda and mn.expert_hidden == 16 and mn.num_experts == 144:
            from .. import _build
            C = _build.require()
            self._recycle_calls = getattr(self, "_recycle_calls", 0) + 1
            if getattr(self, "_recycle_info", None) is None:
                self._recycle_info = torch.zeros(2, dtype=torch.int32, device=mn.expert_counts.device)
            # the parameters keep their shapes ([144,16,1], [144,16], [144,1,16], [144,1]); the kernel sees them as flat rows
            C.sg2_recycle(mn.expert_counts, mn.expert_W1.data.view(-1), mn.expert_b1.data.view(-1), mn.expert_W2.data.view(-1),
                          mn.expert_b2.data.view(-1), [k.data for k in mn.product_keys_A], [k.data for k in mn.product_keys_B],
                          float(mn.recycle_threshold), int(self._recycle_seed), int(self._recycle_calls), self._recycle_info)
        else:
            mn._recycle_dead_experts(generator=self._recycle_gen)
        self._weights_dirty = True

    # ------------------------------------------------------------------ bilevel
    def bilevel_step(self, model, train_x, train_y, val_x, val_y, criterion, meta_optimizer):
        """meta_loss = -sum_tensors <smart_grad, vg/||vg||> through the soft top-4 routed meta-net
        (reference supergrok2.py:516-1330); tensors with non-finite validation gradients are skipped."""
        self._ensure_state()
        named = list(model.named_parameters())
        saved = {n: p.grad.detach().clone() for n, p in named if p.grad is not None}
        if not saved:
            return 0.0
        try:
            model.zero_grad()
            with torch.enable_grad():
                val_loss = criterion(model(val_x), val_y)
                val_loss.backward()
            vgs = {n: p.grad.detach().clone() for n, p in named if p.grad is not None}
            meta_optimizer.zero_grad()
            n_used = sg2_ops.bilevel_backward(self, named, saved, vgs, self.bilevel_checkpoint_interval)
            if n_used:
                meta_optimizer.step()
                self._weights_dirty = True
            return float(val_loss.item())
        finally:
            for n, p in named:
                p.grad = saved.get(n)

    def _bilevel_step_python(self, *a, **k):
        return self.bilevel_step(*a, **k)

    # ------------------------------------------------------------------ state_dict
    def _extra_state(self):
        ex = super()._extra_state()
        ex["step_counter"] = self._step_counter
        ex["recycle_rng"] = self._recycle_gen.get_state()
        ex["recycle_calls"] = self._recycle_calls
        return ex

    def _load_extra_state(self, extra):
        super()._load_extra_state(extra)
        self._step_counter = int(extra.get("step_counter", 0))
        self._recycle_calls = int(extra.get("recycle_calls", 0))
        if "recycle_rng" in extra:
            self._recycle_gen.set_state(extra["recycle_rng"])
