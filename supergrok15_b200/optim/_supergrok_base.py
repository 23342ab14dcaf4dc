"""Machinery shared by SuperGrok v1.1 / v1.5 / v2: flat fp32 state, schedules, SAM, state_dict.

Reference behaviour this file restates: grokking_optimizers/supergrok15.py:74-247 (constructor,
layer-wise beta1/alpha factors, sigmoid schedules), :307-352 (functional-call SAM).

Differences from the reference, all deliberate:
* The per-parameter tensors are kept in the reference's ``_flat_*`` lists AND mirrored under
  ``self.state[p]`` so ``state_dict()`` round-trips them (the reference's state_dict is empty).
  Scalars that the reference keeps as attributes travel in ``state_dict()["extra"]``.
* ``sam_step`` really computes ``sharpness = |g_sam - g|``.  In the reference every tensor given
  to ``functional_call`` is detached, so ``backward()`` raises, gradients are left ``None`` and
  the caller's next ``step()`` is skipped.  ``reference_compat=True`` reproduces exactly that
  (and, for v1.1/v1.5, the bias correction that stays at step 1 because the C++ step counter
  never reaches Python; reference csrc/ops.cpp:114, :237).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
from torch.optim import Optimizer


class SuperGrokBase(Optimizer):
    _STATE_KEYS = ("exp_avg", "exp_avg_sq", "mu", "sharpness")

    def _init_common(self, *, alpha_init, lamb, gamma, gamma_alpha, kappa, warmup_steps, warmup_ramp,
                     gradient_clipping, alpha_update_freq, zero_loss_threshold, zero_acc_threshold, sam_rho,
                     sam_enable_threshold, reference_compat):
        self.alpha_init, self.lamb, self.gamma, self.gamma_alpha, self.kappa = alpha_init, lamb, gamma, gamma_alpha, kappa
        self.warmup_steps, self.warmup_ramp = warmup_steps, max(1, warmup_ramp)
        self.gradient_clipping = gradient_clipping
        self.alpha_update_freq = alpha_update_freq
        self.zero_loss_threshold, self.zero_acc_threshold = zero_loss_threshold, zero_acc_threshold
        self.sam_rho, self.sam_enable_threshold = sam_rho, sam_enable_threshold
        self.reference_compat = bool(reference_compat)
        self._global_step = 0
        self._cached_alpha = alpha_init
        self._cached_train_acc = 0.0
        self._flat_params: List[torch.Tensor] = []
        self._flat_steps: List[int] = []
        self._flat_layer_alphas: List[float] = []
        self._flat_layer_beta1s: List[float] = []
        self._flat_exp_avgs: List[torch.Tensor] = []
        self._flat_exp_avg_sqs: List[torch.Tensor] = []
        self._flat_mus: List[torch.Tensor] = []
        self._flat_sharpness: List[torch.Tensor] = []
        self._param_to_idx: Dict[int, int] = {}
        num_params = sum(len(g["params"]) for g in self.param_groups)
        idx = 0
        for group in self.param_groups:
            beta1 = group["betas"][0]
            for p in group["params"]:
                self._flat_params.append(p)
                self._flat_steps.append(0)
                self._flat_layer_beta1s.append(beta1 * ((1.0 - gamma) ** idx))
                if gamma_alpha == 0.0:
                    self._flat_layer_alphas.append(1.0)
                else:
                    self._flat_layer_alphas.append((1.0 - gamma_alpha) ** (max(num_params - 1, 1) - idx))
                self._param_to_idx[id(p)] = idx
                idx += 1
        self._num_params = num_params
        self._state_initialized = False
        self._weights_dirty = True
        self._cached_weights = None

    # ------------------------------------------------------------------ state
    @property
    def _flat_param_data(self):
        return [p.data for p in self._flat_params]

    def _new_state(self, p) -> Dict[str, torch.Tensor]:
        z = lambda: torch.zeros(p.numel(), dtype=torch.float32, device=p.device)  # noqa: E731
        return {"exp_avg": z(), "exp_avg_sq": z(), "mu": z(), "sharpness": z()}

    def _ensure_state(self):
        if self._state_initialized:
            return
        for p in self._flat_params:
            st = self.state[p]
            for k, v in self._new_state(p).items():
                st.setdefault(k, v)
            st.setdefault("step", 0)
        self._relink()
        self._state_initialized = True

    def _relink(self):
        """Rebuild the ``_flat_*`` lists from ``self.state`` (same tensor objects)."""
        self._flat_exp_avgs = [self.state[p]["exp_avg"] for p in self._flat_params]
        self._flat_exp_avg_sqs = [self.state[p]["exp_avg_sq"] for p in self._flat_params]
        self._flat_mus = [self.state[p]["mu"] for p in self._flat_params]
        self._flat_sharpness = [self.state[p]["sharpness"] for p in self._flat_params]

    def _sync_steps_to_state(self):
        for p, s in zip(self._flat_params, self._flat_steps):
            self.state[p]["step"] = s

    # ------------------------------------------------------------------ schedules
    @staticmethod
    def _sigmoid(scale, value, thresh):
        return 1.0 / (1.0 + math.exp(-scale * (value - thresh)))

    def _update_alpha(self, train_loss, val_loss, train_acc):
        if train_loss is None and train_acc is None:
            return
        signal = 0.0
        memorized = (train_acc is not None and train_acc >= self.zero_acc_threshold) or \
                    (train_loss is not None and train_loss < self.zero_loss_threshold)
        if memorized:
            signal = 10.0
        elif val_loss is not None and train_loss is not None and train_loss > 1e-12:
            signal = max(0.0, (val_loss - train_loss) / train_loss)
        self._cached_alpha = self.alpha_init * math.exp(-self.kappa * signal)

    def _get_ramp_factor(self):
        if self._global_step <= self.warmup_steps:
            return 0.0
        return min(1.0, (self._global_step - self.warmup_steps) / self.warmup_ramp)

    def get_global_step(self):
        return self._global_step

    def get_cached_alpha(self):
        return self._cached_alpha

    # ------------------------------------------------------------------ SAM
    def sam_step(self, model, train_x, train_y, criterion):
        """Sharpness = |grad(p + rho*g/||g||) - g| via ``torch.func.functional_call``; parameters are
        never modified and ``p.grad`` is restored.  Returns the loss at the perturbed point."""
        self._ensure_state()
        named = list(model.named_parameters())
        train_grads = {n: p.grad.detach().clone() for n, p in named if p.grad is not None}
        if not train_grads:
            return 0.0
        if self.reference_compat:
            # literal reference behaviour: the perturbed tensors do not require grad, backward() raises
            # after zero_grad(), gradients stay None and the restore loop is never reached
            model.zero_grad()
            raise RuntimeError("element 0 of tensors does not require grad and does not have a grad_fn")
        sq = None
        for g in train_grads.values():
            if g.numel():
                t = g.float().pow(2).sum()
                sq = t if sq is None else sq + t
        scale = self.sam_rho / (sq.sqrt() + 1e-12)
        perturbed = {}
        for n, p in named:
            if n in train_grads:
                perturbed[n] = (p.detach() + (scale * train_grads[n]).to(p.dtype)).requires_grad_(True)
            else:
                perturbed[n] = p.detach()
        try:
            with torch.enable_grad():
                loss = criterion(torch.func.functional_call(model, perturbed, (train_x,)), train_y)
                names = list(train_grads.keys())
                sam_grads = torch.autograd.grad(loss, [perturbed[n] for n in names], allow_unused=True)
            with torch.no_grad():
                pmap = dict(named)
                for n, gs in zip(names, sam_grads):
                    pidx = self._param_to_idx.get(id(pmap[n]))
                    if pidx is None or gs is None:
                        continue
                    self._flat_sharpness[pidx].copy_((gs.detach().float() - train_grads[n].float()).abs().reshape(-1))
            return float(loss.item())
        finally:
            for n, p in named:
                p.grad = train_grads.get(n)

    # ------------------------------------------------------------------ state_dict
    def _extra_state(self) -> dict:
        return {"global_step": self._global_step, "cached_alpha": self._cached_alpha,
                "cached_train_acc": self._cached_train_acc, "flat_steps": list(self._flat_steps),
                "meta_net": {k: v.detach().cpu() for k, v in self.meta_net.state_dict().items()}}

    def _load_extra_state(self, extra: dict) -> None:
        self._global_step = int(extra.get("global_step", 0))
        self._cached_alpha = float(extra.get("cached_alpha", self.alpha_init))
        self._cached_train_acc = float(extra.get("cached_train_acc", 0.0))
        fs = extra.get("flat_steps")
        if fs is not None and len(fs) == len(self._flat_steps):
            self._flat_steps = [int(s) for s in fs]
        if "meta_net" in extra:
            self.meta_net.load_state_dict(extra["meta_net"])
            self._weights_dirty = True

    def state_dict(self):
        if self._state_initialized:
            self._sync_steps_to_state()
        sd = super().state_dict()
        sd["extra"] = self._extra_state()
        return sd

    def load_state_dict(self, state_dict):
        extra = state_dict.get("extra")
        super().load_state_dict({k: v for k, v in state_dict.items() if k != "extra"})
        if state_dict.get("state"):
            for p in self._flat_params:         # torch casts loaded state to the parameter dtype: undo
                st = self.state[p]
                for k, v in list(st.items()):
                    if torch.is_tensor(v) and v.is_floating_point() and v.dtype != torch.float32:
                        st[k] = v.float()
                for k, v in self._new_state(p).items():
                    st.setdefault(k, v)
                if "step" in st:
                    self._flat_steps[self._param_to_idx[id(p)]] = int(st["step"])
            self._relink()
            self._state_initialized = True
        if extra:
            self._load_extra_state(extra)
