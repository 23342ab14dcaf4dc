"""Training loops of the race: ONE generic loop driven by per-optimizer specs.

The reference has eleven copy-pasted ``train_<optimizer>`` functions (grokking_race_v2.py:560-947).  Here a spec says how
to build the optimizer from the flat config and what extra work a step needs (SAM, bilevel, amplifier training, metrics);
the loop, evaluation schedule, early stopping and result record are shared.  ``OPTIMIZER_REGISTRY[name](c, init, tx, ty,
vx, vy, dev, bp)`` keeps the reference's call signature and registry keys.
"""
from __future__ import annotations

import copy
import math
import time
import warnings
from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import optim as O
from ..models import build_model as _build_model
from .config import DISPLAY_NAMES


class TrainResult:
    __slots__ = ("name", "seed", "steps", "train_losses", "train_accs", "val_losses", "val_accs", "wall_time", "total_steps",
                 "grokking_step", "grokking_wall", "final_val_acc", "final_train_acc", "model_type", "frac_train", "events",
                 "step_ms")

    def __init__(self, name, seed=42, model_type="decoder", frac_train=0.5):
        self.name, self.seed, self.model_type, self.frac_train = name, seed, model_type, frac_train
        self.steps, self.train_losses, self.train_accs, self.val_losses, self.val_accs = [], [], [], [], []
        self.wall_time, self.total_steps, self.grokking_step, self.grokking_wall = 0.0, 0, None, None
        self.final_val_acc, self.final_train_acc = 0.0, 0.0
        self.events: List[str] = []           # failures of SAM / bilevel sub-steps are recorded, not silenced
        self.step_ms: Optional[float] = None

    def to_dict(self) -> Dict:
        return {k: getattr(self, k) for k in ("seed", "steps", "train_losses", "train_accs", "val_losses", "val_accs", "wall_time",
                                              "total_steps", "grokking_step", "grokking_wall", "final_val_acc", "final_train_acc",
                                              "model_type", "frac_train", "events", "step_ms")}

    @classmethod
    def from_dict(cls, name: str, d: Dict) -> "TrainResult":
        r = cls(name, d.get("seed", 42), d.get("model_type", "decoder"), d.get("frac_train", 0.5))
        for k, v in d.items():
            if k in cls.__slots__:
                setattr(r, k, v)
        return r


class EarlyStopper:
    """Records the first evaluation with val_acc >= threshold; stops after `patience` consecutive qualifying evaluations."""

    def __init__(self, threshold=0.95, patience=500, max_steps=100_000):
        self.threshold, self.patience, self.max_steps = threshold, patience, max_steps
        self._triggered, self._counter, self.best_val_acc = False, 0, 0.0
        self.grokking_step, self.grokking_wall, self._t0 = None, None, time.time()

    def step(self, val_acc, current_step) -> bool:
        if current_step >= self.max_steps:
            return True
        self.best_val_acc = max(self.best_val_acc, val_acc)
        if val_acc >= self.threshold:
            if not self._triggered:
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
                self._triggered, self.grokking_step, self.grokking_wall = True, current_step, time.time() - self._t0
            self._counter += 1
            return self._counter >= self.patience
        self._counter = 0
        return False


@torch.no_grad()
def evaluate(model, x, y, p=97):
    logits = model(x).float()
    return F.cross_entropy(logits, y).item(), (logits[:, :p].argmax(-1) == y).float().mean().item()


def progressive_eval_freq(step, base_freq=10, max_freq=50, scale=0.01, thresh=500):
    heat = 1.0 / (1.0 + math.exp(-scale * (step - thresh)))
    return max(base_freq, round(max_freq - (max_freq - base_freq) * heat))


def build_model(c, device):
    return _build_model(c).to(device)


def get_init_state(c, device):
    torch.manual_seed(c["seed"])
    return copy.deepcopy(build_model(c, device).state_dict())


# ------------------------------------------------------------------------------------------------ optimizer specs
class Spec:
    """How one optimizer is built and what its step needs."""
    adaptive = False                      # SuperGrok v1.5 / v2: sigmoid-scheduled SAM / bilevel, metrics into step()

    def __init__(self, key):
        self.key = key

    def build(self, m, c, dev):
        raise NotImplementedError

    def after_backward(self, ctx, step, m, data, c, r):
        """Extra work between backward() and optimizer.step(); returns kwargs for step()."""
        return {}


def _betas(c):
    return (c["beta1"], c["beta2"])


class _AdamW(Spec):
    def build(self, m, c, dev):
        return {"opt": O.AdamW(m.parameters(), lr=c["lr"], betas=_betas(c), weight_decay=c["weight_decay"])}


class _GrokAdamW(Spec):
    def build(self, m, c, dev):
        return {"opt": O.GrokAdamW(m.parameters(), lr=c["lr"], betas=_betas(c), weight_decay=c["weight_decay"],
                                   alpha=c.get("grokadamw_alpha", 0.98), lamb=c.get("grokadamw_lamb", 5.0),
                                   gamma=c.get("grokadamw_gamma", 0.1), decay=c.get("grokadamw_decay", 0.1),
                                   grad_clip=c.get("grokadamw_grad_clip", 1.0))}


class _NeuralGrok(Spec):
    """Inner 90 % of the train split drives the model, the outer 10 % trains the amplifier (loss = beta * CE)."""

    def build(self, m, c, dev):
        opt = O.NeuralGrok(m.parameters(), lr=c["lr"], betas=_betas(c), weight_decay=c["weight_decay"],
                           alpha=c.get("neural_alpha", 10.0), beta=c.get("neural_beta", 4.0), num_layers=c.get("neural_layers", 3),
                           hidden_dim=c.get("neural_hidden", 128), inner_steps=c.get("inner_steps", 1),
                           grad_clip=c.get("neural_grad_clip", 1.0))
        opt.amplifier = opt.amplifier.to(dev)
        return {"opt": opt, "aopt": opt.get_amplifier_optimizer(lr=1e-3), "inner_split": True}

    def after_step(self, ctx, step, m, data, c, r):
        ox, oy = data["ox"], data["oy"]
        ctx["aopt"].zero_grad()
        aloss = c.get("neural_beta", 4.0) * F.cross_entropy(m(ox).float(), oy)
        aloss.backward()
        ctx["aopt"].step()
        if not c.get("reference_compat", False):
            ctx["opt"].mark_amplifier_dirty()      # the reference driver never refreshes the cached amplifier weights


class _SuperGrok11(Spec):
    def build(self, m, c, dev):
        opt = O.SuperGrok11(m.parameters(), lr=c["lr"], betas=_betas(c), weight_decay=c["weight_decay"],
                            alpha_init=c.get("supergrok_alpha", 0.98), lamb=c.get("supergrok_lamb", c.get("supergrok11_lamb", 5.0)),
                            gamma=c.get("supergrok_gamma", 0.1), kappa=c.get("supergrok_kappa", 0.1),
                            warmup_steps=c.get("supergrok_warmup", 100), warmup_ramp=c.get("supergrok_warmup_ramp", 100),
                            gradient_clipping=c.get("supergrok_grad_clip", 1.0), meta_hidden_dim=c.get("supergrok_meta_dim", 32),
                            gate_temperature=c.get("supergrok11_gate_temperature", 5.0),
                            alpha_update_freq=c.get("supergrok11_alpha_update_freq", 50),
                            meta_update_freq=c.get("supergrok_meta_update_freq", 5), reference_compat=c.get("reference_compat", False))
        opt.meta_net = opt.meta_net.to(dev)
        return {"opt": opt, "mopt": torch.optim.Adam(opt.meta_net.parameters(), lr=1e-4), "crit": nn.CrossEntropyLoss()}

    def after_backward(self, ctx, step, m, data, c, r):
        opt = ctx["opt"]
        if step % c.get("supergrok_meta_update_freq", 5) == 0:
            _guard(r, step, "meta_step", lambda: opt.meta_step(m, data["vx"], data["vy"], ctx["crit"], ctx["mopt"]))
        if step % c.get("supergrok11_sam_freq", 10) == 0:
            _guard(r, step, "sam_step", lambda: opt.sam_step(m, data["tx"], data["ty"], ctx["crit"]))
        return _metrics_kw(opt, step, m, data, c, c.get("supergrok11_alpha_update_freq", 50))


def _guard(r, step, what, fn):
    try:
        fn()
    except Exception as e:  # noqa: BLE001
        msg = f"{what} failed at step {step}: {type(e).__name__}: {str(e)[:120]}"
        if len(r.events) < 200:
            r.events.append(msg)
        warnings.warn(msg)


def _metrics_kw(opt, step, m, data, c, alpha_freq):
    eval_freq = progressive_eval_freq(step, base_freq=c["log_every"])
    if not ((step % alpha_freq == 0) or (step % eval_freq == 0) or step == 1):
        return {}
    kw = {}
    with torch.no_grad():
        kw["train_loss"] = float(data["loss"].item())
        kw["train_acc"] = float((data["logits"].detach()[:, :c["p"]].argmax(-1) == data["ty"]).float().mean().item())
        if step % alpha_freq == 0:
            kw["val_loss"] = float(F.cross_entropy(m(data["vx"]).float(), data["vy"]).item())
    return kw


class _SuperGrok15(Spec):
    adaptive = True
    prefix = "supergrok15"

    def _kwargs(self, c):
        g = lambda k, d: c.get(f"{self.prefix}_{k}", d)  # noqa: E731
        return dict(lr=c["lr"], betas=_betas(c), weight_decay=c["weight_decay"], alpha_init=g("alpha", 0.98), lamb=g("lamb", 2.0),
                    gamma=g("gamma", 0.1), kappa=g("kappa", 0.1), warmup_steps=g("warmup", 100), warmup_ramp=g("warmup_ramp", 100),
                    gradient_clipping=g("grad_clip", 1.0), alpha_update_freq=g("alpha_update_freq", 50),
                    zero_loss_threshold=g("zero_loss_thresh", 1e-4), zero_acc_threshold=g("zero_acc_thresh", 0.995),
                    sam_rho=g("sam_rho", 0.05), gate_scale=g("gate_scale", 20.0), gate_thresh=g("gate_thresh", 0.8),
                    sam_freq_min=g("sam_freq_min", 3), sam_freq_max=g("sam_freq_max", 20), sam_scale=g("sam_scale", 20.0),
                    sam_thresh=g("sam_thresh", 0.85), bilevel_freq_min=g("bilevel_freq_min", 5), bilevel_freq_max=g("bilevel_freq_max", 30),
                    bilevel_scale=g("bilevel_scale", 20.0), bilevel_thresh=g("bilevel_thresh", 0.9), wd_ramp=g("wd_ramp", 4.0),
                    wd_scale=g("wd_scale", 20.0), wd_thresh=g("wd_thresh", 0.9), reference_compat=c.get("reference_compat", False))

    def build(self, m, c, dev):
        opt = O.SuperGrok15(m.parameters(), meta_hidden_dim=c.get("supergrok15_meta_dim", 32), **self._kwargs(c))
        opt.meta_net = opt.meta_net.to(dev)
        return {"opt": opt, "mopt": torch.optim.Adam(opt.meta_net.parameters(), lr=1e-4), "crit": nn.CrossEntropyLoss()}

    def after_backward(self, ctx, step, m, data, c, r):
        opt = ctx["opt"]
        sf = opt._get_effective_sam_freq()
        if sf < 999999 and step % sf == 0:
            _guard(r, step, "sam_step", lambda: opt.sam_step(m, data["tx"], data["ty"], ctx["crit"]))
        if step % opt._get_effective_bilevel_freq() == 0:
            _guard(r, step, "bilevel_step", lambda: opt.bilevel_step(m, data["tx"], data["ty"], data["vx"], data["vy"], ctx["crit"], ctx["mopt"]))
        return _metrics_kw(opt, step, m, data, c, c.get(f"{self.prefix}_alpha_update_freq", 50))


class _SuperGrok2(_SuperGrok15):
    prefix = "sg2"

    def build(self, m, c, dev):
        opt = O.SuperGrok2(m.parameters(), expert_hidden=c.get("sg2_expert_hidden", 16), meta_rescale=c.get("sg2_meta_rescale", 0.1),
                           bilevel_checkpoint_interval=c.get("sg2_bilevel_checkpoint_interval", 1), **self._kwargs(c))
        opt.meta_net = opt.meta_net.to(dev)
        return {"opt": opt, "mopt": torch.optim.Adam(opt.meta_net.parameters(), lr=1e-4), "crit": nn.CrossEntropyLoss()}


class _Grokfast(Spec):
    def build(self, m, c, dev):
        return {"opt": O.Grokfast(m.parameters(), lr=c["lr"], betas=_betas(c), weight_decay=c["weight_decay"],
                                  grokfast_alpha=c.get("grokfast_alpha", 0.98), grokfast_lamb=c.get("grokfast_lamb", 2.0))}


class _Muon(Spec):
    def build(self, m, c, dev):
        p2 = [p for p in m.parameters() if p.dim() == 2]
        p1 = [p for p in m.parameters() if p.dim() != 2]
        return {"opt": O.Muon(p2, p1, lr=c.get("muon_lr", 0.02), momentum=c.get("muon_momentum", 0.95), weight_decay=c["weight_decay"],
                              adamw_lr=c["lr"], adamw_betas=_betas(c), ns_steps=c.get("muon_ns_steps", 5))}


class _Lion(Spec):
    def build(self, m, c, dev):
        return {"opt": O.Lion(m.parameters(), lr=c.get("lion_lr", 3e-4), betas=(c["beta1"], c.get("lion_beta2", 0.99)),
                              weight_decay=c.get("lion_wd", 3.0))}


class _LookSAM(Spec):
    def build(self, m, c, dev):
        return {"opt": O.LookSAM(m.parameters(), lr=c["lr"], betas=_betas(c), weight_decay=c["weight_decay"],
                                 rho=c.get("looksam_rho", 0.05), k=c.get("looksam_k", 5), alpha=c.get("looksam_alpha", 0.7)),
                "crit": nn.CrossEntropyLoss()}

    def after_backward(self, ctx, step, m, data, c, r):
        if ctx["opt"].should_sam_step():
            ctx["opt"].sam_step(m, data["tx"], data["ty"], ctx["crit"])
        return {}


class _Prodigy(Spec):
    def build(self, m, c, dev):
        return {"opt": O.Prodigy(m.parameters(), lr=c.get("prodigy_lr", 1.0), weight_decay=c["weight_decay"])}


SPECS: Dict[str, Spec] = {"adamw": _AdamW("adamw"), "grokadamw": _GrokAdamW("grokadamw"), "neuralgrok": _NeuralGrok("neuralgrok"),
                          "supergrok11": _SuperGrok11("supergrok11"), "supergrok15": _SuperGrok15("supergrok15"),
                          "supergrok2": _SuperGrok2("supergrok2"), "grokfast": _Grokfast("grokfast"), "muon": _Muon("muon"),
                          "lion": _Lion("lion"), "looksam": _LookSAM("looksam"), "prodigy": _Prodigy("prodigy")}


# ------------------------------------------------------------------------------------------------ the loop
def train(name: str, c: dict, init_state, tx, ty, vx, vy, dev, bp: int = 0, progress: Optional[Callable] = None) -> TrainResult:
    spec = SPECS[name]
    r = TrainResult(DISPLAY_NAMES.get(name, name), c["seed"], c.get("model_type", "decoder"), c.get("frac_train", 0.5))
    m = build_model(c, dev)
    m.load_state_dict(copy.deepcopy(init_state), strict=True)
    if c.get("compile_model", False) and hasattr(torch, "compile"):
        # the reference wraps the model in torch.compile when asked (grokking_race_v2.py:432-443, 540-546); the parameters stay
        # those of ``m`` (the optimizers hold them), a failed compilation keeps the eager module
        try:
            fwd = torch.compile(m, mode="reduce-overhead", fullgraph=False)
            with torch.no_grad():
                fwd(tx[:2])
            m.forward = fwd.forward if hasattr(fwd, "forward") else m.forward
        except Exception as exc:  # noqa: BLE001
            warnings.warn(f"torch.compile failed ({type(exc).__name__}); running the eager model")
    ctx = spec.build(m, c, dev)
    opt = ctx["opt"]
    if c.get("use_cuda_graph", False) and dev.type == "cuda" and not spec.adaptive:
        opt = O.CUDAGraphOptimizer(opt, warmup_steps=c.get("cuda_graph_warmup", 3), max_graph_age=c.get("cuda_graph_max_age", 1))
    use_amp = bool(c.get("use_amp", False)) and dev.type == "cuda"
    amp_dtype = torch.bfloat16 if c.get("amp_dtype", "bf16") == "bf16" else torch.float16
    scaler = torch.amp.GradScaler("cuda", enabled=use_amp and amp_dtype == torch.float16)
    data = {"tx": tx, "ty": ty, "vx": vx, "vy": vy}
    fx, fy = tx, ty
    if ctx.get("inner_split"):
        ni = int(tx.size(0) * 0.9)
        fx, fy = tx[:ni], ty[:ni]
        data.update(ox=tx[ni:], oy=ty[ni:])
    st = EarlyStopper(c["early_stop_threshold"], c["early_stop_patience"], c["max_steps"])
    m.train()
    t0 = time.time()
    step = 0
    for step in range(1, c["max_steps"] + 1):
        with torch.amp.autocast("cuda", enabled=use_amp, dtype=amp_dtype):
            logits = m(fx)
            loss = F.cross_entropy(logits.float(), fy)
        opt.zero_grad()
        scaler.scale(loss).backward()
        if scaler.is_enabled():
            scaler.unscale_(ctx["opt"])
            if any(p.grad is not None and not torch.isfinite(p.grad).all() for p in m.parameters()):
                scaler.update()                       # fp16 overflow: skip the step
                continue
        data["loss"], data["logits"] = loss, logits
        kw = spec.after_backward(ctx, step, m, data, c, r)
        try:
            opt.step(**kw)
        except TypeError:
            opt.step()
        scaler.update()
        if hasattr(spec, "after_step"):
            spec.after_step(ctx, step, m, data, c, r)
        eval_freq = progressive_eval_freq(step, base_freq=c["log_every"]) if spec.adaptive else c["log_every"]
        if step % eval_freq == 0 or step == 1:
            tl, ta = evaluate(m, tx, ty, c["p"])
            vl, va = evaluate(m, vx, vy, c["p"])
            r.steps.append(step); r.train_losses.append(tl); r.train_accs.append(ta); r.val_losses.append(vl); r.val_accs.append(va)
            if progress is not None:
                progress(name, c["seed"], step, ta, va, tl, vl)
            if st.step(va, step):
                break
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    r.wall_time, r.total_steps = time.time() - t0, step
    r.step_ms = 1e3 * r.wall_time / max(step, 1)
    r.grokking_step, r.grokking_wall = st.grokking_step, st.grokking_wall
    r.final_train_acc = r.train_accs[-1] if r.train_accs else 0.0
    r.final_val_acc = r.val_accs[-1] if r.val_accs else 0.0
    return r


def _make_train_fn(name):
    def fn(c, init, tx, ty, vx, vy, dev, bp=0, progress=None):
        return train(name, c, init, tx, ty, vx, vy, dev, bp, progress)
    fn.__name__ = f"train_{name}"
    return fn


OPTIMIZER_REGISTRY = {name: _make_train_fn(name) for name in SPECS}
# the reference registers SuperGrok v1.1 under "supergrok" (grokking_race_v2.py:940-947): accept that key too
OPTIMIZER_REGISTRY["supergrok"] = OPTIMIZER_REGISTRY["supergrok11"]
SPECS["supergrok"] = SPECS["supergrok11"]
