"""The reference's native entry points, by name and argument order, on top of this package's multi-tensor kernels.

The reference binds 22 functions in its extension module ``grokking_optimizers._ops`` (reference csrc/ops.cpp:897-1087); code and
tests written against it call e.g. ``_ops.lion_fused_step(params, grads, exp_avgs, lr, beta1, beta2, wd)``.  Every function
here takes the reference's arguments, in the reference's order and under the reference's keyword names, and forwards to the
multi-tensor launchers of ``ops/elementwise.py`` / ``ops/muon.py`` / ``ops/sg2.py`` (one launch per group of tensors instead of
one per tensor, global reductions finished on the device instead of with ``.item()``).  ``module()`` returns an object that
resolves these names first and falls back to the attributes of the native extension, so it can stand in for ``_ops``.

Differences that remain visible to a caller, by design:
* ``steps`` lists: the reference's C++ increments a COPY of the Python list (so Python never sees it and the bias
  correction stays at step 1, reference csrc/ops.cpp:114, :237); here ``supergrok15_fused_step`` / ``supergrok11_fused_step``
  take the steps as given plus one and do not write them back either: same visible behaviour.
* the four ``supergrok2_bilevel_*`` launchers work on packed buffers whose layout is private to the reference's Python
  ``bilevel_step`` (reference grokking_optimizers/supergrok2.py:646-1003); they are provided as names that raise with a pointer
  to ``SuperGrok2.bilevel_step`` / ``ops.sg2.bilevel_backward``, which compute the same gradients (exactly, including the
  cross-column terms the reference kernel drops).
"""
from __future__ import annotations

import types
from typing import List, Sequence

import torch

from .. import _build
from . import elementwise as ew
from . import muon as muon_ops


def _flat(ts: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    return [t.detach() if t.requires_grad else t for t in ts]


# ------------------------------------------------------------------------------------------------ SuperGrok v1.5 / v1.1
def supergrok15_fused_step(params, grads, exp_avgs, exp_avg_sqs, mus, sharpness_cache, steps, layer_alphas, layer_beta1s, W1, b1, W2,
                           b2, rescale, hidden_dim, beta2, lr, wd_eff, eps, lamb, ramp, gate_signal, grad_clip_norm):
    """Reference csrc/ops.cpp:83-152: global clip, lambda_eff = ramp * gate * lamb, then mu EMA + meta-net + Adam + weight decay."""
    keep = [i for i, g in enumerate(grads) if g is not None]
    pick = lambda xs: [xs[i] for i in keep]  # noqa: E731
    ew.sg15(_flat(pick(params)), pick(grads), pick(exp_avgs), pick(exp_avg_sqs), pick(mus), pick(sharpness_cache),
            [int(steps[i]) + 1 for i in keep], pick(layer_alphas), pick(layer_beta1s), W1, b1, W2, b2, float(rescale), beta2, lr,
            wd_eff, eps, lamb, ramp, gate_signal, grad_clip_norm)


def supergrok11_fused_step(params, grads, exp_avgs, exp_avg_sqs, mus, sharpness_cache, steps, layer_alphas, layer_beta1s, W1, b1, W2,
                           b2, rescale, hidden_dim, beta2, lr, wd_eff, eps, lamb, ramp, gate_temperature, grad_clip_norm):
    """Reference csrc/ops.cpp:211-291 (per-tensor cosine gate between the two kernels, here finished on the device)."""
    keep = [i for i, g in enumerate(grads) if g is not None]
    pick = lambda xs: [xs[i] for i in keep]  # noqa: E731
    ew.sg11(_flat(pick(params)), pick(grads), pick(exp_avgs), pick(exp_avg_sqs), pick(mus), pick(sharpness_cache),
            [int(steps[i]) + 1 for i in keep], pick(layer_alphas), pick(layer_beta1s), W1, b1, W2, b2, float(rescale), beta2, lr,
            wd_eff, eps, lamb, ramp, gate_temperature, grad_clip_norm)


def supergrok15_sam_perturb_all(params, grads, rho):
    """Returns the backups (clones of the parameters) after p += rho / ||g|| * g (reference csrc/ops.cpp:154-176)."""
    ps = _flat(params)
    backups = [torch.empty(p.numel(), dtype=torch.float32, device=p.device) for p in ps]
    ew.perturb(ps, list(grads), backups, rho)
    return backups


def supergrok15_sharpness_restore_all(params, sharpness_cache, backups, sam_grads, normal_grads):
    """sharpness = |g_sam - g|, parameters restored from the backups (reference csrc/ops.cpp:178-204)."""
    ew.sharpness_restore(_flat(params), list(normal_grads), list(backups), list(sam_grads), list(sharpness_cache))


supergrok11_sam_perturb_all = supergrok15_sam_perturb_all                 # the reference delegates too (csrc/ops.cpp:293-310)
supergrok11_sharpness_restore_all = supergrok15_sharpness_restore_all


# ------------------------------------------------------------------------------------------------ element-wise optimizers
def grokadamw_fused_step(params, grads, exp_avgs, exp_avg_sqs, emas, steps, alpha, lamb, beta1, beta2, lr, wd, eps, grad_clip_norm):
    ew.grokadamw(_flat(params), list(grads), list(exp_avgs), list(exp_avg_sqs), list(emas), [int(s) for s in steps], lr, beta1, beta2,
                 eps, wd, alpha, lamb, grad_clip_norm)


def neuralgrok_fused_step(params, grads, exp_avgs, exp_avg_sqs, steps, W1, b1, W2, b2, alpha_amp, beta_amp, hidden_dim, beta1, beta2,
                          lr, wd, eps, grad_clip_norm):
    ew.neuralgrok(_flat(params), list(grads), list(exp_avgs), list(exp_avg_sqs), [int(s) for s in steps], W1, b1, W2, b2, alpha_amp,
                  beta_amp, lr, beta1, beta2, eps, wd, grad_clip_norm)


def prodigy_fused_step(params, grads, exp_avgs, exp_avg_sqs, s_bufs, param_inits, steps, d_lr, beta1, beta2, lr, wd, eps):
    """Returns the new distance estimate as a float, as the reference does (csrc/ops.cpp:425-507); this read is the one
    host synchronisation of the adapter (``optim.Prodigy`` keeps the estimate on the device and never reads it back)."""
    ps = _flat(params)
    if ps[0].is_cuda:
        d = torch.tensor([float(d_lr)], dtype=torch.float32, device=ps[0].device)
        ew.prodigy_dlr(ps, list(grads), list(s_bufs), list(param_inits), d, float(d_lr))
        ew.prodigy_step(ps, list(grads), list(exp_avgs), list(exp_avg_sqs), list(s_bufs), [int(s) for s in steps], d, lr, beta1, beta2,
                        eps, wd)
        return float(d.item())
    d = ew.prodigy_dlr(ps, list(grads), list(s_bufs), list(param_inits), None, float(d_lr))
    ew.prodigy_step(ps, list(grads), list(exp_avgs), list(exp_avg_sqs), list(s_bufs), [int(s) for s in steps], d, lr, beta1, beta2, eps, wd)
    return float(d)


def grokfast_fused_step(grads, ema_bufs, alpha, lamb):
    ew.grokfast_ema(list(grads), list(ema_bufs), alpha, lamb)


def lion_fused_step(params, grads, exp_avgs, lr, beta1, beta2, wd):
    ew.lion(_flat(params), list(grads), list(exp_avgs), lr, beta1, beta2, wd)


# ------------------------------------------------------------------------------------------------ LookSAM
def looksam_perturb_all(params, grads, rho):
    ps = _flat(params)
    backups = [torch.empty(p.numel(), dtype=torch.float32, device=p.device) for p in ps]
    ew.perturb(ps, list(grads), backups, rho)
    return backups


def looksam_restore_all(params, backups):
    ew.restore(_flat(params), list(backups))


def looksam_compute_directions(v_dirs, sam_grads, normal_grads):
    """v = (g_sam - g) / ||g_sam - g|| per tensor, written in place (reference csrc/ops.cpp:606-632)."""
    from . import oracle
    if not v_dirs[0].is_cuda:
        return oracle.looksam_direction_(list(v_dirs), list(sam_grads), list(normal_grads))
    C = _build.require()
    n, dev = len(v_dirs), v_dirs[0].device
    pt = ew._reduce("OP_DIFF_SQNORM", [[], list(normal_grads), list(sam_grads)], n, dev, "looksam")
    norms = ew.workspace(dev, "looksam_norms", 2 * n)
    C.scalar_finalize(ew._op("SC_LOOKSAM_NORMS"), pt, n, norms, 0.0, 0.0, 0.0)
    C.mt_apply(ew._op("OP_LOOKSAM_DIR"), [[], list(normal_grads), list(v_dirs), list(sam_grads)], [], [], tscal=norms)


def looksam_adjust_grads(grads, v_dirs, la):
    """g += la * ||g|| * v per tensor (reference csrc/ops.cpp:634-656)."""
    ew.looksam_direction_adjust(list(grads), [], list(v_dirs), la, do_direction=False)


# ------------------------------------------------------------------------------------------------ Muon
def muon_fused_step(params, grads, bufs, momentum, lr, wd, ns_steps):
    for p in params:
        if p.dim() != 2:
            raise RuntimeError("self must be a matrix")                      # the reference's torch::mm says the same
    muon_ops.muon_step(_flat(params), list(grads), list(bufs), lr, momentum, wd, int(ns_steps))


# ------------------------------------------------------------------------------------------------ SuperGrok v2
_V2_WEIGHTS = ("input_proj_W", "input_proj_b", "mamba_fwd_in_proj", "mamba_fwd_dt_W", "mamba_fwd_dt_b", "mamba_fwd_B_proj",
               "mamba_fwd_C_proj", "mamba_fwd_A_log", "mamba_fwd_D", "mamba_fwd_rope", "mamba_fwd_out_proj", "mamba_bwd_in_proj",
               "mamba_bwd_dt_W", "mamba_bwd_dt_b", "mamba_bwd_B_proj", "mamba_bwd_C_proj", "mamba_bwd_A_log", "mamba_bwd_D",
               "mamba_bwd_rope", "mamba_bwd_out_proj", "gru_Wz", "gru_bz", "gru_Wr", "gru_br", "gru_Wh", "gru_bh", "peer_query_Ws",
               "prod_keys_A", "prod_keys_B", "expert_W1", "expert_b1", "expert_W2", "expert_b2")


class _V2Shell:
    """The minimum of a SuperGrok2 object that ``ops.sg2.launch`` reads, built from explicit tensors (no optimizer instance)."""


def _v2_pack(w: dict, dev, expert_hidden: int) -> torch.Tensor:
    """Explicit meta-net weight tensors (the reference's argument list) -> the packed vector of csrc/sg_native.h: SG2Pack."""
    from ..optim.metanet import Mamba3PEERMetaNet
    from . import sg2
    mn = Mamba3PEERMetaNet(expert_hidden=int(expert_hidden))
    with torch.no_grad():
        mn.input_proj.weight.copy_(w["input_proj_W"].reshape(8, 2)); mn.input_proj.bias.copy_(w["input_proj_b"].reshape(8))
        for tag, blk in (("fwd", mn.mamba_fwd), ("bwd", mn.mamba_bwd)):
            blk.in_proj.weight.copy_(w[f"mamba_{tag}_in_proj"].reshape(32, 8)); blk.dt_proj.weight.copy_(w[f"mamba_{tag}_dt_W"].reshape(16, 16))
            blk.dt_proj.bias.copy_(w[f"mamba_{tag}_dt_b"].reshape(16)); blk.B_proj.weight.copy_(w[f"mamba_{tag}_B_proj"].reshape(16, 16))
            blk.C_proj.weight.copy_(w[f"mamba_{tag}_C_proj"].reshape(16, 16)); blk.A_log.copy_(w[f"mamba_{tag}_A_log"].reshape(16, 16))
            blk.D.copy_(w[f"mamba_{tag}_D"].reshape(16)); blk.rope_freq.copy_(w[f"mamba_{tag}_rope"].reshape(16, 8))
            blk.out_proj.weight.copy_(w[f"mamba_{tag}_out_proj"].reshape(8, 16))
        for name, lin in (("z", mn.gru.W_z), ("r", mn.gru.W_r), ("h", mn.gru.W_h)):
            lin.weight.copy_(w[f"gru_W{name}"].reshape(4, 22)); lin.bias.copy_(w[f"gru_b{name}"].reshape(4))
        pq, ka, kb = w["peer_query_Ws"].reshape(4, 8, 22), w["prod_keys_A"].reshape(4, 12, 4), w["prod_keys_B"].reshape(4, 12, 4)
        for h in range(4):
            mn.peer_queries[h].weight.copy_(pq[h]); mn.product_keys_A[h].copy_(ka[h]); mn.product_keys_B[h].copy_(kb[h])
        mn.expert_W1.copy_(w["expert_W1"].reshape(mn.expert_W1.shape)); mn.expert_b1.copy_(w["expert_b1"].reshape(mn.expert_b1.shape))
        mn.expert_W2.copy_(w["expert_W2"].reshape(mn.expert_W2.shape)); mn.expert_b2.copy_(w["expert_b2"].reshape(mn.expert_b2.shape))
    return sg2.pack_metanet(mn).to(dev), mn


def supergrok2_mamba_peer_batched_step(params, grads, sharpness_list, exp_avgs, exp_avg_sqs, mus, gru_states, mamba_fwd_states,
                                       mamba_bwd_states, *weights_and_scalars, **kw):
    """Reference csrc/ops.cpp:815-877: one v2 update of all tensors.  Positional arguments after ``mamba_bwd_states`` follow the
    reference: the 33 meta-net weight tensors, then alpha_mus, lamb_effs, beta1s, bc1s, bc2s (one per tensor), rescale, beta2, lr,
    wd_eff, eps, d_model, d_state, d_inner, gru_hidden, num_heads, pk_dim, expert_hidden, num_experts, expert_counts.
    The gradients are taken as given (the reference clips them in Python beforehand)."""
    from . import sg2
    names = list(_V2_WEIGHTS) + ["alpha_mus", "lamb_effs", "beta1s", "bc1s", "bc2s", "rescale", "beta2", "lr", "wd_eff", "eps", "d_model",
                                 "d_state", "d_inner", "gru_hidden", "num_heads", "pk_dim", "expert_hidden", "num_experts", "expert_counts"]
    a = dict(zip(names, weights_and_scalars))
    a.update(kw)
    missing = [n for n in names if n not in a]
    if missing:
        raise TypeError(f"supergrok2_mamba_peer_batched_step: missing arguments {missing}")
    if not params[0].is_cuda:
        raise RuntimeError("supergrok2_mamba_peer_batched_step requires CUDA tensors")   # as in the reference (csrc/ops.cpp:753-877)
    if (a["d_model"], a["d_state"], a["d_inner"], a["gru_hidden"], a["num_heads"], a["pk_dim"], a["num_experts"]) != (8, 16, 16, 4, 4, 12, 144):
        raise ValueError("the fused v2 kernels are built for d_model 8, d_state 16, d_inner 16, GRU 4, 4 heads, 12 x 12 experts")
    dev = params[0].device
    packed, mn = _v2_pack({k: a[k] for k in _V2_WEIGHTS}, dev, a["expert_hidden"])
    sh = _V2Shell()
    sh._flat_params = _flat(params)
    sh._flat_sharpness, sh._flat_exp_avgs, sh._flat_exp_avg_sqs, sh._flat_mus = list(sharpness_list), list(exp_avgs), list(exp_avg_sqs), list(mus)
    sh._flat_gru_states, sh._flat_mamba_fwd_states, sh._flat_mamba_bwd_states = list(gru_states), list(mamba_fwd_states), list(mamba_bwd_states)
    sh._grad_override = [g.reshape(-1) for g in grads]
    sh._packed_w, sh._weights_dirty, sh._native_plan = packed, False, None
    mn.rescale = float(a["rescale"])
    mn.expert_counts = a["expert_counts"] if a["expert_counts"] is not None else mn.expert_counts.to(dev)
    sh.meta_net = mn
    C = _build.require()
    C.sg2_upload_weights(packed)
    sg2._resident["owner"] = sh
    idx = list(range(len(params)))
    per = [(float(al), float(le), float(b1), float(c1), float(c2))
           for al, le, b1, c1, c2 in zip(a["alpha_mus"], a["lamb_effs"], a["beta1s"], a["bc1s"], a["bc2s"])]
    sg2.write_scalars(sh, per, lr=float(a["lr"]), wd_eff=float(a["wd_eff"]), dev=dev)
    sg2.launch(sh, idx, beta2=float(a["beta2"]), eps=float(a["eps"]), clip=1e30)
    sg2._resident["owner"] = None


def supergrok2_mamba_peer_step(param, grad, sharpness, exp_avg, exp_avg_sq, mu, gru_state, mamba_fwd_state, mamba_bwd_state, *rest, **kw):
    """Reference csrc/ops.cpp:753-813: the single-tensor form.  ``rest``: the 33 weight tensors, rescale, alpha_mu, lamb_eff, beta1,
    beta2, lr, wd_eff, eps, bc1, bc2, then the eight geometry integers and expert_counts."""
    names = list(_V2_WEIGHTS) + ["rescale", "alpha_mu", "lamb_eff", "beta1", "beta2", "lr", "wd_eff", "eps", "bc1", "bc2", "d_model", "d_state",
                                 "d_inner", "gru_hidden", "num_heads", "pk_dim", "expert_hidden", "num_experts", "expert_counts"]
    a = dict(zip(names, rest))
    a.update(kw)
    w = [a[k] for k in _V2_WEIGHTS]
    supergrok2_mamba_peer_batched_step([param], [grad], [sharpness], [exp_avg], [exp_avg_sq], [mu], [gru_state], [mamba_fwd_state],
                                       [mamba_bwd_state], *w, [a["alpha_mu"]], [a["lamb_eff"]], [a["beta1"]], [a["bc1"]], [a["bc2"]],
                                       a["rescale"], a["beta2"], a["lr"], a["wd_eff"], a["eps"], a["d_model"], a["d_state"], a["d_inner"],
                                       a["gru_hidden"], a["num_heads"], a["pk_dim"], a["expert_hidden"], a["num_experts"], a["expert_counts"])


def _bilevel_packed(*_a, **_k):
    raise NotImplementedError("the packed-buffer bilevel launchers are internal to the reference's Python bilevel_step; use "
                              "SuperGrok2.bilevel_step(...) or supergrok15_b200.ops.sg2.bilevel_backward(...), which return the same "
                              "meta-net gradients")


supergrok2_bilevel_fwd_save = supergrok2_bilevel_backward = _bilevel_packed
supergrok2_bilevel_fwd_save_batched = supergrok2_bilevel_backward_batched = _bilevel_packed

REFERENCE_NAMES = ("supergrok15_fused_step", "supergrok15_sam_perturb_all", "supergrok15_sharpness_restore_all", "supergrok11_fused_step",
                   "supergrok11_sam_perturb_all", "supergrok11_sharpness_restore_all", "grokadamw_fused_step", "neuralgrok_fused_step",
                   "prodigy_fused_step", "grokfast_fused_step", "lion_fused_step", "looksam_perturb_all", "looksam_restore_all",
                   "looksam_compute_directions", "looksam_adjust_grads", "muon_fused_step", "supergrok2_mamba_peer_step",
                   "supergrok2_mamba_peer_batched_step", "supergrok2_bilevel_fwd_save", "supergrok2_bilevel_backward",
                   "supergrok2_bilevel_fwd_save_batched", "supergrok2_bilevel_backward_batched")


class _OpsModule(types.ModuleType):
    """``grokking_optimizers._ops``: the reference's entry points, then whatever the native extension exports."""

    def __getattr__(self, name):
        native = _build.load()
        if native is not None and hasattr(native, name):
            return getattr(native, name)
        raise AttributeError(f"module '{self.__name__}' has no attribute '{name}'")


def module(name: str = "grokking_optimizers._ops") -> types.ModuleType:
    m = _OpsModule(name, __doc__)
    for n in REFERENCE_NAMES:
        setattr(m, n, globals()[n])
    m.REFERENCE_NAMES = REFERENCE_NAMES
    return m
