"""Dispatch of the element-wise optimizer updates.

CUDA tensors go to the sm_100a multi-tensor kernels (``csrc/mt_kernels.cu``) and raise if the
extension is missing.  fp32 CPU tensors go to the C++ CPU kernels (``csrc/cpu_kernels.cpp``, the same ops through the
same entry points) when the extension is built and ``SG_CPU_NATIVE`` is not ``0``; everything else on the CPU (other
dtypes, no extension) goes to the PyTorch oracle (``ops/oracle.py``), which is also what the tests compare both native
paths against.  Global scalars
(clip coefficient, Prodigy ``d_lr``, cosine gates, SAM scale) stay on the device: the functions
return device tensors and never call ``.item()``.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch

from .. import _build
from . import oracle

Tensors = List[torch.Tensor]
_ws: Dict[torch.device, Dict[str, torch.Tensor]] = {}


CPU_NATIVE = os.environ.get("SG_CPU_NATIVE", "1") != "0"
# GROK_DEBUG=1: every scratch buffer handed out is filled with NaN first, so a kernel that reads scratch it has not written
# (a stale value from an earlier call would otherwise look plausible) shows up as a non-finite result
DEBUG_POISON = os.environ.get("GROK_DEBUG", "0") not in ("", "0")


def _is_cuda(ts: Sequence[Optional[torch.Tensor]]) -> bool:
    for t in ts:
        if t is not None:
            return t.is_cuda
    return False


def _native(*lists: Sequence[Optional[torch.Tensor]]) -> bool:
    """True when the native kernels take these tensors: CUDA always (the extension is then mandatory), CPU when every
    tensor is contiguous fp32, the extension is available and the C++ CPU path is enabled."""
    if _is_cuda(lists[0]):
        return True
    if not CPU_NATIVE or not _build.native_available():
        return False
    for l in lists:
        for t in l:
            if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.device.type != "cpu"):
                return False
    return True


def workspace(dev: torch.device, name: str, numel: int, dtype=torch.float32) -> torch.Tensor:
    """Grow-only per-device scratch buffers (the step path performs no allocation once warm)."""
    d = _ws.setdefault(dev, {})
    t = d.get(name)
    if t is None or t.numel() < numel or t.dtype != dtype:
        t = torch.empty(max(numel, 1024), dtype=dtype, device=dev)
        d[name] = t
    if DEBUG_POISON and t.is_floating_point():
        t[:max(numel, 1)].fill_(float("nan"))
    return t


def _grads(params: Tensors) -> List[Optional[torch.Tensor]]:
    return [p.grad for p in params]


def _filter(params: Tensors, *lists):
    """Keep entries whose parameter has a gradient."""
    keep = [i for i, p in enumerate(params) if p.grad is not None and p.numel() > 0]
    out = [[params[i] for i in keep], [params[i].grad for i in keep]]
    for l in lists:
        out.append([l[i] for i in keep])
    return keep, out


def _op(name: str) -> int:
    return _build.require().ops[name]


def _reduce(op: str, roles, n: int, dev, tag: str) -> torch.Tensor:
    """Run reduction ``op``; returns per-tensor sums [n,3] (device, fp32)."""
    C = _build.require()
    numels = [int(t.numel()) for t in next(r for r in roles if r)]
    nb = C.mt_num_blocks(numels)
    partials = workspace(dev, "partials", 3 * nb)
    out = workspace(dev, "pt_" + tag, 3 * n)
    C.mt_apply(_op(op), roles, [], [], partials=partials, per_tensor_out=out)
    return out


def sqnorm_per_tensor(grads: Tensors, tag: str = "sq") -> torch.Tensor:
    return _reduce("OP_SQNORM", [[], list(grads)], len(grads), grads[0].device, tag)


def clip_coef_device(grads: Tensors, max_norm: float) -> torch.Tensor:
    """Device tensor [3] = (sum of squares, clip coefficient, norm) over ``grads``."""
    dev = grads[0].device
    pt = sqnorm_per_tensor(grads)
    out = workspace(dev, "clip", 4)
    tot = _global_totals(pt, len(grads), dev)
    _build.require().scalar_finalize(_op("SC_CLIP"), tot, 1, out, float(max_norm), 0.0, 0.0)
    return out


_reducer = None


def set_cross_rank_reducer(fn) -> None:
    """Install ``fn(vec) -> vec`` (in-place sum over data-parallel ranks of a small fp32 device vector).
    The sharded engine sets it around an optimizer step so global scalars (clip norm, Prodigy numerator and
    denominator, SAM norm) cover the tensors owned by every rank; ``None`` removes it."""
    global _reducer
    _reducer = fn
    oracle.reducer = fn


def _global_totals(pt: torch.Tensor, n: int, dev) -> torch.Tensor:
    """Column sums of the per-tensor [n,3] partials as a device [3] tensor, combined across ranks if sharded."""
    tot = workspace(dev, "tot3", 4)
    _build.require().scalar_finalize(_op("SC_SUM3"), pt, n, tot, 0.0, 0.0, 0.0)
    if _reducer is not None:
        _reducer(tot[:3])
    return tot


# --------------------------------------------------------------------------- steps
def adamw(params, grads, ms, vs, steps, lr, b1, b2, eps, wd):
    if not _native(params, grads, ms, vs):
        return oracle.adamw_(params, grads, ms, vs, steps, lr, b1, b2, eps, wd)
    ts = [[1 - b1 ** s, 1 - b2 ** s] for s in steps]
    _build.require().mt_apply(_op("OP_ADAMW"), [params, grads, ms, vs], ts, [lr, b1, b2, eps, wd])


def lion(params, grads, ms, lr, b1, b2, wd):
    if not _native(params, grads, ms):
        return oracle.lion_(params, grads, ms, lr, b1, b2, wd)
    _build.require().mt_apply(_op("OP_LION"), [params, grads, ms], [], [lr, b1, b2, 0.0, wd])


def grokfast_ema(grads, emas, alpha, lamb):
    if not _native(grads, emas):
        return oracle.grokfast_ema_(grads, emas, alpha, lamb)
    _build.require().mt_apply(_op("OP_GROKFAST_EMA"), [[], grads, emas], [], [0, 0, 0, 0, 0, alpha, lamb])


def grokfast_adamw(params, grads, ms, vs, emas, steps, lr, b1, b2, eps, wd, alpha, lamb):
    """EMA filter + amplification + AdamW in one pass (the gradient is amplified in place)."""
    if not _native(params, grads, ms, vs, emas):
        oracle.grokfast_ema_(grads, emas, alpha, lamb)
        return oracle.adamw_(params, grads, ms, vs, steps, lr, b1, b2, eps, wd)
    ts = [[1 - b1 ** s, 1 - b2 ** s] for s in steps]
    _build.require().mt_apply(_op("OP_GROKFAST_ADAMW"), [params, grads, ms, vs, emas], ts,
                              [lr, b1, b2, eps, wd, alpha, lamb], write_grad=True)


def grokadamw(params, grads, ms, vs, emas, steps, lr, b1, b2, eps, wd, alpha, lamb, grad_clip):
    if not _native(params, grads, ms, vs, emas):
        return oracle.grokadamw_(params, grads, ms, vs, emas, steps, lr, b1, b2, eps, wd, alpha, lamb, grad_clip)
    clip = clip_coef_device(grads, grad_clip)[1:2] if grad_clip > 0 else None
    ts = [[1 - b1 ** s, 1 - b2 ** s] for s in steps]
    _build.require().mt_apply(_op("OP_GROKADAMW"), [params, grads, ms, vs, emas], ts,
                              [lr, b1, b2, eps, wd, alpha, lamb], clip=clip, write_grad=True)


def prodigy_dlr(params, grads, ss, p0s, d_lr_dev: Optional[torch.Tensor], d_lr: float):
    """Global distance estimate.  CPU: returns the new float.  CUDA: updates ``d_lr_dev`` ([1] fp32) in place."""
    if not _native(params, grads, ss, p0s):
        return oracle.prodigy_dlr(params, grads, ss, p0s, d_lr)
    C = _build.require()
    pt = _reduce("OP_PRODIGY_REDUCE", [params, grads, p0s, ss], len(params), params[0].device, "prodigy")
    tot = _global_totals(pt, len(params), params[0].device)
    if not params[0].is_cuda:                                    # CPU callers keep d_lr as a float
        d_lr_dev = torch.tensor([float(d_lr)], dtype=torch.float32)
        C.scalar_finalize(_op("SC_PRODIGY"), tot, 1, d_lr_dev, 0.0, 0.0, 0.0)
        return max(float(d_lr), float(d_lr_dev[0]))              # the estimate never decreases; fp32 rounding of the old value must not lower it
    C.scalar_finalize(_op("SC_PRODIGY"), tot, 1, d_lr_dev, 0.0, 0.0, 0.0)
    return d_lr_dev


def prodigy_step(params, grads, ms, vs, ss, steps, d_lr, lr, b1, b2, eps, wd):
    """``d_lr`` is a float on CPU and the [1] device tensor on CUDA."""
    if not _native(params, grads, ms, vs, ss):
        return oracle.prodigy_step_(params, grads, ms, vs, ss, steps, d_lr, lr, b1, b2, eps, wd)
    ts = [[1 - b1 ** s, 1 - b2 ** s] for s in steps]
    if not torch.is_tensor(d_lr):
        d_lr = torch.tensor([float(d_lr)], dtype=torch.float32, device=params[0].device)
    _build.require().mt_apply(_op("OP_PRODIGY"), [params, grads, ms, vs, ss], ts, [lr, b1, b2, eps, wd], dscal=d_lr)


def neuralgrok(params, grads, ms, vs, steps, W1, b1w, W2, b2w, alpha, beta, lr, b1, b2, eps, wd, grad_clip):
    if not _native(params, grads, ms, vs):
        return oracle.neuralgrok_(params, grads, ms, vs, steps, W1, b1w, W2, b2w, alpha, beta, lr, b1, b2, eps, wd,
                                  grad_clip)
    clip = clip_coef_device(grads, grad_clip)[1:2] if grad_clip > 0 else None
    ts = [[1 - b1 ** s, 1 - b2 ** s] for s in steps]
    H = W1.numel()
    _build.require().mt_apply(_op("OP_NEURALGROK"), [params, grads, ms, vs], ts,
                              [lr, b1, b2, eps, wd, alpha, 0.0, beta], clip=clip,
                              W1=W1.reshape(-1).float().contiguous(), b1=b1w.reshape(-1).float().contiguous(),
                              W2=W2.reshape(-1).float().contiguous(), b2=b2w.reshape(-1).float().contiguous(),
                              hidden=H, write_grad=True)


def sg15(params, grads, ms, vs, mus, sharps, bc_steps, layer_alphas, layer_beta1s, W1, b1w, W2, b2w, rescale, beta2,
         lr, wd_eff, eps, lamb, ramp, gate, grad_clip, exact_gelu=False):
    if not _native(params, grads, ms, vs, mus, sharps):
        return oracle.sg15_(params, grads, ms, vs, mus, sharps, bc_steps, layer_alphas, layer_beta1s, W1, b1w, W2,
                            b2w, rescale, beta2, lr, wd_eff, eps, lamb, ramp, gate, grad_clip, exact_gelu)
    clip = clip_coef_device(grads, grad_clip)[1:2] if grad_clip > 0 else None
    lamb_eff = ramp * gate * lamb if ramp > 0 else 0.0
    ts = [[a, b1_i, 1 - b1_i ** s, 1 - beta2 ** s] for a, b1_i, s in zip(layer_alphas, layer_beta1s, bc_steps)]
    H = b1w.numel()
    _build.require().mt_apply(_op("OP_SG15"), [params, grads, ms, vs, mus, sharps], ts,
                              [lr, 0.0, beta2, eps, wd_eff, 0.0, lamb_eff, rescale], clip=clip,
                              W1=W1.float().contiguous(), b1=b1w.float().contiguous(),
                              W2=W2.reshape(-1).float().contiguous(), b2=b2w.reshape(-1).float().contiguous(),
                              hidden=H, write_grad=True)


def sg11(params, grads, ms, vs, mus, sharps, bc_steps, layer_alphas, layer_beta1s, W1, b1w, W2, b2w, rescale, beta2,
         lr, wd_eff, eps, lamb, ramp, gate_temperature, grad_clip, exact_gelu=False):
    """Returns the per-tensor gates (list of floats on CPU, device tensor [n] on CUDA)."""
    if not _native(params, grads, ms, vs, mus, sharps):
        return oracle.sg11_(params, grads, ms, vs, mus, sharps, bc_steps, layer_alphas, layer_beta1s, W1, b1w, W2,
                            b2w, rescale, beta2, lr, wd_eff, eps, lamb, ramp, gate_temperature, grad_clip, exact_gelu)
    C = _build.require()
    dev = params[0].device
    n = len(params)
    clip = clip_coef_device(grads, grad_clip)[1:2] if grad_clip > 0 else None
    numel = sum((int(p.numel()) + 3) // 4 * 4 for p in params)
    smart_flat = workspace(dev, "sg11_smart", numel)
    smart, off = [], 0
    for p in params:
        smart.append(smart_flat[off:off + p.numel()])
        off += (p.numel() + 3) // 4 * 4          # keep every view 16-byte aligned for 4-wide accesses
    H = b1w.numel()
    nb = C.mt_num_blocks([int(p.numel()) for p in params])
    partials = workspace(dev, "partials", 3 * nb)
    pt = workspace(dev, "pt_sg11", 3 * n)
    wk = dict(W1=W1.float().contiguous(), b1=b1w.float().contiguous(), W2=W2.reshape(-1).float().contiguous(),
              b2=b2w.reshape(-1).float().contiguous(), hidden=H)
    C.mt_apply(_op("OP_SG11_A"), [[], grads, mus, sharps, smart], [[a] for a in layer_alphas],
               [0, 0, 0, 0, 0, 0, 0, rescale], clip=clip, write_grad=True, partials=partials, per_tensor_out=pt, **wk)
    gates = workspace(dev, "sg11_gates", 2 * n)
    C.scalar_finalize(_op("SC_SG11_GATES"), pt, n, gates, float(gate_temperature), float(ramp), float(lamb))
    ts = [[b1_i, 1 - b1_i ** s, 1 - beta2 ** s] for b1_i, s in zip(layer_beta1s, bc_steps)]
    C.mt_apply(_op("OP_SG11_B"), [params, smart, ms, vs, mus], ts, [lr, 0.0, beta2, eps, wd_eff], tscal=gates)
    return gates[n:2 * n] if dev.type == "cuda" else gates[n:2 * n].tolist()


# --------------------------------------------------------------------------- SAM helpers
def sam_scale_device(grads: Tensors, rho: float) -> torch.Tensor:
    """[1] device tensor rho/(||g||+1e-12) over all gradients."""
    dev = grads[0].device
    pt = sqnorm_per_tensor(grads, "sam")
    out = workspace(dev, "sam_scale", 4)
    tot = _global_totals(pt, len(grads), dev)
    _build.require().scalar_finalize(_op("SC_SAM_SCALE"), tot, 1, out, float(rho), 0.0, 0.0)
    return out


def perturb(params, grads, backups, rho):
    if not _native(params, grads, backups):
        return oracle.looksam_perturb_(params, grads, backups, rho)
    sc = sam_scale_device(grads, rho)
    _build.require().mt_apply(_op("OP_PERTURB"), [params, grads, backups], [], [], dscal=sc)


def restore(params, backups):
    if not _native(params, backups):
        return oracle.looksam_restore_(params, backups)
    _build.require().mt_apply(_op("OP_RESTORE"), [params, [], backups], [], [])


def sharpness_restore(params, grads, backups, sam_grads, sharps):
    """sharp = |g_sam - g| ; p = backup  (reference csrc/supergrok15_kernels.cu:170)."""
    if not _native(params, grads, backups, sam_grads, sharps):
        for p, g, b, gs, s in zip(params, grads, backups, sam_grads, sharps):
            s.view(-1).copy_((gs.reshape(-1).float() - g.reshape(-1).float()).abs())
            p.detach().copy_(b.view(p.shape).to(p.dtype))
        return
    _build.require().mt_apply(_op("OP_SHARP_RESTORE"), [params, grads, backups, sam_grads, sharps], [], [])


def looksam_direction_adjust(grads, sam_grads, v_dirs, alpha, do_direction=True):
    """v = (g_sam-g)/||g_sam-g|| per tensor (skipped below 1e-12), then g += alpha*||g||*v."""
    if not _native(grads, sam_grads if do_direction else [], v_dirs):
        if do_direction:
            oracle.looksam_direction_(v_dirs, sam_grads, grads)
        return oracle.looksam_adjust_(grads, v_dirs, alpha)
    C = _build.require()
    dev = grads[0].device
    n = len(grads)
    other = sam_grads if do_direction else grads
    pt = _reduce("OP_DIFF_SQNORM", [[], grads, other], n, dev, "looksam")
    norms = workspace(dev, "looksam_norms", 2 * n)
    C.scalar_finalize(_op("SC_LOOKSAM_NORMS"), pt, n, norms, 0.0, 0.0, 0.0)
    if do_direction:
        C.mt_apply(_op("OP_LOOKSAM_DIR"), [[], grads, v_dirs, sam_grads], [], [], tscal=norms)
    C.mt_apply(_op("OP_LOOKSAM_ADJ"), [[], grads, v_dirs], [], [0, 0, 0, 0, 0, alpha], tscal=norms)


def scale_(grads, factor: float):
    if not _native(grads):
        for g in grads:
            g.mul_(factor)
        return
    _build.require().mt_apply(_op("OP_SCALE"), [[], grads], [], [0, 0, 0, 0, 0, 0, 0, 0, factor])
