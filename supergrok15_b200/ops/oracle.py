"""Plain-PyTorch fp32 statement of every optimizer update in this package.

These functions are the numerical oracle: the CUDA kernels are tested against them
and the optimizers call them directly when their parameters live on the CPU.  Every
function works in place on lists of tensors (one entry per parameter) and keeps all
state in fp32 regardless of the parameter dtype.

Formulas follow the reference kernels and dispatch code:
  lion       csrc/lion_kernels.cu:20            grokfast   csrc/grokfast_kernels.cu:20
  grokadamw  csrc/grokadamw_kernels.cu:42       prodigy    csrc/prodigy_kernels.cu:50,111 + csrc/ops.cpp:425-507
  neuralgrok csrc/neuralgrok_kernels.cu:244     looksam    csrc/looksam_kernels.cu:19-62 + csrc/ops.cpp:569-656
  muon       csrc/ops.cpp:663-746               sg15       csrc/supergrok15_kernels.cu:323 + csrc/ops.cpp:83-152
  sg11       csrc/supergrok11_kernels.cu:37,109,218 + csrc/ops.cpp:211-291
  adamw      grokking_optimizers/_adamw_helper.py:12-22
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

Tensors = List[torch.Tensor]
reducer = None          # optional fn(vec)->vec summing a small vector over data-parallel ranks (set by the ZeRO engine)


def _f(t: torch.Tensor) -> torch.Tensor:
    return t.detach().reshape(-1).float()


def _store(p: torch.Tensor, new_flat: torch.Tensor) -> None:
    p.detach().copy_(new_flat.reshape(p.shape).to(p.dtype))


# --------------------------------------------------------------------------- reductions
def global_sqnorm(grads: Sequence[Optional[torch.Tensor]]) -> torch.Tensor:
    """Sum of squares over every defined gradient (fp32 scalar tensor)."""
    tot = None
    for g in grads:
        if g is None or g.numel() == 0:
            continue
        s = _f(g).pow(2).sum()
        tot = s if tot is None else tot + s
    if tot is None:
        tot = torch.zeros(())
    if reducer is not None:                       # sharded data parallelism: sum over the ranks' tensors
        tot = reducer(tot.reshape(1).clone())[0]
    return tot


def clip_coef(sqnorm: torch.Tensor, max_norm: float) -> torch.Tensor:
    """Scale applied to every gradient by the global clip: max/(norm+1e-6) when norm>max, else 1."""
    norm = sqnorm.sqrt()
    return torch.where(norm > max_norm, max_norm / (norm + 1e-6), torch.ones_like(norm))


def clip_grads_(grads: Sequence[Optional[torch.Tensor]], max_norm: float) -> torch.Tensor:
    """In-place global-norm clip of the gradient list; returns the pre-clip norm."""
    sq = global_sqnorm(grads)
    c = clip_coef(sq, max_norm)
    for g in grads:
        if g is not None and g.numel() > 0:
            g.mul_(c.to(g.dtype))
    return sq.sqrt()


# --------------------------------------------------------------------------- AdamW
def adamw_(params: Tensors, grads: Tensors, exp_avgs: Tensors, exp_avg_sqs: Tensors, steps: Sequence[int],
           lr: float, beta1: float, beta2: float, eps: float, wd: float) -> None:
    for p, g, m, v, step in zip(params, grads, exp_avgs, exp_avg_sqs, steps):
        if g is None:
            continue
        gf = _f(g)
        mf, vf = m.view(-1), v.view(-1)
        mf.mul_(beta1).add_(gf, alpha=1 - beta1)
        vf.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
        bc1 = 1 - beta1 ** step
        bc2 = 1 - beta2 ** step
        pf = _f(p) * (1 - lr * wd)
        pf = pf - (lr / bc1) * mf / ((vf / bc2).sqrt() + eps)
        _store(p, pf)


# --------------------------------------------------------------------------- Lion
def lion_(params: Tensors, grads: Tensors, exp_avgs: Tensors, lr: float, beta1: float, beta2: float,
          wd: float) -> None:
    for p, g, m in zip(params, grads, exp_avgs):
        if g is None:
            continue
        gf, mf = _f(g), m.view(-1)
        upd = torch.sign(beta1 * mf + (1 - beta1) * gf)
        pf = _f(p)
        pf = pf - lr * (upd + wd * pf)
        mf.mul_(beta2).add_(gf, alpha=1 - beta2)
        _store(p, pf)


# --------------------------------------------------------------------------- Grokfast
def grokfast_ema_(grads: Tensors, emas: Tensors, alpha: float, lamb: float) -> None:
    """e = a*e + (1-a)*g ; g += lamb*e   (the gradient is modified in place)."""
    for g, e in zip(grads, emas):
        if g is None:
            continue
        gf, ef = _f(g), e.view(-1)
        ef.mul_(alpha).add_(gf, alpha=1 - alpha)
        g.detach().copy_((gf + lamb * ef).reshape(g.shape).to(g.dtype))


# --------------------------------------------------------------------------- GrokAdamW
def grokadamw_(params: Tensors, grads: Tensors, exp_avgs: Tensors, exp_avg_sqs: Tensors, emas: Tensors,
               steps: Sequence[int], lr: float, beta1: float, beta2: float, eps: float, wd: float,
               alpha: float, lamb: float, grad_clip: float) -> None:
    c = clip_coef(global_sqnorm(grads), grad_clip) if grad_clip > 0 else torch.ones(())
    for p, g, m, v, e, step in zip(params, grads, exp_avgs, exp_avg_sqs, emas, steps):
        if g is None:
            continue
        gf = _f(g) * c.to(g.device)
        g.detach().copy_(gf.reshape(g.shape).to(g.dtype))       # the clip is visible in p.grad
        ef, mf, vf = e.view(-1), m.view(-1), v.view(-1)
        ef.mul_(alpha).add_(gf, alpha=1 - alpha)
        a = gf + lamb * ef
        mf.mul_(beta1).add_(a, alpha=1 - beta1)
        vf.mul_(beta2).addcmul_(a, a, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        pf = _f(p) * (1 - lr * wd) - (lr / bc1) * mf / ((vf / bc2).sqrt() + eps)
        _store(p, pf)


# --------------------------------------------------------------------------- Prodigy
def prodigy_dlr(params: Tensors, grads: Tensors, s_bufs: Tensors, param_inits: Tensors, d_lr: float) -> float:
    """d_lr <- max(d_lr, |sum g.(p-p0)| / (sum s + 1e-12)) when sum s > 1e-30 (global over all tensors)."""
    num = 0.0
    den = 0.0
    for p, g, s, p0 in zip(params, grads, s_bufs, param_inits):
        if g is None:
            continue
        num = num + float((_f(g) * (_f(p) - p0.view(-1))).sum())
        den = den + float(s.view(-1).sum())
    if reducer is not None:
        nd = reducer(torch.tensor([num, den], dtype=torch.float32))
        num, den = float(nd[0]), float(nd[1])
    if den > 1e-30:
        d_lr = max(d_lr, abs(num) / (den + 1e-12))
    return d_lr


def prodigy_step_(params: Tensors, grads: Tensors, exp_avgs: Tensors, exp_avg_sqs: Tensors, s_bufs: Tensors,
                  steps: Sequence[int], d_lr: float, lr: float, beta1: float, beta2: float, eps: float,
                  wd: float) -> None:
    for p, g, m, v, s, step in zip(params, grads, exp_avgs, exp_avg_sqs, s_bufs, steps):
        if g is None:
            continue
        dg = _f(g) * d_lr
        sf, mf, vf = s.view(-1), m.view(-1), v.view(-1)
        sf.mul_(beta2).addcmul_(dg, dg, value=1 - beta2)
        mf.mul_(beta1).add_(dg, alpha=1 - beta1)
        vf.mul_(beta2).addcmul_(dg, dg, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        pf = _f(p) * (1 - lr * d_lr * wd) - (lr / bc1) * mf / ((vf / bc2).sqrt() + d_lr * eps)
        _store(p, pf)


def prodigy_(params: Tensors, grads: Tensors, exp_avgs: Tensors, exp_avg_sqs: Tensors, s_bufs: Tensors,
             param_inits: Tensors, steps: Sequence[int], d_lr: float, lr: float, beta1: float, beta2: float,
             eps: float, wd: float) -> float:
    d_lr = prodigy_dlr(params, grads, s_bufs, param_inits, d_lr)
    prodigy_step_(params, grads, exp_avgs, exp_avg_sqs, s_bufs, steps, d_lr, lr, beta1, beta2, eps, wd)
    return d_lr


# --------------------------------------------------------------------------- NeuralGrok
def neuralgrok_amplify(g: torch.Tensor, W1: torch.Tensor, b1: torch.Tensor, W2: torch.Tensor, b2: torch.Tensor,
                       alpha: float, beta: float) -> torch.Tensor:
    """ag = g*(alpha*(W2.relu(W1 g + b1) + b2) + beta); W1 [H,1] or [H], W2 [1,H] or [H]."""
    h = torch.relu(g.unsqueeze(-1) * W1.reshape(-1) + b1.reshape(-1))
    mlp = (h * W2.reshape(-1)).sum(-1) + b2.reshape(-1)[0]
    return g * (alpha * mlp + beta)


def neuralgrok_(params: Tensors, grads: Tensors, exp_avgs: Tensors, exp_avg_sqs: Tensors, steps: Sequence[int],
                W1, b1, W2, b2, alpha: float, beta: float, lr: float, beta1: float, beta2: float, eps: float,
                wd: float, grad_clip: float) -> None:
    c = clip_coef(global_sqnorm(grads), grad_clip) if grad_clip > 0 else torch.ones(())
    for p, g, m, v, step in zip(params, grads, exp_avgs, exp_avg_sqs, steps):
        if g is None:
            continue
        gf = _f(g) * c.to(g.device)
        g.detach().copy_(gf.reshape(g.shape).to(g.dtype))
        ag = neuralgrok_amplify(gf, W1.float(), b1.float(), W2.float(), b2.float(), alpha, beta)
        mf, vf = m.view(-1), v.view(-1)
        mf.mul_(beta1).add_(ag, alpha=1 - beta1)
        vf.mul_(beta2).addcmul_(ag, ag, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        pf = _f(p) * (1 - lr * wd) - (lr / bc1) * mf / ((vf / bc2).sqrt() + eps)
        _store(p, pf)


# --------------------------------------------------------------------------- LookSAM pieces
def sam_grad_norm(grads: Sequence[Optional[torch.Tensor]]) -> torch.Tensor:
    return global_sqnorm(grads).sqrt() + 1e-12


def looksam_perturb_(params: Tensors, grads: Tensors, backups: Tensors, rho: float) -> None:
    norm = sam_grad_norm(grads)
    for p, g, b in zip(params, grads, backups):
        if g is None:
            continue
        b.view(-1).copy_(_f(p))
        _store(p, _f(p) + (rho / norm).to(p.device) * _f(g))


def looksam_restore_(params: Tensors, backups: Tensors) -> None:
    for p, b in zip(params, backups):
        _store(p, b.view(-1))


def looksam_direction_(v_dirs: Tensors, sam_grads: Tensors, grads: Tensors) -> None:
    for v, gs, g in zip(v_dirs, sam_grads, grads):
        if g is None or gs is None:
            continue
        d = _f(gs) - _f(g)
        n = d.norm()
        if float(n) < 1e-12:
            continue
        v.view(-1).copy_(d / n)


def looksam_adjust_(grads: Tensors, v_dirs: Tensors, alpha: float) -> None:
    for g, v in zip(grads, v_dirs):
        if g is None:
            continue
        gf = _f(g)
        g.detach().copy_((gf + alpha * gf.norm() * v.view(-1)).reshape(g.shape).to(g.dtype))


# --------------------------------------------------------------------------- Muon
NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(X: torch.Tensor, steps: int = 5, coeffs=NS_COEFFS) -> torch.Tensor:
    """Reference left-form iteration X <- aX + b(XX^T)X + c(XX^T)^2 X (csrc/ops.cpp:713-727)."""
    a, b, c = coeffs
    for _ in range(steps):
        A = X @ X.t()
        AX = A @ X
        AAX = A @ AX
        X = a * X + b * AX + c * AAX
    return X


def newton_schulz_gram(X: torch.Tensor, steps: int = 5, coeffs=NS_COEFFS) -> torch.Tensor:
    """Right-Gram form X <- X(aI + bG + cG^2), G = X^T X; algebraically equal to the left form."""
    a, b, c = coeffs
    eye = torch.eye(X.shape[1], dtype=X.dtype, device=X.device)
    for _ in range(steps):
        G = X.t() @ X
        X = X @ (a * eye + b * G + c * (G @ G))
    return X


def muon_(params: Tensors, grads: Tensors, bufs: Tensors, lr: float, momentum: float, wd: float,
          ns_steps: int = 5) -> None:
    for p, g, buf in zip(params, grads, bufs):
        if g is None:
            continue
        if p.dim() != 2:
            raise ValueError("Muon group holds a non-2-D parameter; pass it as params_1d")
        bf = buf.view(p.shape)
        bf.mul_(momentum).add_(g.detach().float())
        X = bf / (bf.norm() + 1e-7)
        X = newton_schulz(X, ns_steps)
        pf = (p.detach().float() + (-0.2 * lr) * X) * (1 - lr * wd)
        p.detach().copy_(pf.to(p.dtype))


# --------------------------------------------------------------------------- SuperGrok meta-net (v1.1 / v1.5)
def fast_gelu(z: torch.Tensor) -> torch.Tensor:
    return z / (1 + torch.exp(-1.702 * z))


def sharpness_mlp(g: torch.Tensor, s: torch.Tensor, W1, b1, W2, b2, rescale: float, exact_gelu: bool = False):
    """g + rescale*MLP([g,s]); W1 [H,2], b1 [H], W2 [1,H] or [H], b2 [1]."""
    z = g.unsqueeze(-1) * W1[:, 0] + s.unsqueeze(-1) * W1[:, 1] + b1
    act = torch.nn.functional.gelu(z) if exact_gelu else fast_gelu(z)
    return g + rescale * ((act * W2.reshape(-1)).sum(-1) + b2.reshape(-1)[0])


def sg15_(params: Tensors, grads: Tensors, exp_avgs: Tensors, exp_avg_sqs: Tensors, mus: Tensors,
          sharps: Tensors, steps: Sequence[int], layer_alphas: Sequence[float], layer_beta1s: Sequence[float],
          W1, b1, W2, b2, rescale: float, beta2: float, lr: float, wd_eff: float, eps: float, lamb: float,
          ramp: float, gate: float, grad_clip: float, exact_gelu: bool = False) -> None:
    """`steps[i]` is the value used for bias correction (the caller decides frozen-at-1 or real)."""
    c = clip_coef(global_sqnorm(grads), grad_clip) if grad_clip > 0 else torch.ones(())
    lamb_eff = ramp * gate * lamb if ramp > 0 else 0.0
    for i, (p, g) in enumerate(zip(params, grads)):
        if g is None or g.numel() == 0:
            continue
        gf = _f(g) * c.to(g.device)
        g.detach().copy_(gf.reshape(g.shape).to(g.dtype))
        mu, m, v = mus[i].view(-1), exp_avgs[i].view(-1), exp_avg_sqs[i].view(-1)
        a, b1_i, step = layer_alphas[i], layer_beta1s[i], steps[i]
        mu.mul_(a).add_(gf, alpha=1 - a)
        sg = sharpness_mlp(gf, sharps[i].reshape(-1).float(), W1.float(), b1.float(), W2.float(), b2.float(),
                           rescale, exact_gelu)
        fg = sg + lamb_eff * mu
        m.mul_(b1_i).add_(fg, alpha=1 - b1_i)
        v.mul_(beta2).addcmul_(fg, fg, value=1 - beta2)
        bc1, bc2 = 1 - b1_i ** step, 1 - beta2 ** step
        pf = _f(p) * (1 - lr * wd_eff) - (lr / bc1) * m / ((v / bc2).sqrt() + eps)
        _store(p, pf)


def sg11_(params: Tensors, grads: Tensors, exp_avgs: Tensors, exp_avg_sqs: Tensors, mus: Tensors,
          sharps: Tensors, steps: Sequence[int], layer_alphas: Sequence[float], layer_beta1s: Sequence[float],
          W1, b1, W2, b2, rescale: float, beta2: float, lr: float, wd_eff: float, eps: float, lamb: float,
          ramp: float, gate_temperature: float, grad_clip: float, exact_gelu: bool = False) -> List[float]:
    c = clip_coef(global_sqnorm(grads), grad_clip) if grad_clip > 0 else torch.ones(())
    gates = []
    for i, (p, g) in enumerate(zip(params, grads)):
        if g is None or g.numel() == 0:
            gates.append(0.0)
            continue
        gf = _f(g) * c.to(g.device)
        g.detach().copy_(gf.reshape(g.shape).to(g.dtype))
        mu, m, v = mus[i].view(-1), exp_avgs[i].view(-1), exp_avg_sqs[i].view(-1)
        a, b1_i, step = layer_alphas[i], layer_beta1s[i], steps[i]
        mu.mul_(a).add_(gf, alpha=1 - a)
        sg = sharpness_mlp(gf, sharps[i].reshape(-1).float(), W1.float(), b1.float(), W2.float(), b2.float(),
                           rescale, exact_gelu)
        cos = float((sg * mu).sum()) / (float(sg.norm()) * float(mu.norm()) + 1e-8)
        gate = 1.0 / (1.0 + math.exp(-gate_temperature * cos))
        gates.append(gate)
        lamb_eff = ramp * gate * lamb if ramp > 0 else 0.0
        fg = sg + lamb_eff * mu
        m.mul_(b1_i).add_(fg, alpha=1 - b1_i)
        v.mul_(beta2).addcmul_(fg, fg, value=1 - beta2)
        bc1, bc2 = 1 - b1_i ** step, 1 - beta2 ** step
        pf = _f(p) * (1 - lr * wd_eff) - (lr / bc1) * m / ((v / bc2).sqrt() + eps)
        _store(p, pf)
    return gates


# --------------------------------------------------------------------------- SuperGrok v2 element step
def sg2_adam_(p: torch.Tensor, smart: torch.Tensor, g: torch.Tensor, mu: torch.Tensor, m: torch.Tensor,
              v: torch.Tensor, alpha: float, lamb_eff: float, beta1: float, beta2: float, lr: float, wd_eff: float,
              eps: float, bc1: float, bc2: float) -> None:
    """Tail of the v2 element step (csrc/supergrok2_mamba_peer_kernels.cu:1068-1088)."""
    mu_f, m_f, v_f = mu.view(-1), m.view(-1), v.view(-1)
    mu_f.mul_(alpha).add_(g, alpha=1 - alpha)
    fg = smart + lamb_eff * mu_f
    m_f.mul_(beta1).add_(fg, alpha=1 - beta1)
    v_f.mul_(beta2).addcmul_(fg, fg, value=1 - beta2)
    pf = _f(p) * (1 - lr * wd_eff) - (lr / bc1) * m_f / ((v_f / bc2).sqrt() + eps)
    _store(p, pf)
