"""tcgen05 GEMM wrappers: ``gemm_tn``, the ``linear`` autograd function and the Newton-Schulz chain of Muon.

``gemm_tn(a, b)`` computes ``a @ b.T`` for bf16 row-major ``a [M,K]`` and ``b [N,K]`` on the 5th-generation tensor
cores (``csrc/gemm_sm100.cu``) with an fp32 TMEM accumulator and a fused epilogue
``act(alpha*acc + beta*d + bias + diag*I)``; an optional second output receives the transposed result.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import _build

_err: Dict[torch.device, torch.Tensor] = {}
ACT = {None: 0, "none": 0, "gelu": 1, "silu": 2}


def _err_flag(dev) -> torch.Tensor:
    t = _err.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _err[dev] = t
    return t


_ws: Dict[torch.device, torch.Tensor] = {}


def _splitk_ws(dev) -> torch.Tensor:
    """64 MB fp32 scratch for split-K partial tiles (used when the output has too few tiles to fill the GPU)."""
    t = _ws.get(dev)
    if t is None:
        t = torch.empty(16 * 1024 * 1024, dtype=torch.float32, device=dev)
        _ws[dev] = t
    return t


def check(dev=None) -> None:
    """Raise if a GEMM pipeline wait timed out since the last check (one device-to-host read)."""
    for d, t in _err.items():
        if dev is None or d == dev:
            v = int(t.item())
            if v:
                t.zero_()
                raise RuntimeError(f"tcgen05 GEMM pipeline wait timed out (site {v}) on {d}")


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *, alpha: float = 1.0, beta: float = 0.0,
            d: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, diag: float = 0.0, act=None,
            out_dtype=torch.bfloat16, out_t: Optional[torch.Tensor] = None, a_t: bool = False, b_t: bool = False) -> torch.Tensor:
    """``a_t`` / ``b_t``: the operand is passed transposed (``a`` as [K, M], ``b`` as [K, N]) and read in place through an
    MN-major descriptor; supported combinations: none, ``b_t``, ``a_t and b_t``."""
    C = _build.require()
    if out is None:
        n = b.shape[1 if b_t else 0]
        q = 8 if out_dtype == torch.bfloat16 else 4          # the output is written by TMA: 16-byte row pitch
        npad = -(-n // q) * q
        out = torch.empty(a.shape[1 if a_t else 0], npad, dtype=out_dtype, device=a.device)[:, :n]
    C.gemm_tn(a, b, out, alpha, beta, d, bias, diag, ACT[act], out_t, _err_flag(a.device), _splitk_ws(a.device), a_t, b_t)
    return out


def _pad8(t: torch.Tensor) -> torch.Tensor:
    """bf16 copy whose row stride is a multiple of 8 elements (TMA needs 16-byte row pitch)."""
    t = t.to(torch.bfloat16)
    k = t.shape[1]
    if k % 8 == 0 and t.is_contiguous():
        return t
    kp = -(-k // 8) * 8
    buf = torch.zeros(t.shape[0], kp, dtype=torch.bfloat16, device=t.device)
    buf[:, :k] = t
    return buf[:, :k]


class _Linear(torch.autograd.Function):
    """y = x @ W.T + b with the three GEMMs (forward, dgrad, wgrad) on the tcgen05 kernel."""

    @staticmethod
    def forward(ctx, x, weight, bias, act):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.has_bias, ctx.xshape = bias is not None, x.shape
        y = gemm_tn(_pad8(x2), _pad8(weight), bias=bias, act=act, out_dtype=x.dtype if x.dtype != torch.float32 else torch.float32)
        return y.contiguous().view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dyb = _pad8(dy2)
        # dgrad and wgrad read W, dy and x where they are (transposed operands through MN-major descriptors): no copies
        dx = gemm_tn(dyb, _pad8(weight), out_dtype=x2.dtype, b_t=True).contiguous().view(ctx.xshape)          # dy [M,N] @ W [N,K]
        dw = gemm_tn(dyb, _pad8(x2), out_dtype=weight.dtype, a_t=True, b_t=True).contiguous()                   # dy^T [N,M] @ x [M,K]
        db = _build.require().col_sum(dyb) if ctx.has_bias else None                 # two-stage fp32 column sum, fixed order
        return dx, dw, db, None


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None) -> torch.Tensor:
    if not x.is_cuda:
        y = torch.nn.functional.linear(x, weight, bias)
        return y
    assert act is None, "fused activations are forward-only (used by inference paths)"
    return _Linear.apply(x, weight, bias, act)


def newton_schulz(X: torch.Tensor, steps: int, coeffs, precision: str = "bf16") -> torch.Tensor:
    """X <- aX + b(XX^T)X + c(XX^T)^2X, `steps` times, on the tcgen05 GEMM.  X fp32 [r,c] -> fp32 [r,c].

    rows >= cols: right-Gram form  G = X^T X, P = aI + bG + cG^2, X <- X P   (cols^2-sized intermediates);
    rows <  cols: left form        A = X X^T, Q = aI + bA + cA^2, X <- Q X.
    Both X and X^T are kept in bf16 (the last GEMM of an iteration writes both), so every GEMM is K-major on both operands.
    """
    a, b, c = coeffs
    r, cc = X.shape
    rp, cp = -(-r // 8) * 8, -(-cc // 8) * 8
    dev = X.device
    Xb = torch.zeros(r, cp, dtype=torch.bfloat16, device=dev)[:, :cc]
    XTb = torch.zeros(cc, rp, dtype=torch.bfloat16, device=dev)[:, :r]
    Xb.copy_(X)
    XTb.copy_(X.t())
    tall = r >= cc
    n = cc if tall else r
    npad = -(-n // 8) * 8
    G = torch.zeros(n, npad, dtype=torch.bfloat16, device=dev)[:, :n]
    P = torch.zeros(n, npad, dtype=torch.bfloat16, device=dev)[:, :n]
    out32 = torch.empty(r, -(-cc // 4) * 4, dtype=torch.float32, device=dev)[:, :cc]
    for it in range(steps):
        last = it == steps - 1
        src = XTb if tall else Xb
        gemm_tn(src, src, out=G)                                            # Gram matrix (symmetric)
        gemm_tn(G, G, out=P, alpha=c, beta=b, d=G, diag=a)                  # aI + bG + cG^2 (symmetric)
        if last:
            if tall:
                gemm_tn(Xb, P, out=out32)                                   # X P
            else:
                gemm_tn(P, XTb, out=out32)                                  # Q X   (B operand = X^T [c, r])
        else:
            Xn = torch.empty(r, cp, dtype=torch.bfloat16, device=dev)[:, :cc]       # padded row pitch (16-byte multiple)
            XTn = torch.empty(cc, rp, dtype=torch.bfloat16, device=dev)[:, :r]
            if tall:
                gemm_tn(Xb, P, out=Xn, out_t=XTn)
            else:
                gemm_tn(P, XTb, out=Xn, out_t=XTn)
            Xb, XTb = Xn, XTn
    return out32
