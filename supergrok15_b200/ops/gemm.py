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


_ws: Dict[tuple, torch.Tensor] = {}


def _splitk_ws(dev, slot: int = 0) -> torch.Tensor:
    """64 MB fp32 scratch for split-K partial tiles (used when the output has too few tiles to fill the GPU).  ``slot``: GEMMs
    that may run at the same time on different streams take different scratch buffers."""
    t = _ws.get((dev, slot))
    if t is None:
        t = torch.empty(16 * 1024 * 1024, dtype=torch.float32, device=dev)
        _ws[(dev, slot)] = t
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
            out_dtype=torch.bfloat16, out_t: Optional[torch.Tensor] = None, a_t: bool = False, b_t: bool = False,
            ws_slot: int = 0) -> torch.Tensor:
    """``a_t`` / ``b_t``: the operand is passed transposed (``a`` as [K, M], ``b`` as [K, N]) and read in place through an
    MN-major descriptor; supported combinations: none, ``b_t``, ``a_t and b_t``.  ``ws_slot``: which split-K scratch to use."""
    C = _build.require()
    if out is None:
        n = b.shape[1 if b_t else 0]
        q = 8 if out_dtype == torch.bfloat16 else 4          # the output is written by TMA: 16-byte row pitch
        npad = -(-n // q) * q
        out = torch.empty(a.shape[1 if a_t else 0], npad, dtype=out_dtype, device=a.device)[:, :n]
    C.gemm_tn(a, b, out, alpha, beta, d, bias, diag, ACT[act], out_t, _err_flag(a.device), _splitk_ws(a.device, ws_slot), a_t, b_t)
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


def _split(x32: torch.Tensor):
    """fp32 matrix -> (hi, lo) bf16 with hi + lo = x to ~16 bits (row pitch padded to 8 elements for TMA)."""
    r, c = x32.shape
    cp = -(-c // 8) * 8
    hi = torch.zeros(r, cp, dtype=torch.bfloat16, device=x32.device)[:, :c]
    lo = torch.zeros(r, cp, dtype=torch.bfloat16, device=x32.device)[:, :c]
    hi.copy_(x32)
    lo.copy_(x32 - hi.float())
    return hi, lo


def _mm3(a32: torch.Tensor, b32: torch.Tensor, *, alpha=1.0, beta=0.0, d=None, diag=0.0) -> torch.Tensor:
    """alpha * a @ b.T + beta * d + diag * I in fp32 from three bf16 tensor-core products (hi.hi + hi.lo + lo.hi): the dropped
    lo.lo term is 2^-16 of the result, so the product carries ~16 bits instead of bf16's 8."""
    ah, al = _split(a32)
    bh, bl = _split(b32)
    m, n = a32.shape[0], b32.shape[0]
    out = torch.empty(m, -(-n // 4) * 4, dtype=torch.float32, device=a32.device)[:, :n]
    gemm_tn(ah, bl, out=out, alpha=alpha, beta=beta, d=d, diag=diag)
    gemm_tn(al, bh, out=out, alpha=alpha, beta=1.0, d=out)
    gemm_tn(ah, bh, out=out, alpha=alpha, beta=1.0, d=out)
    return out


def newton_schulz(X: torch.Tensor, steps: int, coeffs, precision: str = "bf16") -> torch.Tensor:
    """X <- aX + b(XX^T)X + c(XX^T)^2X, `steps` times, on the tcgen05 GEMM.  X fp32 [r,c] -> fp32 [r,c].

    rows >= cols: right-Gram form  G = X^T X, P = aI + bG + cG^2, X <- X P   (cols^2-sized intermediates);
    rows <  cols: left form        A = X X^T, Q = aI + bA + cA^2, X <- Q X.
    ``precision="bf16"``: operands are rounded to bf16 once per product (fp32 accumulation in TMEM); X and X^T are both kept,
    so every GEMM is K-major on both operands.  The reference iterates in fp32 (``torch::mm`` with TF32 off, reference
    csrc/ops.cpp:713-727); the bf16 iteration differs from it by a few per cent in Frobenius norm, which Muon tolerates (the
    iteration is a contraction towards the orthogonal factor).  ``precision="bf16x3"``: every product is three bf16 products of
    hi / lo splits with fp32 results carried between the products (~16 bits per product, 3x the tensor-core work): within
    2e-3 of the fp32 iteration, for callers who want the reference's numerics.
    """
    if precision not in ("bf16", "bf16x3"):
        raise ValueError("precision must be 'bf16' or 'bf16x3'")
    a, b, c = coeffs
    r, cc = X.shape
    if precision == "bf16x3":
        X32 = X.float().contiguous()
        tall = r >= cc
        for _ in range(steps):
            src = X32.t().contiguous() if tall else X32                  # Gram matrix of the short side
            G = _mm3(src, src)
            Pm = _mm3(G, G, alpha=c, beta=b, d=G, diag=a)                # symmetric
            X32 = _mm3(X32, Pm) if tall else _mm3(Pm, X32.t().contiguous())
        return X32
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
    # ping-pong operand buffers allocated once per call (not once per iteration)
    Xn = torch.empty(r, cp, dtype=torch.bfloat16, device=dev)[:, :cc]
    XTn = torch.empty(cc, rp, dtype=torch.bfloat16, device=dev)[:, :r]
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
            if tall:
                gemm_tn(Xb, P, out=Xn, out_t=XTn)
            else:
                gemm_tn(P, XTb, out=Xn, out_t=XTn)
            Xb, Xn = Xn, Xb
            XTb, XTn = XTn, XTb
    return out32
