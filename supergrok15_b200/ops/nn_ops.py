"""Autograd wrappers of the model-side sm_100a kernels (``csrc/nn_kernels.cu``).

``attention_small(qkv, n_heads)``   causal self-attention for S in {4, 8}, head_dim in {32, 64}; qkv is the
                                    fused projection [B, S, 3*D] and the gradient comes back in the same layout.
``layer_norm(x, residual, w, b)``   LayerNorm(x + residual) with the add fused in; backward is deterministic.
Both fall back to the equivalent PyTorch expression on CPU tensors (used by the CPU tests as the oracle).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .. import _build


def attention_small_reference(qkv: torch.Tensor, n_heads: int, causal: bool = True) -> torch.Tensor:
    B, S, D3 = qkv.shape
    D = D3 // 3
    q, k, v = (t.transpose(1, 2) for t in qkv.view(B, S, 3, n_heads, D // n_heads).unbind(2))
    return F.scaled_dot_product_attention(q, k, v, is_causal=causal).transpose(1, 2).reshape(B, S, D)


class _AttnSmall(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, n_heads, causal):
        C = _build.require()
        qkv = qkv.contiguous()
        ctx.save_for_backward(qkv)
        ctx.n_heads, ctx.causal = n_heads, causal
        return C.attn_small_fwd(qkv, n_heads, causal)

    @staticmethod
    def backward(ctx, dout):
        (qkv,) = ctx.saved_tensors
        return _build.require().attn_small_bwd(qkv, dout, ctx.n_heads, ctx.causal), None, None


def attention_small_supported(qkv: torch.Tensor, n_heads: int) -> bool:
    if not qkv.is_cuda or qkv.dtype not in (torch.bfloat16, torch.float32):
        return False
    return qkv.shape[1] in (4, 8) and (qkv.shape[2] // 3) // n_heads in (32, 64)


def attention_small(qkv: torch.Tensor, n_heads: int, causal: bool = True) -> torch.Tensor:
    if not attention_small_supported(qkv, n_heads):
        return attention_small_reference(qkv, n_heads, causal)
    return _AttnSmall.apply(qkv, n_heads, causal)


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, bias, eps):
        C = _build.require()
        y, z, stats = C.ln_fwd(x.contiguous(), residual, weight, bias, eps)
        ctx.save_for_backward(z, weight, stats)
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        z, weight, stats = ctx.saved_tensors
        dz, dg, db = _build.require().ln_bwd(z, dy, weight, stats, ctx.has_bias)
        return dz, (dz if ctx.has_res else None), dg, (db if ctx.has_bias else None), None


def layer_norm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
               eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm(x + residual) over the last dimension (residual may be None)."""
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32) or x.shape[-1] % 4 or x.shape[-1] > 3072:
        z = x if residual is None else x + residual
        return F.layer_norm(z, (x.shape[-1],), weight, bias, eps)
    return _LayerNorm.apply(x, residual, weight, bias, eps)
