"""Autograd wrappers of the model-side sm_100a kernels (``csrc/nn_kernels.cu``).

``attention_small(qkv, n_heads)``   causal self-attention for S in {4, 8}, head_dim in {32, 64}; qkv is the
                                    fused projection [B, S, 3*D] and the gradient comes back in the same layout.
``layer_norm(x, residual, w, b)``   LayerNorm(x + residual) with the add fused in; backward is deterministic.
``rms_norm(x, residual, w)``        RMSNorm(x + residual), same kernels with the mean fixed at zero.
``rope(x, cos, sin)``               rotary position embedding of [B, S, H, hd] (interleaved pairs).
``swiglu(gate, up)``                silu(gate) * up in one pass; ``gelu(x)`` exact GELU.
``embedding(ids, weight)``          row gather; the gradient is a deterministic sorted segment sum (no atomics).
``cross_entropy(logits, target)``   mean softmax cross-entropy with ``ignore_index``; forward reads the logits once.
``linear(x, w, b)`` / ``grad_sink``  F.linear whose backward, inside a ``grad_sink`` block, adds the weight and bias gradients
                                    straight into ``w.grad`` / ``b.grad`` (the wgrad GEMM runs with beta = 1 on a side stream,
                                    next to the dgrad GEMM) instead of returning them for a separate accumulation kernel.
All fall back to the equivalent PyTorch expression on CPU tensors (used by the CPU tests as the oracle).
"""
from __future__ import annotations

import contextlib
import os
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


class _GradSink:
    """State of the gradient sink.  While ``on``, the backward functions of this module add parameter gradients to the
    parameters' ``.grad`` tensors themselves and return None for them: autograd then launches no accumulation kernel (one per
    parameter otherwise) and allocates no temporary.  ``stream``: side stream of the weight-gradient GEMMs; ``keep`` holds
    their operands until the main stream has waited for them, so the caching allocator cannot hand the memory out earlier."""

    def __init__(self):
        self.on, self.stream, self.forked, self.keep = False, None, False, []

    def join(self):
        if self.forked:
            torch.cuda.current_stream().wait_stream(self.stream)
            self.forked = False
        self.keep = []


_SINK = _GradSink()


@contextlib.contextmanager
def grad_sink(enabled: bool = True, side_stream: Optional["torch.cuda.Stream"] = None):
    """Inside the block, ``linear`` and ``layer_norm`` write parameter gradients in place (see ``_GradSink``).  The caller
    guarantees that every ``.grad`` involved exists, is zero or holds this step's earlier contributions, and that nothing
    relies on autograd's accumulation hooks.  Leaving the block joins the side stream."""
    prev = (_SINK.on, _SINK.stream)
    _SINK.on, _SINK.stream = enabled, side_stream
    try:
        yield _SINK
    finally:
        _SINK.join()
        _SINK.on, _SINK.stream = prev


def _sink_target(p: Optional[torch.Tensor], like: torch.Tensor) -> Optional[torch.Tensor]:
    g = None if p is None else p.grad
    return g if g is not None and g.dtype == like.dtype and g.is_contiguous() and g.device == like.device else None


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, bias, eps, rms=False):
        C = _build.require()
        y, z, stats = C.ln_fwd(x.contiguous(), residual, weight, bias, eps, rms)
        ctx.save_for_backward(z, weight, stats)
        ctx.has_bias, ctx.has_res, ctx.rms = bias is not None, residual is not None, rms
        ctx.params = (weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        z, weight, stats = ctx.saved_tensors
        C = _build.require()
        if _SINK.on:
            gw, gb = _sink_target(ctx.params[0], z), _sink_target(ctx.params[1], z)
            if gw is not None and (gb is not None or not ctx.has_bias):
                dz = C.ln_bwd(z, dy, weight, stats, ctx.has_bias, ctx.rms, None, gw, gb)[0]
                return dz, (dz if ctx.has_res else None), None, None, None, None
        dz, dg, db = C.ln_bwd(z, dy, weight, stats, ctx.has_bias, ctx.rms)
        return dz, (dz if ctx.has_res else None), dg, (db if ctx.has_bias else None), None, None


def _tc_linear_ok(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> bool:
    """Shapes the tcgen05 GEMM takes without copies: bf16, 16-byte row pitches, at least one full tile of rows."""
    return (x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x2.shape[0] >= 128 and x2.shape[1] % 8 == 0
            and weight.shape[0] % 8 == 0 and x2.is_contiguous() and weight.is_contiguous() and (bias is None or bias.dtype == torch.bfloat16))


class _LinearSink(torch.autograd.Function):
    """F.linear; the backward adds dW = dy^T x into ``weight.grad`` with the GEMM's beta = 1 and db into ``bias.grad``, on the
    sink's side stream when it has one, while the dgrad GEMM runs on the main stream.  With SG_LINEAR=tcgen05 the three GEMMs
    run on the hand-written tcgen05 kernel (bias in the forward epilogue, W / dy / x read where they are through MN-major
    descriptors, beta = 1 accumulation in the wgrad epilogue) instead of cuBLAS."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.params = (weight, bias)
        x2 = x.reshape(-1, x.shape[-1])
        ctx.tc = os.environ.get("SG_LINEAR", "cublas") == "tcgen05" and _tc_linear_ok(x2, weight, bias)
        if ctx.tc:
            from . import gemm
            return gemm.gemm_tn(x2, weight, bias=bias, out_dtype=torch.bfloat16).view(*x.shape[:-1], weight.shape[0])
        return F.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        wp, bp = ctx.params
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        gw = _sink_target(wp, dy2) if _SINK.on else None
        gb = _sink_target(bp, dy2) if _SINK.on else None
        if gw is None or (bp is not None and gb is None):
            dx = (dy2 @ weight).view(x.shape) if ctx.needs_input_grad[0] else None
            return dx, dy2.t() @ x2, (dy2.sum(0) if bp is not None else None)
        tc = ctx.tc and dy2.is_contiguous()
        _SINK.join()                                   # the previous layer's side work becomes a dependency; its operands are released
        side = _SINK.stream if dy2.is_cuda else None
        if side is not None:
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                _param_grads(gw, gb, dy2, x2, tc)
            _SINK.keep, _SINK.forked = [dy2, x2], True
        else:
            _param_grads(gw, gb, dy2, x2, tc)
        dx = None
        if ctx.needs_input_grad[0]:
            if tc:
                from . import gemm
                dx = gemm.gemm_tn(dy2, weight, out_dtype=torch.bfloat16, b_t=True).view(x.shape)      # dy [M,N] @ W [N,K]
            else:
                dx = (dy2 @ weight).view(x.shape)
        return dx, None, None


def _param_grads(gw, gb, dy2, x2, tc=False):
    if tc:
        from . import gemm
        # dy^T [N,M] @ x [M,K] added to the gradient buffer in the epilogue; own split-K scratch: the dgrad GEMM runs concurrently
        gemm.gemm_tn(dy2, x2, out=gw, beta=1.0, d=gw, a_t=True, b_t=True, ws_slot=1)
    else:
        gw.addmm_(dy2.t(), x2)                                         # the GEMM's beta = 1: no temporary, no separate add
    if gb is not None:
        if dy2.is_cuda and dy2.stride(-1) == 1 and dy2.dtype in (torch.bfloat16, torch.float32, torch.float16):
            _build.require().col_sum(dy2, gb)                          # two-stage fp32 column sum added to the bias gradient
        else:
            gb.add_(dy2.sum(0))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``F.linear``; inside a ``grad_sink`` block the parameter gradients go straight into ``.grad``.  SG_LINEAR=tcgen05 routes the
    GEMMs of bf16 CUDA layers through ``csrc/gemm_sm100.cu`` (inside and outside the sink)."""
    if _SINK.on and torch.is_grad_enabled() and weight.requires_grad and weight.grad is not None:
        return _LinearSink.apply(x, weight, bias)
    if x.is_cuda and x.dtype == torch.bfloat16 and os.environ.get("SG_LINEAR", "cublas") == "tcgen05":
        from . import gemm
        return gemm.linear(x, weight, bias)
    return F.linear(x, weight, bias)


def layer_norm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, bias: Optional[torch.Tensor],
               eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm(x + residual) over the last dimension (residual may be None)."""
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32) or x.shape[-1] % 4 or x.shape[-1] > 3072:
        z = x if residual is None else x + residual
        return F.layer_norm(z, (x.shape[-1],), weight, bias, eps)
    return _LayerNorm.apply(x, residual, weight, bias, eps)


class _NormResidual(torch.autograd.Function):
    """(y, z) = (norm(x + residual), x + residual): z is the new residual stream, so its own gradient joins the norm's input gradient
    inside the backward kernel."""

    @staticmethod
    def forward(ctx, x, residual, weight, bias, eps, rms):
        y, z, stats = _build.require().ln_fwd(x.contiguous(), residual.contiguous(), weight, bias, eps, rms)
        ctx.save_for_backward(z, weight, stats)
        ctx.has_bias, ctx.rms = bias is not None, rms
        return y, z

    @staticmethod
    def backward(ctx, dy, dz_out):
        z, weight, stats = ctx.saved_tensors
        dz, dg, db = _build.require().ln_bwd(z, dy, weight, stats, ctx.has_bias, ctx.rms, dz_out)
        return dz, dz, dg, (db if ctx.has_bias else None), None, None


def _norm_native(x, weight):
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] % 4 == 0 and x.shape[-1] <= 3072 and weight.dtype == x.dtype


def norm_residual(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float = 1e-5,
                  rms: bool = False):
    """Returns (norm(x + residual), x + residual) from one pass over x and residual."""
    if not _norm_native(x, weight):
        z = x + residual
        y = F.rms_norm(z, (x.shape[-1],), weight, eps) if rms else F.layer_norm(z, (x.shape[-1],), weight, bias, eps)
        return y, z
    return _NormResidual.apply(x, residual, weight, bias, eps, rms)


def attention_reference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """q, k, v: [B, S, H, hd] -> [B, S, H, hd]."""
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal)
    return o.transpose(1, 2)


def flash_supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    """The tcgen05 kernel takes bf16 [B, S, H, hd] views with S a multiple of 128, hd 64 or 128, adjacent heads and one position stride."""
    if not (q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape == k.shape == v.shape):
        return False
    B, S, H, HD = q.shape
    if S % 128 or HD not in (64, 128):
        return False
    for t in (q, k, v):
        if t.stride(3) != 1 or t.stride(2) != HD or t.stride(1) != q.stride(1) or t.stride(0) != S * t.stride(1) or t.stride(1) % 8 or t.data_ptr() % 16:
            return False
    return True


class _FlashAttention(torch.autograd.Function):
    """Forward and backward on the tcgen05 kernels of ``csrc/flash_attn_sm100.cu`` (the forward also returns the row
    log-sum-exp that the backward needs; nothing of size S x S is ever stored)."""

    @staticmethod
    def forward(ctx, q, k, v, causal):
        from . import gemm as _gemm
        out, lse = _build.require().flash_fwd(q, k, v, causal, _gemm._err_flag(q.device))
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal = causal
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import gemm as _gemm
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = _build.require().flash_bwd(q, k, v, out, lse, dout, ctx.causal, _gemm._err_flag(q.device))
        return dq, dk, dv, None


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, impl: Optional[str] = None) -> torch.Tensor:
    """Multi-head attention over [B, S, H, hd] tensors (heads stay in the projection layout, no transposes).

    ``impl`` (default: environment variable ``SG_ATTN``, else "sdpa"): "tcgen05" runs the forward pass on this package's flash
    attention kernel when the shapes allow it; "sdpa" calls ``F.scaled_dot_product_attention``, which is ~3x faster at sequence
    2048 on B200 (measured) and therefore the default of the training path."""
    import os
    impl = impl or os.environ.get("SG_ATTN", "sdpa")
    if impl == "tcgen05" and flash_supported(q, k, v):
        return _FlashAttention.apply(q, k, v, causal)
    return attention_reference(q, k, v, causal)


def _native_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32)


def rms_norm(x: torch.Tensor, residual: Optional[torch.Tensor], weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """RMSNorm(x + residual) over the last dimension (residual may be None)."""
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32) or x.shape[-1] % 4 or x.shape[-1] > 3072 or weight.dtype != x.dtype:
        z = x if residual is None else x + residual
        return F.rms_norm(z, (x.shape[-1],), weight, eps)
    return _LayerNorm.apply(x, residual, weight, None, eps, True)


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, S, H, hd]; cos/sin [S, hd/2]; pairs (2i, 2i+1) rotate by the position angle."""
    x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
    c, s = cos[None, : x.shape[1], None], sin[None, : x.shape[1], None]
    return torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], -1).flatten(-2).to(x.dtype)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        return _build.require().rope(x.contiguous(), cos, sin, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return _build.require().rope(dy.contiguous(), cos, sin, True), None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    if not _native_ok(x) or x.shape[-1] % 8:
        return rope_reference(x, cos, sin)
    return _Rope.apply(x, cos.float().contiguous(), sin.float().contiguous())


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        g, u = g.contiguous(), u.contiguous()
        ctx.save_for_backward(g, u)
        return _build.require().swiglu_fwd(g, u)

    @staticmethod
    def backward(ctx, dy):
        g, u = ctx.saved_tensors
        dg, du = _build.require().swiglu_bwd(g, u, dy)
        return dg, du


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if not _native_ok(gate) or gate.numel() % 8 or gate.dtype != up.dtype:
        return F.silu(gate) * up
    return _SwiGLU.apply(gate, up)


class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        ctx.save_for_backward(x)
        return _build.require().gelu_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return _build.require().gelu_bwd(x, dy)


def gelu(x: torch.Tensor) -> torch.Tensor:
    if not _native_ok(x) or x.numel() % 8:
        return F.gelu(x)
    return _Gelu.apply(x)


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        ids = ids.contiguous()
        ctx.save_for_backward(ids)
        ctx.vocab, ctx.table = weight.shape[0], weight
        return _build.require().embedding_fwd(ids, weight)

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        gw = _sink_target(ctx.table, dout) if _SINK.on else None
        if gw is not None:
            _build.require().embedding_bwd(ids, dout, ctx.vocab, gw)
            return None, None
        return None, _build.require().embedding_bwd(ids, dout, ctx.vocab)


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if (not _native_ok(weight) or not weight.is_contiguous() or (weight.shape[1] * weight.element_size()) % 16 or weight.shape[1] % 8
            or ids.dtype != torch.int64 or ids.device != weight.device):
        return F.embedding(ids, weight)
    return _Embedding.apply(ids, weight)


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, ignore_index):
        logits, target = logits.contiguous(), target.contiguous()
        loss, lse, mean_out = _build.require().ce_fwd(logits, target, ignore_index)
        ctx.save_for_backward(logits, target, lse, mean_out)
        ctx.ignore_index = ignore_index
        return loss

    @staticmethod
    def backward(ctx, gout):
        logits, target, lse, mean_out = ctx.saved_tensors
        return _build.require().ce_bwd(logits, target, lse, mean_out, gout.reshape(1), ctx.ignore_index), None, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean cross-entropy of logits [rows, V] against int64 targets [rows]; the result is an fp32 scalar."""
    if not _native_ok(logits) or logits.dim() != 2 or logits.shape[1] % 8:
        return F.cross_entropy(logits.float(), target, ignore_index=ignore_index)
    return _CrossEntropy.apply(logits, target, ignore_index)
