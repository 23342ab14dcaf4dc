"""Decoder transformers for the modular-arithmetic tasks.

``Transformer``  : the race driver's model (reference grokking_race_v2.py:310-331): token + position
  embeddings, post-LN blocks (x = LN(x + attn(x)); x = LN(x + MLP(x))), biases everywhere, GELU 4*d MLP,
  final LayerNorm, linear head on the LAST token only -> logits [B, ntok].  Parameter names and shapes
  match ``nn.MultiheadAttention``-based blocks (in_proj_weight [3d,d], in_proj_bias, out_proj) so the
  counts are those of the reference: 422,755 / 3,211,363 / 19,018,851 for the small / medium / large scale.
``PreLNTransformer`` : bias-free pre-LN variant with a tied output head and a parameter-free final norm:
  2 + 6*layers tensors (26 tensors, about 3.17 M parameters at d=256, 4 layers).

``fused=True`` routes Linear / LayerNorm / attention / cross-entropy through the hand-written sm_100a
kernels of ``supergrok15_b200.ops.nn_ops``; the default uses plain PyTorch modules (needed on CPU).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

import os

from ..ops import nn_ops


def _linear(x, weight, bias):
    """nn.Linear forward: ``nn_ops.linear`` (gradient sink inside the engine; SG_LINEAR=tcgen05 puts the three GEMMs of the layer
    on the hand-written tcgen05 kernel instead of cuBLAS)."""
    return nn_ops.linear(x, weight, bias)


class _Attn(nn.Module):
    """Causal multi-head self-attention with MultiheadAttention's parameter layout."""

    def __init__(self, d: int, h: int, bias: bool = True):
        super().__init__()
        assert d % h == 0
        self.d, self.h = d, h
        self.fused = True            # use the short-sequence attention kernel when the input qualifies (CUDA, S in {4,8})
        self.in_proj_weight = nn.Parameter(torch.empty(3 * d, d))
        self.in_proj_bias = nn.Parameter(torch.zeros(3 * d)) if bias else None
        self.out_proj = nn.Linear(d, d, bias=bias)
        nn.init.xavier_uniform_(self.in_proj_weight)
        if bias:
            nn.init.zeros_(self.out_proj.bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, D = x.shape
        qkv = _linear(x, self.in_proj_weight, self.in_proj_bias)
        if self.fused and nn_ops.attention_small_supported(qkv, self.h):
            return _linear(nn_ops.attention_small(qkv, self.h, True), self.out_proj.weight, self.out_proj.bias)
        qkv = qkv.view(B, S, 3, self.h, D // self.h)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.out_proj(o.transpose(1, 2).reshape(B, S, D))


class DecoderBlock(nn.Module):
    def __init__(self, d: int, h: int, seq_len: int = 4):
        super().__init__()
        self.attn = _Attn(d, h)
        self.n1, self.n2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.ff = nn.Sequential(nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d))

    def forward(self, x):
        if x.is_cuda:                    # LayerNorm(x + sublayer) with the add fused into the normalisation kernel
            x = nn_ops.layer_norm(x, self.attn(x), self.n1.weight, self.n1.bias, self.n1.eps)
            u = _linear(x, self.ff[0].weight, self.ff[0].bias)
            h = nn_ops.gelu(u) if u.dtype != torch.float32 else F.gelu(u)   # 16-bit: the kernel with the cheaper erf
            return nn_ops.layer_norm(x, _linear(h, self.ff[2].weight, self.ff[2].bias), self.n2.weight, self.n2.bias, self.n2.eps)
        x = self.n1(x + self.attn(x))
        return self.n2(x + self.ff(x))


class Transformer(nn.Module):
    def __init__(self, nl: int = 2, d: int = 128, h: int = 4, ntok: int = 99, seq: int = 4):
        super().__init__()
        self.tok, self.pos = nn.Embedding(ntok, d), nn.Embedding(seq, d)
        self.layers = nn.ModuleList([DecoderBlock(d, h, seq) for _ in range(nl)])
        self.norm = nn.LayerNorm(d)
        self.out = nn.Linear(d, ntok)
        self.register_buffer("pos_ids", torch.arange(seq).unsqueeze(0), persistent=False)

    def forward(self, x):
        if x.is_cuda:        # token gather and (in backward) its small-table gradient kernel; final LayerNorm on the fused kernel
            h = nn_ops.embedding(x, self.tok.weight) + self.pos(self.pos_ids[:, : x.shape[1]])
            for l in self.layers:
                h = l(h)
            last = nn_ops.layer_norm(h[:, -1].contiguous(), None, self.norm.weight, self.norm.bias, self.norm.eps)
            return _linear(last, self.out.weight, self.out.bias)
        h = self.tok(x) + self.pos(self.pos_ids[:, : x.shape[1]])
        for l in self.layers:
            h = l(h)
        return _linear(self.norm(h[:, -1]), self.out.weight, self.out.bias)


class PreLNBlock(nn.Module):
    def __init__(self, d: int, h: int):
        super().__init__()
        self.n1 = nn.LayerNorm(d, bias=False)
        self.attn = _Attn(d, h, bias=False)
        self.n2 = nn.LayerNorm(d, bias=False)
        self.fc1 = nn.Linear(d, 4 * d, bias=False)
        self.fc2 = nn.Linear(4 * d, d, bias=False)

    def forward(self, x):
        x = x + self.attn(self.n1(x))
        return x + self.fc2(F.gelu(self.fc1(self.n2(x))))


class PreLNTransformer(nn.Module):
    def __init__(self, nl: int = 2, d: int = 128, h: int = 4, ntok: int = 99, seq: int = 4):
        super().__init__()
        self.tok, self.pos = nn.Embedding(ntok, d), nn.Embedding(seq, d)
        self.layers = nn.ModuleList([PreLNBlock(d, h) for _ in range(nl)])
        self.d = d
        self.register_buffer("pos_ids", torch.arange(seq).unsqueeze(0), persistent=False)

    def forward(self, x):
        h = self.tok(x) + self.pos(self.pos_ids[:, : x.shape[1]])
        for l in self.layers:
            h = l(h)
        h = F.layer_norm(h[:, -1], (self.d,))
        return F.linear(h, self.tok.weight)
