"""Llama-style decoder for the Muon benchmark: RMSNorm, rotary position embedding, causal attention,
SwiGLU MLP, untied output head.  The 1.3 B configuration is 24 layers, d_model 2048, 16 heads, MLP 5504,
vocabulary 32000 (1,345,423,360 parameters, 168 two-dimensional block weights)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class LlamaConfig:
    n_layers: int = 24
    d_model: int = 2048
    n_heads: int = 16
    d_ff: int = 5504
    vocab: int = 32000
    max_seq: int = 2048
    rope_theta: float = 10000.0
    eps: float = 1e-5


LLAMA_1P3B = LlamaConfig()
LLAMA_TINY = LlamaConfig(n_layers=2, d_model=128, n_heads=4, d_ff=352, vocab=256, max_seq=64)


class RMSNorm(nn.Module):
    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rope_tables(seq, hd, theta, device, dtype=torch.float32):
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x, cos, sin):                     # x [B,H,S,hd]
    x1, x2 = x[..., 0::2], x[..., 1::2]
    c, s = cos[None, None], sin[None, None]
    return torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], -1).flatten(-2)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        d = cfg.d_model
        self.h = cfg.n_heads
        self.attn_norm, self.mlp_norm = RMSNorm(d, cfg.eps), RMSNorm(d, cfg.eps)
        self.wq, self.wk, self.wv, self.wo = (nn.Linear(d, d, bias=False) for _ in range(4))
        self.w_gate, self.w_up = nn.Linear(d, cfg.d_ff, bias=False), nn.Linear(d, cfg.d_ff, bias=False)
        self.w_down = nn.Linear(cfg.d_ff, d, bias=False)

    def forward(self, x, cos, sin):
        B, S, D = x.shape
        y = self.attn_norm(x)
        q, k, v = (w(y).view(B, S, self.h, D // self.h).transpose(1, 2) for w in (self.wq, self.wk, self.wv))
        q, k = apply_rope(q, cos, sin).to(v.dtype), apply_rope(k, cos, sin).to(v.dtype)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.wo(o.transpose(1, 2).reshape(B, S, D))
        y = self.mlp_norm(x)
        return x + self.w_down(F.silu(self.w_gate(y)) * self.w_up(y))


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig = LLAMA_1P3B):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab, cfg.d_model)
        self.layers = nn.ModuleList([LlamaBlock(cfg) for _ in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.d_model, cfg.eps)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab, bias=False)

    def forward(self, ids):
        B, S = ids.shape
        cos, sin = rope_tables(S, self.cfg.d_model // self.cfg.n_heads, self.cfg.rope_theta, ids.device)
        h = self.embed(ids)
        for l in self.layers:
            h = l(h, cos, sin)
        return self.lm_head(self.norm(h))

    def matrix_params(self):
        """2-D weights of the blocks (Muon group); everything else (embedding, head, norms) goes to AdamW."""
        return [p for l in self.layers for p in l.parameters() if p.dim() == 2]

    def other_params(self):
        ids = {id(p) for p in self.matrix_params()}
        return [p for p in self.parameters() if id(p) not in ids]
