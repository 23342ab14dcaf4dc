"""Llama-style decoder for the Muon benchmark: RMSNorm, rotary position embedding, causal attention,
SwiGLU MLP, untied output head.  The 1.3 B configuration is 24 layers, d_model 2048, 16 heads, MLP 5504,
vocabulary 32000 (1,345,423,360 parameters, 168 two-dimensional block weights)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import nn_ops


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
        return nn_ops.rms_norm(x, None, self.weight, self.eps)

    def add_norm(self, x, residual):
        """(RMSNorm(x + residual), x + residual); on CUDA one kernel does the add, the statistics and the scaling."""
        if residual is None:
            return self.forward(x), x
        return nn_ops.norm_residual(x, residual, self.weight, None, self.eps, rms=True)


def rope_tables(seq, hd, theta, device, dtype=torch.float32):
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        d = cfg.d_model
        self.h = cfg.n_heads
        self.attn_norm, self.mlp_norm = RMSNorm(d, cfg.eps), RMSNorm(d, cfg.eps)
        self.wq, self.wk, self.wv, self.wo = (nn.Linear(d, d, bias=False) for _ in range(4))
        self.w_gate, self.w_up = nn.Linear(d, cfg.d_ff, bias=False), nn.Linear(d, cfg.d_ff, bias=False)
        self.w_down = nn.Linear(cfg.d_ff, d, bias=False)

    def forward(self, x, pending, cos, sin):
        """The residual stream entering the block is x + pending (pending = the previous block's MLP output, not yet added:
        the add is fused into this block's first norm).  Returns the same pair for the next block."""
        B, S, D = x.shape
        y, x = self.attn_norm.add_norm(x, pending)
        q, k, v = (w(y).view(B, S, self.h, D // self.h) for w in (self.wq, self.wk, self.wv))
        q, k = nn_ops.rope(q, cos, sin), nn_ops.rope(k, cos, sin)
        o = nn_ops.attention(q, k, v, causal=True)                      # [B, S, H, hd]
        y, x = self.mlp_norm.add_norm(self.wo(o.reshape(B, S, D)), x)
        return x, self.w_down(nn_ops.swiglu(self.w_gate(y), self.w_up(y)))


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
        h = nn_ops.embedding(ids, self.embed.weight)
        pending = None
        for l in self.layers:
            h, pending = l(h, pending, cos, sin)
        return self.lm_head(self.norm.add_norm(h, pending)[0])

    def matrix_params(self):
        """2-D weights of the blocks (Muon group); everything else (embedding, head, norms) goes to AdamW."""
        return [p for l in self.layers for p in l.parameters() if p.dim() == 2]

    def other_params(self):
        ids = {id(p) for p in self.matrix_params()}
        return [p for p in self.parameters() if id(p) not in ids]
