"""ViT for the MNIST-addition task (reference grokking_race_v2.py:334-358): 16 patches x 49 pixels,
CLS token, post-LN encoder blocks (no causal mask), linear head on the CLS token -> [B, p]."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class _EncAttn(nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.h = h
        self.in_proj_weight = nn.Parameter(torch.empty(3 * d, d))
        self.in_proj_bias = nn.Parameter(torch.zeros(3 * d))
        self.out_proj = nn.Linear(d, d)
        nn.init.xavier_uniform_(self.in_proj_weight)

    def forward(self, x):
        B, S, D = x.shape
        qkv = F.linear(x, self.in_proj_weight, self.in_proj_bias).view(B, S, 3, self.h, D // self.h)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        return self.out_proj(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, S, D))


class EncoderBlock(nn.Module):
    def __init__(self, d, h):
        super().__init__()
        self.attn = _EncAttn(d, h)
        self.n1, self.n2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.ff = nn.Sequential(nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d))

    def forward(self, x):
        x = self.n1(x + self.attn(x))
        return self.n2(x + self.ff(x))


class ViT(nn.Module):
    def __init__(self, nl=2, d=128, h=4, p=97, patch_dim=49, num_patches=16):
        super().__init__()
        self.patch = nn.Linear(patch_dim, d)
        self.cls = nn.Parameter(torch.zeros(1, 1, d))
        self.pos = nn.Parameter(torch.randn(1, num_patches + 1, d) * 0.02)
        self.layers = nn.ModuleList([EncoderBlock(d, h) for _ in range(nl)])
        self.norm = nn.LayerNorm(d)
        self.out = nn.Linear(d, p)

    def forward(self, x):                       # x [B, patches, patch_dim]
        h = self.patch(x)
        h = torch.cat([self.cls.expand(h.shape[0], -1, -1), h], 1) + self.pos
        for l in self.layers:
            h = l(h)
        return self.out(self.norm(h[:, 0]))
