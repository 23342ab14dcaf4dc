"""Selective-SSM sequence model for the chained-division task (reference grokking_race_v2.py:361-415):
per layer LayerNorm -> in_proj (x, z) -> depthwise conv1d(k=3) -> SiLU -> selective scan -> gate -> out_proj,
residual.  The scan over the (short, <= 17 token) sequence is vectorised over batch and channels."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class SelectiveSSMLayer(nn.Module):
    def __init__(self, d: int, d_state: int = 16, expand: int = 2, dt_rank: int = 0):
        super().__init__()
        self.d_inner, self.d_state = d * expand, d_state
        self.dt_rank = dt_rank or max(1, math.ceil(d / 16))
        self.norm = nn.LayerNorm(d)
        self.in_proj = nn.Linear(d, 2 * self.d_inner, bias=False)
        self.conv = nn.Conv1d(self.d_inner, self.d_inner, 3, padding=2, groups=self.d_inner)
        self.x_proj = nn.Linear(self.d_inner, self.dt_rank + 2 * d_state, bias=False)
        self.dt_proj = nn.Linear(self.dt_rank, self.d_inner)
        self.A_log = nn.Parameter(torch.log(torch.arange(1, d_state + 1).float()).repeat(self.d_inner, 1))
        self.D = nn.Parameter(torch.ones(self.d_inner))
        self.out_proj = nn.Linear(self.d_inner, d, bias=False)

    def forward(self, u):                        # [B,S,d]
        B_, S, _ = u.shape
        x, z = self.in_proj(self.norm(u)).chunk(2, -1)
        x = F.silu(self.conv(x.transpose(1, 2))[..., :S].transpose(1, 2))
        dt, Bm, Cm = self.x_proj(x).split([self.dt_rank, self.d_state, self.d_state], -1)
        dt = F.softplus(self.dt_proj(dt))
        A = -torch.exp(self.A_log)
        h = x.new_zeros(B_, self.d_inner, self.d_state)
        ys = []
        for t in range(S):
            dA = torch.exp(dt[:, t].unsqueeze(-1) * A)
            h = dA * h + (dt[:, t] * x[:, t]).unsqueeze(-1) * Bm[:, t].unsqueeze(1)
            ys.append((h * Cm[:, t].unsqueeze(1)).sum(-1))
        y = torch.stack(ys, 1) + self.D * x
        return u + self.out_proj(y * F.silu(z))


class MambaModel(nn.Module):
    def __init__(self, nl=2, d=128, ntok=99, seq=8, d_state=16):
        super().__init__()
        self.tok = nn.Embedding(ntok, d)
        self.layers = nn.ModuleList([SelectiveSSMLayer(d, d_state) for _ in range(nl)])
        self.norm = nn.LayerNorm(d)
        self.out = nn.Linear(d, ntok)

    def forward(self, x):
        h = self.tok(x)
        for l in self.layers:
            h = l(h)
        return self.out(self.norm(h[:, -1]))
