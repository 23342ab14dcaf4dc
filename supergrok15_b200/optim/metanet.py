"""Meta-networks of the SuperGrok family, in plain PyTorch (autograd-capable oracle).

* ``SharpnessMetaNet``  : 2 -> H -> 1 GELU MLP used by SuperGrok v1.1 / v1.5
  (reference grokking_optimizers/supergrok15.py:25-64).
* ``Mamba3ScanBlock``   : selective scan with trapezoidal discretisation and paired RoPE
  (reference grokking_optimizers/mamba3_peer_metanet.py:44-160).  The reference calls the
  non-existent ``torch.softplus``; this class uses ``F.softplus`` (threshold 20, the same
  form the reference CUDA kernel uses, csrc/supergrok2_mamba_peer_kernels.cu:221).
* ``MiniGRU``           : 4-wide per-element GRU (mamba3_peer_metanet.py:163-192).
* ``Mamba3PEERMetaNet`` : input projection, bidirectional scan, GRU, 4-head product-key
  routing over 144 experts (mamba3_peer_metanet.py:195-567).  ``forward`` uses hard top-1
  routing (what the optimizer step uses); ``forward_for_bilevel`` uses soft top-4 routing.

Parameter names match the reference so a reference ``state_dict`` loads unchanged.

The scan is available in two algebraically equal forms: ``serial`` (one Python iteration per
timestep; the literal recurrence) and ``chunked`` (a work-efficient blocked prefix scan over
2x2 affine maps written with tensor ops, differentiable, used for long sequences).
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


class SharpnessMetaNet(nn.Module):
    """out = g + rescale * MLP([g, sharpness]);  weights N(0, 0.01^2), biases 0, rescale 0."""

    def __init__(self, hidden_dim: int = 32):
        super().__init__()
        self.hidden_dim = hidden_dim
        self.net = nn.Sequential(nn.Linear(2, hidden_dim), nn.GELU(), nn.Linear(hidden_dim, 1))
        self.rescale = nn.Parameter(torch.zeros(1))
        with torch.no_grad():
            self.net[0].weight.normal_(0, 0.01)
            self.net[0].bias.zero_()
            self.net[2].weight.normal_(0, 0.01)
            self.net[2].bias.zero_()

    def forward(self, grad: torch.Tensor, sharpness: torch.Tensor) -> torch.Tensor:
        if grad.numel() == 0:
            return grad
        shape = grad.shape
        inp = torch.stack([grad.reshape(-1), sharpness.reshape(-1)], dim=1)
        return (inp[:, :1] + self.rescale * self.net(inp)).reshape(shape)

    def get_weights(self):
        """(W1 [H,2], b1 [H], W2 [1,H], b2 [1], rescale float) as contiguous fp32 tensors."""
        return (self.net[0].weight.detach().float().contiguous(), self.net[0].bias.detach().float().contiguous(),
                self.net[2].weight.detach().float().contiguous(), self.net[2].bias.detach().float().contiguous(),
                float(self.rescale.detach().item()))


# --------------------------------------------------------------------------- affine scan helpers
def _compose(M2, b2, M1, b1):
    """(M2,b2) after (M1,b1) for stacked 2x2 maps: M = (a,b,c,d) rows [[a,b],[c,d]], bias (e,o)."""
    a2, b2_, c2, d2 = M2
    a1, b1_, c1, d1 = M1
    e2, o2 = b2
    e1, o1 = b1
    M = (a2 * a1 + b2_ * c1, a2 * b1_ + b2_ * d1, c2 * a1 + d2 * c1, c2 * b1_ + d2 * d1)
    b = (a2 * e1 + b2_ * o1 + e2, c2 * e1 + d2 * o1 + o2)
    return M, b


def affine_scan_chunked(M, b, h0_e, h0_o, chunk: int = 64):
    """Inclusive prefix application of h[t] = M[t] h[t-1] + b[t] over dim 0.

    ``M`` is a 4-tuple and ``b`` a 2-tuple of tensors shaped [N, ...]; ``h0_*`` are shaped [...].
    Returns (h_e [N,...], h_o [N,...]).  Work O(N), depth O(chunk * log_chunk N).
    """
    N = M[0].shape[0]
    if N <= chunk:
        he, ho = h0_e, h0_o
        outs_e, outs_o = [], []
        for t in range(N):
            he, ho = (M[0][t] * he + M[1][t] * ho + b[0][t], M[2][t] * he + M[3][t] * ho + b[1][t])
            outs_e.append(he)
            outs_o.append(ho)
        return torch.stack(outs_e), torch.stack(outs_o)
    L = chunk
    nc = (N + L - 1) // L
    pad = nc * L - N
    tail = M[0].shape[1:]

    def _pad(x, fill):
        if pad == 0:
            return x.reshape(nc, L, *tail)
        filler = torch.full((pad, *tail), fill, dtype=x.dtype, device=x.device)
        return torch.cat([x, filler], 0).reshape(nc, L, *tail)

    Mp = (_pad(M[0], 1.0), _pad(M[1], 0.0), _pad(M[2], 0.0), _pad(M[3], 1.0))   # identity padding
    bp = (_pad(b[0], 0.0), _pad(b[1], 0.0))
    # local inclusive prefixes inside every chunk (sequential over L, vectorised over chunks)
    cm = tuple(x[:, 0] for x in Mp)
    cb = tuple(x[:, 0] for x in bp)
    pm, pb = [cm], [cb]
    for t in range(1, L):
        cm, cb = _compose(tuple(x[:, t] for x in Mp), tuple(x[:, t] for x in bp), cm, cb)
        pm.append(cm)
        pb.append(cb)
    # carry-in state of every chunk = scan over chunk aggregates (recursive)
    agg_e, agg_o = affine_scan_chunked(cm, cb, h0_e, h0_o, chunk)        # state at the END of each chunk
    in_e = torch.cat([h0_e.unsqueeze(0).expand(1, *tail), agg_e[:-1]], 0)
    in_o = torch.cat([h0_o.unsqueeze(0).expand(1, *tail), agg_o[:-1]], 0)
    PM = tuple(torch.stack([m[i] for m in pm], 1) for i in range(4))     # [nc, L, ...]
    PB = tuple(torch.stack([x[i] for x in pb], 1) for i in range(2))
    he = PM[0] * in_e.unsqueeze(1) + PM[1] * in_o.unsqueeze(1) + PB[0]
    ho = PM[2] * in_e.unsqueeze(1) + PM[3] * in_o.unsqueeze(1) + PB[1]
    return he.reshape(nc * L, *tail)[:N], ho.reshape(nc * L, *tail)[:N]


class Mamba3ScanBlock(nn.Module):
    def __init__(self, d_model: int = 8, d_state: int = 16, expand: int = 2):
        super().__init__()
        assert d_state % 2 == 0, "d_state must be even for paired RoPE"
        self.d_model, self.d_state, self.d_inner = d_model, d_state, d_model * expand
        self.in_proj = nn.Linear(d_model, 2 * self.d_inner, bias=False)
        self.dt_proj = nn.Linear(self.d_inner, self.d_inner, bias=True)
        self.B_proj = nn.Linear(self.d_inner, d_state, bias=False)
        self.C_proj = nn.Linear(self.d_inner, d_state, bias=False)
        self.A_log = nn.Parameter(torch.log(torch.linspace(1, d_state, d_state)).unsqueeze(0).repeat(self.d_inner, 1))
        self.D = nn.Parameter(torch.ones(self.d_inner))
        self.rope_freq = nn.Parameter(torch.randn(self.d_inner, d_state // 2) * 0.01)
        self.out_proj = nn.Linear(self.d_inner, d_model, bias=False)

    def precompute(self, x: torch.Tensor):
        xz = self.in_proj(x)
        xb, z = xz.chunk(2, dim=-1)
        dt = F.softplus(self.dt_proj(xb))
        return xb, z, dt, self.B_proj(xb), self.C_proj(xb)

    def step_maps(self, xb, dt, B):
        """Per-timestep 2x2 affine maps, each [N, d_inner, d_state/2]."""
        A = -torch.exp(self.A_log)                                   # [J,S]
        dtA = dt.unsqueeze(-1) * A / 2.0                              # [N,J,S]
        Abar = (1.0 + dtA) / (1.0 - dtA + 1e-8)
        ang = dt.unsqueeze(-1) * self.rope_freq                       # [N,J,S/2]
        c, s = torch.cos(ang), torch.sin(ang)
        Ae, Ao = Abar[..., 0::2], Abar[..., 1::2]
        M = (Ae * c, -Ae * s, Ao * s, Ao * c)
        bx = (dt * xb).unsqueeze(-1) * B.unsqueeze(1)                  # [N,J,S]
        return M, (bx[..., 0::2], bx[..., 1::2])

    def forward(self, x: torch.Tensor, initial_state: Optional[torch.Tensor] = None, impl: str = "auto",
                return_inner: bool = False):
        """x [N, d_model] -> (out [N, d_model], final_state [d_inner, d_state])."""
        N = x.shape[0]
        h0 = (initial_state.to(x.dtype) if initial_state is not None
              else torch.zeros(self.d_inner, self.d_state, device=x.device, dtype=x.dtype))
        if N == 0:
            return x.new_zeros(0, self.d_model), h0
        xb, z, dt, B, C = self.precompute(x)
        if impl == "auto":
            impl = "serial" if N <= 32 else "chunked"
        if impl == "serial":
            A = -torch.exp(self.A_log)
            h = h0
            ys = []
            for t in range(N):
                dti = dt[t].unsqueeze(-1)
                Abar = (1.0 + dti * A / 2.0) / (1.0 - dti * A / 2.0 + 1e-8)
                ang = dti * self.rope_freq
                c, s = torch.cos(ang), torch.sin(ang)
                he, ho = h[:, 0::2], h[:, 1::2]
                hr = torch.stack([he * c - ho * s, ho * c + he * s], dim=-1).reshape(self.d_inner, self.d_state)
                h = Abar * hr + (dti * B[t].unsqueeze(0)) * xb[t].unsqueeze(-1)
                ys.append((h * C[t].unsqueeze(0)).sum(-1))
            y = torch.stack(ys)
            final = h
        else:
            M, b = self.step_maps(xb, dt, B)
            he, ho = affine_scan_chunked(M, b, h0[:, 0::2], h0[:, 1::2])
            y = (he * C[:, 0::2].unsqueeze(1)).sum(-1) + (ho * C[:, 1::2].unsqueeze(1)).sum(-1)
            final = torch.stack([he[-1], ho[-1]], dim=-1).reshape(self.d_inner, self.d_state)
        y = y * F.silu(z) + self.D.unsqueeze(0) * xb
        if return_inner:
            return y, final
        return self.out_proj(y), final


class MiniGRU(nn.Module):
    def __init__(self, input_dim: int, hidden_dim: int = 4):
        super().__init__()
        self.hidden_dim = hidden_dim
        self.W_z = nn.Linear(input_dim + hidden_dim, hidden_dim)
        self.W_r = nn.Linear(input_dim + hidden_dim, hidden_dim)
        self.W_h = nn.Linear(input_dim + hidden_dim, hidden_dim)

    def forward(self, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        xh = torch.cat([x, h], dim=-1)
        z = torch.sigmoid(self.W_z(xh))
        r = torch.sigmoid(self.W_r(xh))
        cand = torch.tanh(self.W_h(torch.cat([x, r * h], dim=-1)))
        return (1 - z) * h + z * cand


class Mamba3PEERMetaNet(nn.Module):
    def __init__(self, d_model: int = 8, d_state: int = 16, mamba_expand: int = 2, num_peer_heads: int = 4,
                 num_experts: int = 144, expert_hidden: int = 16, gru_hidden: int = 4, rescale: float = 0.1,
                 recycle_interval: int = 100, recycle_threshold: float = 0.001):
        super().__init__()
        self.d_model, self.d_state = d_model, d_state
        self.num_peer_heads, self.num_experts = num_peer_heads, num_experts
        self.expert_hidden, self.gru_hidden = expert_hidden, gru_hidden
        self.rescale = rescale
        self.recycle_interval, self.recycle_threshold = recycle_interval, recycle_threshold
        self.pk_dim = int(math.isqrt(num_experts))
        assert self.pk_dim * self.pk_dim == num_experts, f"num_experts must be a perfect square, got {num_experts}"
        self.input_proj = nn.Linear(2, d_model, bias=True)
        self.mamba_fwd = Mamba3ScanBlock(d_model, d_state, mamba_expand)
        self.mamba_bwd = Mamba3ScanBlock(d_model, d_state, mamba_expand)
        self.gru = MiniGRU(2 + 2 * d_model, gru_hidden)
        peer_in = gru_hidden + 2 * d_model + 2
        self.peer_queries = nn.ModuleList([nn.Linear(peer_in, d_model, bias=False) for _ in range(num_peer_heads)])
        self.product_keys_A = nn.ParameterList(
            [nn.Parameter(torch.randn(self.pk_dim, d_model // 2) * 0.02) for _ in range(num_peer_heads)])
        self.product_keys_B = nn.ParameterList(
            [nn.Parameter(torch.randn(self.pk_dim, d_model // 2) * 0.02) for _ in range(num_peer_heads)])
        self.expert_W1 = nn.Parameter(torch.randn(num_experts, expert_hidden, 1) * 0.02)
        self.expert_b1 = nn.Parameter(torch.zeros(num_experts, expert_hidden))
        self.expert_W2 = nn.Parameter(torch.randn(num_experts, 1, expert_hidden) * 0.02)
        self.expert_b2 = nn.Parameter(torch.zeros(num_experts, 1))
        self.register_buffer("expert_counts", torch.zeros(num_experts, dtype=torch.int32))
        self.register_buffer("step_counter", torch.tensor(0, dtype=torch.long))

    # ------------------------------------------------------------------ shared front part
    def _contexts(self, g, s, fwd_state, bwd_state, impl):
        sort_idx = torch.argsort(g.abs(), stable=True)
        x = self.input_proj(torch.stack([g[sort_idx], s[sort_idx]], dim=-1))
        fwd_out, new_fwd = self.mamba_fwd(x, fwd_state, impl)
        bwd_out, new_bwd = self.mamba_bwd(x.flip(0), bwd_state, impl)
        bwd_out = bwd_out.flip(0)
        unsort = torch.empty_like(sort_idx)
        unsort[sort_idx] = torch.arange(sort_idx.numel(), device=sort_idx.device)
        return fwd_out[unsort], bwd_out[unsort], new_fwd, new_bwd

    def _expert_out(self, g, idx):
        """Evaluate expert ``idx`` ([N] or [N,K]) on scalar input g ([N]); returns same shape as idx."""
        W1 = self.expert_W1.squeeze(-1)[idx]
        z = torch.relu(W1 * g.reshape(-1, *([1] * (idx.dim()))) + self.expert_b1[idx])
        return (z * self.expert_W2.squeeze(1)[idx]).sum(-1) + self.expert_b2.squeeze(-1)[idx]

    def forward(self, grad, sharpness, gru_state, mamba_fwd_state=None, mamba_bwd_state=None, impl: str = "auto"):
        g = grad.reshape(-1).float()
        s = sharpness.reshape(-1).float()
        fwd_ctx, bwd_ctx, new_fwd, new_bwd = self._contexts(g, s, mamba_fwd_state, mamba_bwd_state, impl)
        gs = torch.stack([g, s], dim=-1)
        new_gru = self.gru(torch.cat([gs, fwd_ctx, bwd_ctx], dim=-1), gru_state.float())
        peer_in = torch.cat([new_gru, fwd_ctx, bwd_ctx, gs], dim=-1)
        half = self.d_model // 2
        total = torch.zeros_like(g)
        for h in range(self.num_peer_heads):
            q = self.peer_queries[h](peer_in)
            ia = (q[:, :half] @ self.product_keys_A[h].T).argmax(-1)
            ib = (q[:, half:] @ self.product_keys_B[h].T).argmax(-1)
            eidx = ia * self.pk_dim + ib
            if self.training:
                with torch.no_grad():
                    self.expert_counts.scatter_add_(0, eidx, torch.ones_like(eidx, dtype=torch.int32))
            total = total + self._expert_out(g, eidx)
        smart = g + self.rescale * total / self.num_peer_heads
        return smart.reshape(grad.shape).to(grad.dtype), new_gru, new_fwd, new_bwd

    def forward_for_bilevel(self, grad, sharpness, gru_state, mamba_fwd_state=None, mamba_bwd_state=None,
                            impl: str = "auto", topk: int = 4):
        g = grad.reshape(-1).float()
        s = sharpness.reshape(-1).float()
        fwd_ctx, bwd_ctx, new_fwd, new_bwd = self._contexts(g, s, mamba_fwd_state, mamba_bwd_state, impl)
        gs = torch.stack([g, s], dim=-1)
        new_gru = self.gru(torch.cat([gs, fwd_ctx, bwd_ctx], dim=-1), gru_state.float())
        peer_in = torch.cat([new_gru, fwd_ctx, bwd_ctx, gs], dim=-1)
        half = self.d_model // 2
        total = torch.zeros_like(g)
        for h in range(self.num_peer_heads):
            q = self.peer_queries[h](peer_in)
            ta, ia = (q[:, :half] @ self.product_keys_A[h].T).topk(topk, dim=-1)
            tb, ib = (q[:, half:] @ self.product_keys_B[h].T).topk(topk, dim=-1)
            wa, wb = torch.softmax(ta * 10.0, -1), torch.softmax(tb * 10.0, -1)
            eidx = (ia.unsqueeze(2) * self.pk_dim + ib.unsqueeze(1)).reshape(g.numel(), -1)
            w = (wa.unsqueeze(2) * wb.unsqueeze(1)).reshape(g.numel(), -1)
            total = total + (w * self._expert_out(g, eidx)).sum(-1)
        smart = g + self.rescale * total / self.num_peer_heads
        return smart.reshape(grad.shape).to(grad.dtype), new_gru, new_fwd, new_bwd

    def soft_head(self, g, s, gru_state, fwd_ctx, bwd_ctx, topk: int = 4):
        """Everything after the scan of ``forward_for_bilevel`` (GRU, soft top-k routing, experts) for elements whose
        contexts are given: returns smart_grad [n].  Element-wise over n, so it can be applied to any slice."""
        gs = torch.stack([g, s], dim=-1)
        # On CUDA the GRU and the product-key routing run as native kernels each way (ops/sg2_bilevel.py: gru, routing) when the
        # shapes are the ones they are built for; SG_BILEVEL_TAIL=torch keeps the PyTorch statements below, =native also takes
        # the C++ loops on CPU
        mode = os.environ.get("SG_BILEVEL_TAIL", "native" if g.is_cuda else "torch")
        native_tail = mode == "native" and g.dtype == torch.float32 and fwd_ctx.dtype == torch.float32
        if native_tail:
            from ..ops import sg2_bilevel as _sb
            native_tail = (_sb.gru_supported(2 + fwd_ctx.shape[1] + bwd_ctx.shape[1], self.gru_hidden) and
                           _sb.routing_supported(self.num_peer_heads, self.gru_hidden + fwd_ctx.shape[1] + bwd_ctx.shape[1] + 2,
                                                 self.pk_dim, self.d_model, topk))
        gru_in = torch.cat([gs, fwd_ctx, bwd_ctx], dim=-1)
        if native_tail:
            Wg = torch.stack([self.gru.W_z.weight, self.gru.W_r.weight, self.gru.W_h.weight])
            bg = torch.stack([self.gru.W_z.bias, self.gru.W_r.bias, self.gru.W_h.bias])
            new_gru = _sb.gru(gru_in, gru_state.float(), Wg, bg)
        else:
            new_gru = self.gru(gru_in, gru_state.float())
        peer_in = torch.cat([new_gru, fwd_ctx, bwd_ctx, gs], dim=-1)
        n = g.numel()
        # Every head evaluates the SAME experts on the SAME scalar g, so the heads only differ in their routing weights:
        # total = sum_e (sum_heads R_h[n,e]) * expert_e(g_n).  The routing weights are scattered into a dense [n, E]
        # matrix (whose backward is a gather) and all E experts are evaluated densely; gathering expert weights per
        # element instead would turn the backward into hundreds of millions of atomic adds onto E*hidden addresses.
        # On CUDA (g being data, not differentiated) the expert stage is one kernel each way instead; SG_BILEVEL_EXPERTS=dense
        # keeps the dense PyTorch formulation.
        use_kernel = False
        if g.is_cuda and not g.requires_grad and os.environ.get("SG_BILEVEL_EXPERTS", "kernel") != "dense":
            from ..ops import sg2_bilevel
            use_kernel = sg2_bilevel.routed_experts_supported(self.num_peer_heads, self.num_experts, self.expert_hidden, topk)
        # All heads at once: one matrix product for the queries, one against a block-diagonal key matrix for the 2 * heads
        # score vectors, ONE top-k and ONE softmax over [n, heads, 2, pk] (instead of 2 * heads of each).
        H, pk = self.num_peer_heads, self.pk_dim
        Wq = torch.cat([lin.weight for lin in self.peer_queries], 0)                                # [H * d_model, peer_in]
        if native_tail:
            # queries, scores, top-4 and softmax of all heads in one native kernel each way
            ia, ib, wa, wb = _sb.routing(peer_in, Wq, torch.stack(list(self.product_keys_A)), torch.stack(list(self.product_keys_B)))
        else:
            q = peer_in @ Wq.T                                                                      # [n, H * d_model]
            keys = torch.block_diag(*[blk for h in range(H) for blk in (self.product_keys_A[h].T, self.product_keys_B[h].T)])
            scores = (q @ keys).view(n, H, 2, pk)                                                   # [..., 0, :] sub-key A, [..., 1, :] sub-key B
            top, idx = scores.topk(topk, dim=-1)
            w = torch.softmax(top * 10.0, -1)
            ia, ib, wa, wb = idx[:, :, 0], idx[:, :, 1], w[:, :, 0], w[:, :, 1]                      # [n, H, topk] each
        if use_kernel:
            # one kernel evaluates the 16 selected experts of every head; its backward sums the expert gradients in a fixed order
            total = sg2_bilevel.routed_experts(g.reshape(-1), ia, ib, wa, wb, self.expert_W1.squeeze(-1), self.expert_b1,
                                               self.expert_W2.squeeze(1), self.expert_b2.squeeze(-1), pk)
            return g + self.rescale * total / self.num_peer_heads
        eidx = (ia.unsqueeze(3) * pk + ib.unsqueeze(2)).reshape(n, -1)                               # [n, H * topk * topk]
        wr = (wa.unsqueeze(3) * wb.unsqueeze(2)).reshape(n, -1)
        route = torch.zeros(n, self.num_experts, device=g.device, dtype=wr.dtype).scatter_add(1, eidx, wr)
        z = torch.relu(g.view(n, 1, 1) * self.expert_W1.squeeze(-1).unsqueeze(0) + self.expert_b1.unsqueeze(0))   # [n,E,H]
        out_all = (z * self.expert_W2.squeeze(1).unsqueeze(0)).sum(-1) + self.expert_b2.squeeze(-1).unsqueeze(0)   # [n,E]
        total = (route * out_all).sum(-1)
        return g + self.rescale * total / self.num_peer_heads

    # ------------------------------------------------------------------ expert recycling
    @torch.no_grad()
    def _recycle_dead_experts(self, generator: Optional[torch.Generator] = None):
        """Replace experts whose share of activations is below the threshold by noisy clones of a donor
        sampled in proportion to activation counts (reference mamba3_peer_metanet.py:437-491).  A
        generator makes the draw reproducible (and identical on every data-parallel rank)."""
        total = int(self.expert_counts.sum().item())
        if total == 0:
            return
        dead = (self.expert_counts.float() / total) < self.recycle_threshold
        if not bool(dead.any()):
            self.expert_counts.zero_()
            return
        dev = self.expert_counts.device

        def randn(shape):
            if generator is None:
                return torch.randn(shape, device=dev)
            return torch.randn(shape, generator=generator, device=generator.device).to(dev)

        cf = self.expert_counts.float()
        donor = int(torch.multinomial(cf if generator is None else cf.to(generator.device), 1,
                                      generator=generator).item())
        for i in dead.nonzero(as_tuple=True)[0].tolist():
            for prm in (self.expert_W1, self.expert_b1, self.expert_W2, self.expert_b2):
                prm.data[i] = prm.data[donor] + 0.01 * randn(prm.data[i].shape)
            a, b = divmod(i, self.pk_dim)
            if bool(dead[a * self.pk_dim:(a + 1) * self.pk_dim].all()):
                for h in range(self.num_peer_heads):
                    self.product_keys_A[h].data[a] = randn(self.product_keys_A[h].data[a].shape) * 0.02
            if bool(dead[b::self.pk_dim].all()):
                for h in range(self.num_peer_heads):
                    self.product_keys_B[h].data[b] = randn(self.product_keys_B[h].data[b].shape) * 0.02
        self.expert_counts.zero_()

    @property
    def has_cuda_bilevel(self) -> bool:
        from .. import _build
        return _build.native_available() and next(self.parameters()).is_cuda

    def forward_for_bilevel_cuda(self, *a, **k):
        return self.forward_for_bilevel(*a, **k)

    # ------------------------------------------------------------------ weight export
    def get_weights(self) -> Dict[str, object]:
        """Dictionary with the reference's key names (mamba3_peer_metanet.py:515-567)."""
        def c(t):
            return t.detach().float().contiguous()
        w: Dict[str, object] = {"input_proj_W": c(self.input_proj.weight), "input_proj_b": c(self.input_proj.bias)}
        for tag, blk in (("fwd", self.mamba_fwd), ("bwd", self.mamba_bwd)):
            w[f"mamba_{tag}_in_proj"] = c(blk.in_proj.weight)
            w[f"mamba_{tag}_dt_proj_W"] = c(blk.dt_proj.weight)
            w[f"mamba_{tag}_dt_proj_b"] = c(blk.dt_proj.bias)
            w[f"mamba_{tag}_B_proj"] = c(blk.B_proj.weight)
            w[f"mamba_{tag}_C_proj"] = c(blk.C_proj.weight)
            w[f"mamba_{tag}_A_log"] = c(blk.A_log)
            w[f"mamba_{tag}_D"] = c(blk.D)
            w[f"mamba_{tag}_rope_freq"] = c(blk.rope_freq)
            w[f"mamba_{tag}_out_proj"] = c(blk.out_proj.weight)
        for n, lin in (("z", self.gru.W_z), ("r", self.gru.W_r), ("h", self.gru.W_h)):
            w[f"gru_W_{n}"] = c(lin.weight)
            w[f"gru_b_{n}"] = c(lin.bias)
        w["peer_queries"] = [c(q.weight) for q in self.peer_queries]
        w["product_keys_A"] = [c(k) for k in self.product_keys_A]
        w["product_keys_B"] = [c(k) for k in self.product_keys_B]
        w["expert_W1"], w["expert_b1"] = c(self.expert_W1), c(self.expert_b1)
        w["expert_W2"], w["expert_b2"] = c(self.expert_W2), c(self.expert_b2)
        w.update(rescale=self.rescale, d_model=self.d_model, d_state=self.d_state, d_inner=self.mamba_fwd.d_inner,
                 pk_dim=self.pk_dim, expert_hidden=self.expert_hidden, gru_hidden=self.gru_hidden,
                 num_peer_heads=self.num_peer_heads, num_experts=self.num_experts)
        return w

    # Layout of the packed fp32 weight blob consumed by the CUDA kernels (offsets in floats).
    # Only the default geometry (d_model 8, d_inner 16, d_state 16, gru 4, heads 4, pk 12, hidden <= 16) is packed.
    def pack_weights(self) -> torch.Tensor:
        """One contiguous fp32 vector: see ``PACK_LAYOUT`` in ops/sg2.py for the offsets."""
        from ..ops.sg2 import pack_metanet
        return pack_metanet(self)
