"""CUDA bilevel path of SuperGrok v2: batched forward scan + parallel scan adjoint (``csrc/sg2_bilevel.cuh``).

All parameter tensors are processed in ONE batched call: sort -> gather -> forward scan (the step kernels, with scratch
copies of the persistent states) -> contexts ``ctx [total, 16]``.  The part after the scan (GRU, soft top-4 product-key
routing, experts) is element-wise and runs through autograd in slices, producing d(meta_loss)/d ctx.  The scan adjoint
kernels turn that into gradients of A_log, rope_freq, D, out_proj and of the folded affine tables; autograd through
``scan_params`` (a few 16x16 matrix products) carries the table gradients to input_proj / in_proj / dt_proj / B_proj / C_proj.
The result equals autograd of ``Mamba3PEERMetaNet.forward_for_bilevel`` (tested), including the cross-column terms that
the reference kernel drops.

``routed_experts`` is the expert stage of that tail as one forward and one backward kernel (``csrc/sg2_experts.cu``): the
16 experts per head selected by the top-4 x top-4 product keys are evaluated on the element's gradient and weighted; the
backward pass returns the routing-weight gradients per element and the expert-parameter gradients summed over all
elements in a fixed order.  Without it the stage materialises [n, experts, hidden] tensors in both passes.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

from .. import _build
from . import sg2 as sg2_ops


class _RoutedExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, ia, ib, wa, wb, W1, b1, W2, b2, pk):
        C = _build.require()
        args = [t.contiguous() for t in (g.float(), ia.int(), ib.int(), wa.float(), wb.float(), W1.float(), b1.float(), W2.float(), b2.float())]
        ctx.save_for_backward(*args)
        ctx.pk = int(pk)
        return C.sg2_routed_experts_fwd(*args, ctx.pk)

    @staticmethod
    def backward(ctx, dtotal):
        C = _build.require()
        g, ia, ib, wa, wb, W1, b1, W2, b2 = ctx.saved_tensors
        dwa, dwb, dp = C.sg2_routed_experts_bwd(g, ia, ib, wa, wb, W1, b1, W2, b2, ctx.pk, dtotal.contiguous().float())
        E, H = W1.shape
        return (None, None, None, dwa, dwb, dp[:E * H].view(E, H), dp[E * H:2 * E * H].view(E, H), dp[2 * E * H:3 * E * H].view(E, H),
                dp[3 * E * H:].view(E), None)


def routed_experts_supported(heads: int, experts: int, hidden: int, topk: int) -> bool:
    return bool(_build.require().sg2_routed_experts_supported(heads, experts, hidden, topk))


def routed_experts(g, ia, ib, wa, wb, W1, b1, W2, b2, pk: int) -> torch.Tensor:
    """total[n] = sum over heads h and key pairs (a, b) of wa[n,h,a] * wb[n,h,b] * expert_{ia[n,h,a]*pk + ib[n,h,b]}(g[n]).

    g [n]; ia, ib int [n, heads, 4]; wa, wb [n, heads, 4]; W1, b1, W2 [experts, 16]; b2 [experts].  Differentiable with
    respect to wa, wb and the four expert tables (not g, which is data on this path)."""
    return _RoutedExperts.apply(g, ia, ib, wa, wb, W1, b1, W2, b2, pk)


class _Routing(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pin, Wq, KA, KB):
        C = _build.require()
        a = [t.detach().contiguous().float() for t in (pin, Wq, KA, KB)]
        ia, ib, wa, wb = C.sg2_routing_fwd(*a)
        ctx.save_for_backward(*a, ia, ib, wa, wb)
        ctx.mark_non_differentiable(ia, ib)
        return ia, ib, wa, wb

    @staticmethod
    def backward(ctx, _dia, _dib, dwa, dwb):
        C = _build.require()
        pin, Wq, KA, KB, ia, ib, wa, wb = ctx.saved_tensors
        dwa = torch.zeros_like(wa) if dwa is None else dwa.contiguous().float()
        dwb = torch.zeros_like(wb) if dwb is None else dwb.contiguous().float()
        dpin, dp = C.sg2_routing_bwd(pin, Wq, KA, KB, ia, ib, wa, wb, dwa, dwb)
        nq, nk = Wq.numel(), KA.numel()
        return dpin, dp[:nq].view_as(Wq), dp[nq:nq + nk].view_as(KA), dp[nq + nk:].view_as(KB)


def routing_supported(heads: int, width: int, pk: int, d_model: int, topk: int) -> bool:
    return bool(_build.require().sg2_routing_supported(heads, width, pk, d_model, topk))


def routing(pin, Wq, KA, KB):
    """Product-key routing of all heads: pin [n, P], Wq [heads * 8, P], KA / KB [heads, pk, 4] ->
    (ia, ib int32 [n, heads, 4], wa, wb [n, heads, 4]); differentiable with respect to pin, Wq, KA and KB through wa and wb.
    CUDA tensors run ``csrc/sg2_routing.cu``, CPU tensors the same arithmetic in a C++ loop (``csrc/sg2_routing_math.h``)."""
    return _Routing.apply(pin, Wq, KA, KB)


class _Gru(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, h, W, b):
        C = _build.require()
        a = [t.detach().contiguous().float() for t in (x, h, W, b)]
        ctx.save_for_backward(*a)
        return C.sg2_gru_fwd(*a)

    @staticmethod
    def backward(ctx, dhn):
        C = _build.require()
        x, h, W, b = ctx.saved_tensors
        dx, dp = C.sg2_gru_bwd(x, h, W, b, dhn.contiguous().float())
        return dx, None, dp[:W.numel()].view_as(W), dp[W.numel():].view_as(b)


def gru_supported(width: int, hidden: int) -> bool:
    return bool(_build.require().sg2_gru_supported(width, hidden))


def gru(x, h, W, b):
    """New GRU state [n, 4] from inputs x [n, IN] and the previous state h [n, 4] (data: no gradient); W [3, 4, IN + 4] and
    b [3, 4] hold the z, r and candidate gates.  Differentiable with respect to x, W and b.  CUDA tensors run ``csrc/sg2_gru.cu``,
    CPU tensors the same arithmetic in a C++ loop (``csrc/sg2_gru_math.h``)."""
    return _Gru.apply(x, h, W, b)


def scan_params(meta_net) -> List[torch.Tensor]:
    """Differentiable tensors the adjoint kernel reports gradients for, per direction:
    A_log [16,16], rope [16,8], D [16], U_x, U_z, U_dt, U_B, U_C [16,3] each, out_proj [8,16]."""
    Wi, bi = meta_net.input_proj.weight.double(), meta_net.input_proj.bias.double()
    inp = torch.cat([Wi, bi.unsqueeze(1)], 1)                                   # [8,3]
    out = []
    for blk in (meta_net.mamba_fwd, meta_net.mamba_bwd):
        xz = blk.in_proj.weight.double() @ inp
        x_t, z_t = xz[:16], xz[16:]
        dt_t = blk.dt_proj.weight.double() @ x_t
        dt_t = torch.cat([dt_t[:, :2], (dt_t[:, 2] + blk.dt_proj.bias.double()).unsqueeze(1)], 1)
        b_t = blk.B_proj.weight.double() @ x_t
        c_t = blk.C_proj.weight.double() @ x_t
        out += [blk.A_log, blk.rope_freq, blk.D, x_t, z_t, dt_t, b_t, c_t, blk.out_proj.weight]
    return out


_SLICES = [(0, 256, (16, 16)), (256, 384, (16, 8)), (384, 400, (16,)), (400, 448, (16, 3)), (448, 496, (16, 3)), (496, 544, (16, 3)),
           (544, 592, (16, 3)), (592, 640, (16, 3)), (640, 768, (8, 16))]


class _Workspace:
    """Plan + scratch for a batched bilevel call over a fixed list of tensor sizes."""

    def __init__(self, numels, device, snap_every: int = 1):
        C = _build.require()
        info = C.sg2_bilevel_info()
        self.snap_every = max(1, int(snap_every))
        self.h_fwd = [torch.zeros(16, 16, device=device) for _ in numels]
        self.h_bwd = [torch.zeros(16, 16, device=device) for _ in numels]
        self.plan = sg2_ops.Plan(numels, self.h_fwd, self.h_bwd, device)
        p = self.plan
        items = p.items.cpu().numpy().view(sg2_ops.Plan.ITEM)
        tiles = np.where(items["tensor"] >= 0, -(-(items["ue"] - items["ub"]) // info["tile"]), 0).astype(np.int64)
        tiles = -(-tiles // self.snap_every)                                  # one state snapshot per snap_every tiles
        base = np.concatenate([[0], np.cumsum(tiles)[:-1]]).astype(np.int64)
        self.snap_base = torch.from_numpy(base).to(device)
        n_snap = int(tiles.sum())
        f32 = dict(dtype=torch.float32, device=device)
        p.ws["dcarry"] = torch.empty_like(p.ws["carry"])
        self.snaps = torch.empty(max(n_snap, 1) * 256, **f32)
        self.partial = torch.empty(max(p.n_items, 1) * info["ng"], **f32)
        self.grads = torch.empty(2 * info["ng"], **f32)
        self.ng = info["ng"]


class _ScanCtx(torch.autograd.Function):
    @staticmethod
    def forward(ctx, wsp, grads_list, sharps, fwd_states, bwd_states, *params):
        C = _build.require()
        p = wsp.plan
        for dst, src in zip(wsp.h_fwd, fwd_states):
            dst.copy_(src)
        for dst, src in zip(wsp.h_bwd, bwd_states):
            dst.copy_(src)
        buf = C.sg2_prepare(grads_list, sharps, p.offsets[:-1], p.total, p.seg_off, 1e30, p.ws)      # no clipping: raw gradients
        C.sg2_scan(p.items, p.n_items, p.dir1_start, p.tds, p.n_td, p.any_multi, buf, p.ws)
        ctx.wsp, ctx.buf = wsp, buf
        return p.ws["ctx"][: 16 * p.total].view(p.total, 16).clone()

    @staticmethod
    def backward(ctx, dctx):
        C = _build.require()
        wsp, p = ctx.wsp, ctx.wsp.plan
        C.sg2_scan_backward(p.items, p.n_items, p.dir1_start, p.tds, p.n_td, wsp.snap_base, ctx.buf, dctx.contiguous().float(), p.ws,
                            wsp.snaps, wsp.partial, wsp.grads, snap_every=wsp.snap_every)
        g = wsp.grads.view(2, wsp.ng)
        outs = []
        for d in range(2):
            for a, b, shape in _SLICES:
                t = g[d, a:b].reshape(shape).clone()
                outs.append(t.double() if shape == (16, 3) else t)
        return (None, None, None, None, None, *outs)


def snapshot_tiles(checkpoint_interval: int) -> int:
    """Tiles of 16 timesteps per saved scan state for a requested checkpoint interval C (reference supergrok2.py:93, 667-674:
    every C-th state is kept and segments of C steps are recomputed).  The adjoint works on 16-step tiles, so intervals up to 16
    keep a state per tile (64 bytes per element, already 1/16 of the reference's C = 1) and larger ones keep one per
    ceil(C / 16) tiles; the gradients are the same for every interval."""
    return max(1, -(-int(checkpoint_interval) // 16))


def bilevel_backward_cuda(opt, named, train_grads: Dict[str, torch.Tensor], val_grads: Dict[str, torch.Tensor],
                          slice_elems: int = 0, checkpoint_interval: int = 1) -> int:
    """Accumulate d(meta_loss)/d(meta-net parameters) into their ``.grad`` with the batched CUDA pipeline.
    ``slice_elems``: elements per slice of the element-wise tail (0: 2M with the expert kernel, 256K with the dense PyTorch
    expert stage, whose [slice, experts, hidden] intermediates bound the slice)."""
    import os
    C = _build.require()
    mn = opt.meta_net
    if slice_elems <= 0:
        kernel = os.environ.get("SG_BILEVEL_EXPERTS", "kernel") != "dense" and \
            routed_experts_supported(mn.num_peer_heads, mn.num_experts, mn.expert_hidden, 4)
        slice_elems = (1 << 21) if kernel else (1 << 18)
    sel = []
    for name, p in named:
        if name not in train_grads or name not in val_grads or p.numel() == 0:
            continue
        i = opt._param_to_idx.get(id(p))
        if i is None:
            continue
        vg = val_grads[name].detach().reshape(-1).float()
        sel.append((i, train_grads[name].detach().reshape(-1).float().contiguous(), vg))
    if not sel:
        return 0
    dev = sel[0][1].device
    # tensors with non-finite validation gradients are skipped (decided on the device, applied as a zero weight)
    vus = []
    for _, _, vg in sel:
        ok = torch.isfinite(vg).all()
        n = torch.where(torch.isfinite(vg), vg, torch.zeros_like(vg)).norm()
        vus.append(torch.where(ok & (n > 1e-12), 1.0 / n.clamp_min(1e-30), torch.where(ok, torch.ones_like(n), torch.zeros_like(n)))
                   * torch.where(torch.isfinite(vg), vg, torch.zeros_like(vg)))
    numels = tuple(g.numel() for _, g, _ in sel)
    g_snap = snapshot_tiles(checkpoint_interval)
    key = (numels, str(dev), g_snap)
    cache = getattr(opt, "_bilevel_ws", None)
    if cache is None or cache[0] != key:
        opt._bilevel_ws = cache = (key, _Workspace(list(numels), dev, g_snap))
    wsp = cache[1]
    w = sg2_ops.pack_metanet(mn).to(dev)
    C.sg2_upload_weights(w)
    sg2_ops._resident["owner"] = None                      # the optimizer step must re-upload its own copy afterwards
    idxs = [i for i, _, _ in sel]
    params = scan_params(mn)
    with torch.enable_grad():
        ctx_all = _ScanCtx.apply(wsp, [g for _, g, _ in sel], [opt._flat_sharpness[i] for i in idxs],
                                 [opt._flat_mamba_fwd_states[i] for i in idxs], [opt._flat_mamba_bwd_states[i] for i in idxs], *params)
    p = wsp.plan
    g_all = p.ws["g"][: p.total]
    s_all = p.ws["s"][: p.total]
    gru_all = torch.cat([opt._flat_gru_states[i] for i in idxs], 0)
    vu_all = torch.cat(vus)
    dctx = torch.zeros(p.total, 16, device=dev)
    for a in range(0, p.total, slice_elems):                # element-wise tail of the meta-net, slice by slice
        b = min(p.total, a + slice_elems)
        c = ctx_all[a:b].detach().requires_grad_(True)
        with torch.enable_grad():
            smart = mn.soft_head(g_all[a:b], s_all[a:b], gru_all[a:b], c[:, :8], c[:, 8:])
            loss = -(smart * vu_all[a:b]).sum()
        loss.backward()
        dctx[a:b] = c.grad
    ctx_all.backward(dctx)
    return len(sel)
