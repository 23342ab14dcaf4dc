"""SuperGrok v2 step and bilevel orchestration.

CUDA: all tensors of the optimizer go through ONE batched pipeline of sm_100a kernels
(``csrc/sg2_kernels.cu`` + ``csrc/sg2_sort.cu``): per-tensor clip -> packed keys -> segmented radix
sort -> gather -> 3-phase multi-CTA bidirectional scan -> fused element step.  A *plan* (offsets,
scan work items, workspace) is built once per set of tensors and reused; a step allocates nothing.
CPU: the PyTorch oracle (meta-net ``forward`` per tensor + ``oracle.sg2_adam_``).

The packed weight vector layout is defined once, in ``csrc/sg_native.h`` (``SG2Pack``), and read
back from the extension so Python and CUDA cannot drift apart.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

from .. import _build
from . import oracle

# Scan items that are resident at once: 148 SMs x the CTAs per SM the kernel is compiled for (three; 26.6 KB shared memory each) x 8 items per CTA.  All chunks
# take about the same time, so the items should fill WHOLE waves of that many: one item too many starts a second wave that costs as
# much as the first.  One wave for small steps (longer chunks: the per-chunk aggregate pass of phase 1 costs a fixed ~300 timesteps
# per chunk), two for large ones.
_MIN_CHUNK = 512


def _wave_items() -> int:
    C = _build.load()
    ctas = C.sg2_scan_ctas_per_sm() if C is not None and hasattr(C, "sg2_scan_ctas_per_sm") else 4
    return 148 * ctas * 8


def _pick_chunk_len(numels: Sequence[int]) -> int:
    total2 = 2 * sum(numels)
    wave = _wave_items()
    waves = 1 if total2 <= wave * 2048 else 2
    cap = wave * waves - 8                            # the forward-direction items are padded to a multiple of 8
    L = max(_MIN_CHUNK, -(-total2 // cap))
    L = -(-L // 16) * 16
    while 2 * sum(max(1, -(-n // L)) for n in numels) > cap and L < (1 << 30):      # partial last chunks of the tensors must fit as well
        L += 16
    return L

_FALLBACK_LAYOUT = None


def layout() -> Dict[str, int]:
    """Offsets of ``SG2Pack`` (from the extension; a pure-Python copy is used when it is not built)."""
    global _FALLBACK_LAYOUT
    C = _build.load()
    if C is not None:
        return dict(C.sg2_layout())
    if _FALLBACK_LAYOUT is None:
        L, o = {}, 0
        def put(name, size):
            nonlocal o
            L[name] = o
            o += size
        put("IN_W", 16); put("IN_B", 8); put("DIR0", 0)
        d = {"D_INPROJ": 256, "D_DTW": 256, "D_DTB": 16, "D_BW": 256, "D_CW": 256, "D_ALOG": 256, "D_D": 16,
             "D_ROPE": 128, "D_OUT": 128}
        oo = 0
        for k, v in d.items():
            L[k] = oo
            oo += v
        L["DIR_SIZE"] = oo
        L["DIR1"] = L["DIR0"] + oo
        o = L["DIR1"] + oo
        for name, size in (("GRU_WZ", 88), ("GRU_WR", 88), ("GRU_WH", 88), ("GRU_BZ", 4), ("GRU_BR", 4), ("GRU_BH", 4),
                           ("PQ", 704), ("KA", 192), ("KB", 192), ("EW1", 2304), ("EB1", 2304), ("EW2", 2304),
                           ("EB2", 144)):
            put(name, size)
        L["NET"] = o
        for k, name in enumerate(("A_X", "A_Z", "A_DT", "A_B", "A_C")):
            L[name] = 48 * k
        L["AFF_SIZE"] = 240
        L["AFF0"], L["AFF1"] = o, o + 240
        L["TOTAL"] = o + 480
        _FALLBACK_LAYOUT = L
    return _FALLBACK_LAYOUT


def supports_native(meta_net) -> bool:
    """The fused kernels are compiled for the default geometry (expert_hidden may be smaller than 16)."""
    return (meta_net.d_model == 8 and meta_net.d_state == 16 and meta_net.mamba_fwd.d_inner == 16 and
            meta_net.gru_hidden == 4 and meta_net.num_peer_heads == 4 and meta_net.num_experts == 144 and
            meta_net.expert_hidden <= 16)


@torch.no_grad()
def pack_metanet(meta_net) -> torch.Tensor:
    """Meta-net weights as one fp32 vector in ``SG2Pack`` order (experts zero-padded to 16 hidden units)."""
    if not supports_native(meta_net):
        raise ValueError("the fused v2 kernels support d_model 8, d_state 16, expand 2, gru 4, 4 heads, 144 experts, "
                         "expert_hidden <= 16")
    L = layout()
    dev = meta_net.input_proj.weight.device
    out = torch.zeros(L["TOTAL"], dtype=torch.float32, device=dev)

    def put(off, t):
        t = t.detach().float().reshape(-1)
        out[off:off + t.numel()] = t

    put(L["IN_W"], meta_net.input_proj.weight)
    put(L["IN_B"], meta_net.input_proj.bias)
    for base, blk in ((L["DIR0"], meta_net.mamba_fwd), (L["DIR1"], meta_net.mamba_bwd)):
        put(base + L["D_INPROJ"], blk.in_proj.weight)
        put(base + L["D_DTW"], blk.dt_proj.weight)
        put(base + L["D_DTB"], blk.dt_proj.bias)
        put(base + L["D_BW"], blk.B_proj.weight)
        put(base + L["D_CW"], blk.C_proj.weight)
        put(base + L["D_ALOG"], blk.A_log)
        put(base + L["D_D"], blk.D)
        put(base + L["D_ROPE"], blk.rope_freq)
        put(base + L["D_OUT"], blk.out_proj.weight)
    put(L["GRU_WZ"], meta_net.gru.W_z.weight); put(L["GRU_WR"], meta_net.gru.W_r.weight); put(L["GRU_WH"], meta_net.gru.W_h.weight)
    put(L["GRU_BZ"], meta_net.gru.W_z.bias); put(L["GRU_BR"], meta_net.gru.W_r.bias); put(L["GRU_BH"], meta_net.gru.W_h.bias)
    put(L["PQ"], torch.stack([q.weight for q in meta_net.peer_queries]))
    put(L["KA"], torch.stack(list(meta_net.product_keys_A)))
    put(L["KB"], torch.stack(list(meta_net.product_keys_B)))
    eh = meta_net.expert_hidden
    pad = lambda t: torch.nn.functional.pad(t.detach().float().reshape(144, eh), (0, 16 - eh))  # noqa: E731
    put(L["EW1"], pad(meta_net.expert_W1)); put(L["EB1"], pad(meta_net.expert_b1)); put(L["EW2"], pad(meta_net.expert_W2))
    put(L["EB2"], meta_net.expert_b2)
    # Every per-timestep input of the scan is an affine function of (g, s): fold input_proj with in_proj and the
    # dt / B / C projections into [16][3] tables (coefficient of g, coefficient of s, constant), in fp64.
    Wi = meta_net.input_proj.weight.detach().double()          # [8,2]
    bi = meta_net.input_proj.bias.detach().double()            # [8]
    inp = torch.cat([Wi, bi.unsqueeze(1)], 1)                  # [8,3]: inp_d = inp[d,0] g + inp[d,1] s + inp[d,2]
    for base, blk in ((L["AFF0"], meta_net.mamba_fwd), (L["AFF1"], meta_net.mamba_bwd)):
        Win = blk.in_proj.weight.detach().double()             # [32,8]
        xz = Win @ inp                                         # [32,3]
        x_t, z_t = xz[:16], xz[16:]
        dt_t = blk.dt_proj.weight.detach().double() @ x_t
        dt_t[:, 2] += blk.dt_proj.bias.detach().double()
        b_t = blk.B_proj.weight.detach().double() @ x_t
        c_t = blk.C_proj.weight.detach().double() @ x_t
        for name, tab in (("A_X", x_t), ("A_Z", z_t), ("A_DT", dt_t), ("A_B", b_t), ("A_C", c_t)):
            put(base + L[name], tab)
    return out


# --------------------------------------------------------------------------- plan
class Plan:
    """Static description of a v2 step over a fixed list of tensors (sizes, device tables, workspace)."""

    ITEM = np.dtype([("off", "<i8"), ("n", "<i4"), ("ub", "<i4"), ("ue", "<i4"), ("tensor", "<i4"), ("td", "<i4"),
                     ("last", "<i4")])
    TD = np.dtype([("h", "<u8"), ("item0", "<i4"), ("nc", "<i4"), ("pad", "<i4", (4,))])

    def __init__(self, numels: Sequence[int], h_fwd: List[torch.Tensor], h_bwd: List[torch.Tensor], device,
                 chunk_len: int = 0):
        C = _build.require()
        assert self.ITEM.itemsize == C.sg2_layout()["item_bytes"] and self.TD.itemsize == C.sg2_layout()["td_bytes"]
        self.numels = [int(n) for n in numels]
        self.n = len(self.numels)
        self.offsets = [0]
        for n in self.numels:
            self.offsets.append(self.offsets[-1] + n)
        self.total = self.offsets[-1]
        if max(self.numels) >= 2 ** 31 or self.total >= 2 ** 32:
            raise ValueError("a v2 step handles < 2^31 elements per tensor and < 2^32 in total per call")
        if chunk_len <= 0:
            chunk_len = _pick_chunk_len(self.numels)
        chunk_len = -(-chunk_len // 16) * 16
        self.chunk_len = chunk_len
        items, tds = [], []
        for d, hs in ((0, h_fwd), (1, h_bwd)):
            if d == 1:
                while len(items) % 8:
                    items.append((0, 0, 0, 0, -1, 0, 0))
                self.dir1_start = len(items)
            for t, n in enumerate(self.numels):
                nc = max(1, -(-n // chunk_len))
                tds.append((hs[t].data_ptr(), len(items), nc, (0, 0, 0, 0)))
                for c in range(nc):
                    items.append((self.offsets[t], n, c * chunk_len, min(n, (c + 1) * chunk_len), t, len(tds) - 1,
                                  1 if c == nc - 1 else 0))
        self.n_items = len(items)
        self.n_td = len(tds)
        self.any_multi = any(td[2] > 1 for td in tds)
        self._keep = (h_fwd, h_bwd)
        self.items = torch.from_numpy(np.array(items, dtype=self.ITEM).view(np.uint8).copy()).to(device)
        self.tds = torch.from_numpy(np.array(tds, dtype=self.TD).view(np.uint8).copy()).to(device)
        self.seg_off = torch.tensor(self.offsets, dtype=torch.int64, device=device)
        tot = max(self.total, 1)
        nb_sort = C.sg2_sort_blocks(tot)
        nb_mt = C.mt_num_blocks(self.numels)
        f32 = dict(dtype=torch.float32, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        self.ws = {
            "partials": torch.empty(3 * max(nb_mt, 1), **f32), "tnorm": torch.empty(3 * self.n, **f32),
            "tclip": torch.empty(self.n, **f32), "g": torch.empty(tot, **f32), "s": torch.empty(tot, **f32),
            "keys0": torch.empty(tot, **i32), "keys1": torch.empty(tot, **i32), "vals0": torch.empty(tot, **i32),
            "vals1": torch.empty(tot, **i32), "hist": torch.empty(256 * nb_sort, **i32), "tot": torch.empty(256, **i32),
            "gs": torch.empty(2 * tot, **f32), "ctx": torch.empty(16 * tot, **f32),
            "agg": torch.empty(max(self.n_items, 1) * 16 * 48, **f32),
            "carry": torch.empty(max(self.n_items, 1) * 16 * 16, **f32),
        }
        from . import elementwise as _ew
        if _ew.DEBUG_POISON:                                          # GROK_DEBUG=1: float scratch starts as NaN (see ops/elementwise.py)
            for t in self.ws.values():
                if t.is_floating_point():
                    t.fill_(float("nan"))

    def workspace_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.ws.values())


def _plan_for(opt, idx: List[int]) -> Plan:
    key = (tuple(idx), tuple(opt._flat_mamba_fwd_states[i].data_ptr() for i in idx))
    plan = getattr(opt, "_native_plan", None)
    if plan is None or plan[0] != key:
        dev = opt._flat_params[idx[0]].device
        p = Plan([opt._flat_params[i].numel() for i in idx], [opt._flat_mamba_fwd_states[i] for i in idx],
                 [opt._flat_mamba_bwd_states[i] for i in idx], dev, getattr(opt, "scan_chunk_len", 0))
        opt._native_plan = plan = (key, p)
    return plan[1]


def _packed_weights(opt, dev) -> Tuple[torch.Tensor, bool]:
    """Packed meta-net weights of ``opt`` on ``dev``.  The buffer is allocated once and refreshed in place, so kernels captured
    in a CUDA graph keep reading the right address."""
    cur = getattr(opt, "_packed_w", None)
    if opt._weights_dirty or cur is None or cur.device != dev:
        w = pack_metanet(opt.meta_net).to(dev)
        if cur is not None and cur.device == dev and cur.numel() == w.numel():
            cur.copy_(w)
        else:
            opt._packed_w = w
        opt._weights_dirty = False
        return opt._packed_w, True
    return cur, False


# the constant-memory copy of the weights is per process: remember whose weights it holds
_resident = {"owner": None}

DYN_WORDS = 16          # words of the table of step scalars before the per-tensor entries (csrc/sg_native.h: DYN_*)


def refresh_weights(opt, dev) -> torch.Tensor:
    """Make the device copies of the meta-net weights (global-memory vector and ``__constant__`` copy) current.  Runs outside
    any CUDA graph: the kernels of a captured step read both copies."""
    w, fresh = _packed_weights(opt, dev)
    if fresh or _resident["owner"] is not opt:
        _build.require().sg2_upload_weights(w)
        _resident["owner"] = opt
    return w


def dyn_table(opt, n_tensors: int, dev) -> torch.Tensor:
    """Device table of the scalars that change from step to step (learning rate, effective weight decay, lambda_eff, per-tensor
    alpha / beta1 / bias corrections, barrier epoch).  Its address is fixed, so the kernels that read it can be replayed from a
    CUDA graph; ``write_scalars`` refreshes it before every step."""
    t = getattr(opt, "_dyn", None)
    need = DYN_WORDS + 4 * max(n_tensors, 1)
    if t is None or t.device != dev or t.numel() < need:
        opt._dyn = t = torch.zeros(need, dtype=torch.float32, device=dev)
    return t


def write_scalars(opt, per, *, lr, wd_eff, dev, epoch_base: int = 0):
    """One tiny kernel whose arguments are the values: no host staging buffer that a later step could overwrite too early."""
    t = dyn_table(opt, len(per), dev)
    floats = [lr, wd_eff, per[0][1] if per else 0.0, 0.0, 0.0, 0.0, 0.0, 0.0]
    for (a, _l, b1, bc1, bc2) in per:
        floats += [a, b1, bc1, bc2]
    _build.require().write_table(t, [int(epoch_base) & 0xffffffff, 0, 0, 0, 0, 0, 0, 0], floats)
    return t


@torch.no_grad()
def launch(opt, idx: List[int], *, beta2, eps, clip, pull=None, status=None, stage_hook=None):
    """Enqueue the kernels of one v2 update of tensors ``idx``; every scalar that changes between steps is read from the device
    table, so the same sequence can be captured once and replayed.  ``pull = (bases, rank, scale)``: the gradients are this
    rank's slices of its flat gradient buffer (``opt._pull_grads``) and the first kernel sums the copies of all ranks
    (reduce-scatter fused in).  ``stage_hook(name)`` is called between the phases (per-phase CUDA-event timing)."""
    C = _build.require()
    params = [opt._flat_params[i] for i in idx]
    dev = params[0].device
    plan = _plan_for(opt, idx)
    sharps = [opt._flat_sharpness[i] for i in idx]
    offs = plan.offsets[:-1]
    hook = stage_hook or (lambda _n: None)
    if pull is not None:
        grads = [opt._pull_grads[i] for i in idx]
        kw = dict(pull_bases=list(pull[0]), pull_rank=int(pull[1]), pull_scale=float(pull[2]))
    else:
        gsrc = getattr(opt, "_grad_override", None)     # reduced fp32 gradients supplied by the ZeRO engine (NCCL / CPU paths)
        grads = [gsrc[i] for i in idx] if gsrc else [p.grad for p in params]
        kw = {}
    if stage_hook is None:
        buf = C.sg2_prepare(grads, sharps, offs, plan.total, plan.seg_off, float(clip), plan.ws, **kw)
    else:
        C.sg2_prepare(grads, sharps, offs, plan.total, plan.seg_off, float(clip), plan.ws, stage=1, **kw)
        hook("reduce+prep")
        buf = C.sg2_prepare(grads, sharps, offs, plan.total, plan.seg_off, float(clip), plan.ws, stage=2, **kw)
        hook("sort")
    C.sg2_scan(plan.items, plan.n_items, plan.dir1_start, plan.tds, plan.n_td, plan.any_multi, buf, plan.ws, status=status)
    hook("scan")
    counts = opt.meta_net.expert_counts if opt.meta_net.training else None
    masters = getattr(opt, "_flat_masters", None)
    push = getattr(opt, "_peer_push", None)         # (local_base, [peer bases]) set by the ZeRO engine
    C.sg2_elem(params, [opt._flat_exp_avgs[i] for i in idx], [opt._flat_exp_avg_sqs[i] for i in idx],
               [opt._flat_mus[i] for i in idx], [opt._flat_gru_states[i] for i in idx],
               [masters[i] for i in idx] if masters else [], dyn_table(opt, len(idx), dev), opt._packed_w, offs, beta2, eps,
               float(opt.meta_net.rescale), counts, plan.ws, push[0] if push else 0, push[1] if push else [], status=status)
    hook("elem+push")


@torch.no_grad()
def step(opt, idx: List[int], per: List[Tuple[float, float, float, float, float]], *, beta2, lr, wd_eff, eps, clip):
    """One v2 update of tensors ``idx`` of ``opt``; ``per[k] = (alpha, lamb_eff, beta1, bc1, bc2)``."""
    params = [opt._flat_params[i] for i in idx]
    if not params[0].is_cuda:
        return _step_cpu(opt, idx, per, beta2=beta2, lr=lr, wd_eff=wd_eff, eps=eps, clip=clip)
    dev = params[0].device
    refresh_weights(opt, dev)
    write_scalars(opt, per, lr=lr, wd_eff=wd_eff, dev=dev)
    launch(opt, idx, beta2=beta2, eps=eps, clip=clip)


def clip_scrub(g: torch.Tensor, clip: float) -> torch.Tensor:
    """Per-tensor preprocessing of the v2 step: non-finite entries -> 0, then clip to ``clip`` by the 2-norm."""
    gf = g.detach().reshape(-1).float()
    gf = torch.where(torch.isfinite(gf), gf, torch.zeros_like(gf))
    n = gf.norm()
    return gf * torch.where(n > clip, clip / (n + 1e-12), torch.ones_like(n))


@torch.no_grad()
def _step_cpu(opt, idx, per, *, beta2, lr, wd_eff, eps, clip):
    mn = opt.meta_net
    for k, i in enumerate(idx):
        p = opt._flat_params[i]
        alpha, lamb_eff, b1, bc1, bc2 = per[k]
        gsrc = getattr(opt, "_grad_override", None)
        g = clip_scrub(gsrc[i] if gsrc else p.grad, clip)
        s = opt._flat_sharpness[i].reshape(-1).float()
        s = torch.where(torch.isfinite(s), s, torch.zeros_like(s))
        smart, gru, hf, hb = mn(g, s, opt._flat_gru_states[i], opt._flat_mamba_fwd_states[i],
                                opt._flat_mamba_bwd_states[i])
        opt._flat_gru_states[i].copy_(gru)
        opt._flat_mamba_fwd_states[i].copy_(hf)
        opt._flat_mamba_bwd_states[i].copy_(hb)
        masters = getattr(opt, "_flat_masters", None)
        tgt = masters[i] if masters else p                 # fp32 master copy under ZeRO, else the parameter itself
        oracle.sg2_adam_(tgt, smart.reshape(-1).float(), g, opt._flat_mus[i], opt._flat_exp_avgs[i],
                         opt._flat_exp_avg_sqs[i], alpha, lamb_eff, b1, beta2, lr, wd_eff, eps, bc1, bc2)
        if masters:
            p.detach().copy_(tgt.reshape(p.shape).to(p.dtype))


# --------------------------------------------------------------------------- bilevel
def bilevel_backward(opt, named, train_grads: Dict[str, torch.Tensor], val_grads: Dict[str, torch.Tensor],
                     checkpoint_interval: int = 1) -> int:
    """Accumulate d(meta_loss)/d(meta-net weights) into ``.grad`` of the meta-net parameters.

    meta_loss = -sum_tensors <smart_grad(train_grad, sharpness), vg/||vg||>; gradients do not flow into the
    inputs, the sort permutation, the previous GRU state or the initial scan state
    (reference supergrok2.py:815-1019).  Returns the number of tensors that contributed.
    ``checkpoint_interval`` C: on CUDA a scan state is kept every max(16, 16 * ceil(C / 16)) timesteps and the steps between
    are recomputed in the adjoint (``ops/sg2_bilevel.py: snapshot_tiles``); the PyTorch path processes one tensor at a time and
    keeps no scan states beyond that tensor's autograd graph.  The gradients do not depend on the interval.
    """
    mn = opt.meta_net
    first = next((p for _, p in named), None)
    if first is not None and first.is_cuda and supports_native(mn) and not getattr(opt, "bilevel_force_autograd", False):
        from .sg2_bilevel import bilevel_backward_cuda
        return bilevel_backward_cuda(opt, named, train_grads, val_grads, checkpoint_interval=checkpoint_interval)
    used = 0
    for name, p in named:
        if name not in train_grads or name not in val_grads:
            continue
        i = opt._param_to_idx.get(id(p))
        if i is None:
            continue
        vg = val_grads[name].detach().reshape(-1).float()
        if not bool(torch.isfinite(vg).all()):
            continue
        vn = vg.norm()
        vu = vg / vn if float(vn) > 1e-12 else vg
        g = train_grads[name].detach().reshape(-1).float()      # raw (unclipped) training gradient, as in the reference
        g = torch.where(torch.isfinite(g), g, torch.zeros_like(g))
        s = opt._flat_sharpness[i].reshape(-1).float()
        with torch.enable_grad():
            def fwd(g=g, s=s, i=i):
                return mn.forward_for_bilevel(g, s, opt._flat_gru_states[i], opt._flat_mamba_fwd_states[i],
                                              opt._flat_mamba_bwd_states[i])[0]
            smart = fwd()
            loss = -(smart.reshape(-1) * vu).sum()
            loss.backward()           # per tensor: the graph of one tensor is alive at a time
        used += 1
    return used
