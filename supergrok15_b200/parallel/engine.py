"""ZeRO-2 data-parallel training engine with in-kernel collectives.

One process per GPU.  The model is replicated in low precision (bf16); gradients are written by autograd
into one flat peer-mapped buffer; the fp32 master weights and every optimizer state are sharded: each
rank keeps them only for the tensors (or flat range) it owns.  A step is

    barrier (all gradients written)
    owner pulls the peers' gradient shards over NVLink and reduces them in fp32 registers
    sharded optimizer step on the fp32 master
    updated low-precision parameters are stored into every peer's parameter buffer
    barrier (all parameters written)

For SuperGrok v2 the pull feeds the batched sort/scan pipeline and the element-step kernel itself stores
the new bf16 parameters to the peers (all-gather fused into the step).  For AdamW and Lion the whole step
is ONE kernel over the flat shard (reduce-scatter + step + all-gather).  The other optimizers use the
pull kernel, their multi-tensor kernels on the fp32 master, and a cast-and-push kernel; their global
scalars (clip norm, Prodigy numerator / denominator, SAM norm) are combined across ranks by a small
deterministic slot all-reduce.  ``comm="nccl"`` runs the same sharded step around NCCL all-reduce /
broadcast and is the baseline the fused path is measured against.

``overlap=True`` (AdamW / Lion) cuts the flat buffer into buckets of consecutive parameters, last parameters first, and
gives every rank an equal slice of EACH bucket.  A hook on the gradient accumulation of every parameter marks its bucket;
as soon as a bucket is complete (buckets are issued strictly in order, so that every rank issues the same sequence) a side
stream waits for that point of the backward stream, runs a barrier over the ranks and the fused reduce-scatter + step +
all-gather kernel on this rank's slice of the bucket, while backward carries on with the earlier layers on the main stream.
With ``comm="nccl"`` (and on CPU / gloo) the bucket's all-reduce is started asynchronously at the same point instead.

Waits on peers are bounded on the device (``timeout_s``); ``check()`` raises ``CommTimeout`` when a wait
ran out, leaving the CUDA context usable.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..ops import nn_ops

from .. import _build
from .. import optim as O
from ..ops import elementwise as ew
from . import ownership, symm

FLAT_OPTIMIZERS = {"adamw": 0, "lion": 1}
OPTIMIZERS = {"supergrok2": O.SuperGrok2, "supergrok15": O.SuperGrok15, "supergrok11": O.SuperGrok11,
              "grokadamw": O.GrokAdamW, "neuralgrok": O.NeuralGrok, "prodigy": O.Prodigy, "grokfast": O.Grokfast,
              "lion": O.Lion, "looksam": O.LookSAM, "muon": O.Muon, "adamw": O.AdamW}
_DT = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}
# optimizers whose step combines global scalars across the ranks (every rank must take part in every such reduction)
_REDUCING = {"grokadamw", "neuralgrok", "supergrok15", "supergrok11", "prodigy", "looksam"}


class CommTimeout(RuntimeError):
    """A bounded device-side wait on a peer ran out (the peer id and the wait site are in the message)."""


class ZeroEngine:
    def __init__(self, model: torch.nn.Module, optimizer: str = "supergrok2", opt_kwargs: Optional[dict] = None,
                 comm: Optional[str] = None, param_dtype: torch.dtype = torch.bfloat16, group=None,
                 timeout_s: float = 20.0, criterion=None, graph: Optional[bool] = None, graph_warmup: int = 3,
                 overlap: bool = False, bucket_numel: int = 1 << 24, heartbeat=None, gather: str = "push"):
        self.comm = comm or os.environ.get("GROK_COMM", "p2p")
        assert self.comm in ("p2p", "nvls", "nccl")
        self.rank, self.world = symm.world_info(group)
        self.group = group
        self.name = optimizer
        self.opt_kwargs = dict(opt_kwargs or {})
        self.timeout_s = timeout_s
        self.criterion = criterion                                       # None: the fused softmax cross-entropy kernel
        # forward + backward of a step are captured into a CUDA graph per batch shape (after `graph_warmup` eager steps): the
        # small models of the grokking tasks launch hundreds of short kernels per step and are bound by the host otherwise
        self.use_graph = (os.environ.get("SG_GRAPH", "1") != "0") if graph is None else bool(graph)
        self.graph_warmup = graph_warmup
        self._graphs, self._graph_seen = {}, {}
        self.model = model.to(param_dtype)
        named = [(n, p) for n, p in self.model.named_parameters() if p.requires_grad]
        self.param_names = [n for n, _ in named]
        self.params = [p for _, p in named]
        self.device = self.params[0].device
        self.cuda = self.device.type == "cuda"
        self.pdtype = param_dtype
        numels = [p.numel() for p in self.params]
        self.flat_mode = optimizer in FLAT_OPTIMIZERS
        self.overlap = bool(overlap) and self.flat_mode                  # bucket-by-bucket overlap of the sharded step with backward
        if overlap and not self.flat_mode:
            import warnings
            warnings.warn(f"overlap=True is implemented for the flat optimizers ({', '.join(FLAT_OPTIMIZERS)}); '{optimizer}' needs "
                          "global scalars or whole tensors before its first update and runs its step after backward")
        self.buckets: List[dict] = []
        # gather="gemm" (AdamW / Lion): the rows of every Linear weight the fused kernel takes are owned by the ranks in turn; the
        # step updates only the owner's rows and the all-gather happens inside the first GEMM that consumes the weight
        assert gather in ("push", "gemm")
        self.gw_idx: List[int] = []
        self._gather_mods = []
        if gather == "gemm":
            if not (self.flat_mode and self.cuda and self.comm != "nccl" and not overlap):
                raise ValueError("gather='gemm' needs a flat optimizer (adamw / lion) on the in-kernel collectives, without overlap")
            by_id = {id(p): i for i, p in enumerate(self.params)}
            for mod in self.model.modules():
                if isinstance(mod, torch.nn.Linear) and id(mod.weight) in by_id:
                    n_out, n_in = mod.weight.shape
                    if n_out % (32 * self.world) == 0 and n_in % 8 == 0 and param_dtype == torch.bfloat16:
                        self.gw_idx.append(by_id[id(mod.weight)])
                        self._gather_mods.append(mod)
        # ---- layout of the flat parameter / gradient buffers
        if self.flat_mode:
            self.owner = [0] * len(numels)
            gw = set(self.gw_idx)
            order = self.gw_idx + [i for i in range(len(numels)) if i not in gw]     # row-owned weights first, the rest after them
            offs, pos = [0] * len(numels), 0
            self.rest_lo = 0
            for k, i in enumerate(order):
                if k == len(self.gw_idx) and self.gw_idx:               # the rest starts on a boundary every rank's slice can share
                    pos = self.rest_lo = -(-pos // (8 * self.world)) * 8 * self.world
                offs[i] = pos
                pos += -(-numels[i] // 8) * 8
            total = self.rest_lo + -(-(pos - self.rest_lo) // (8 * self.world)) * 8 * self.world
            self.offsets, self.total = offs, total
            self.regions = ownership.flat_ranges(total, self.world)
            if self.overlap:
                # every rank owns an equal slice of every bucket: its state is the concatenation of those slices
                so = 0
                for lo, hi, idx in ownership.reverse_buckets(offs, numels, int(bucket_numel)):
                    sl = ownership.bucket_slices(lo, hi, self.world)
                    b, e = sl[self.rank]
                    self.buckets.append({"lo": lo, "hi": hi, "params": idx, "slices": sl, "mine": (b, e), "state_off": so})
                    so += e - b
        else:
            # Muon with sharding="rows": the rows of every block matrix the fused kernels take are split over the ranks (the
            # Newton-Schulz GEMMs then carry their own collectives, ops/muon_sharded.py); everything else is owned whole
            self.rs_idx: List[int] = []
            if optimizer == "muon" and self.opt_kwargs.pop("sharding", "tensors") == "rows":
                from ..ops import muon_sharded
                if not (self.cuda and self.comm != "nccl"):
                    raise ValueError("Muon with sharding='rows' runs on the in-kernel collectives (CUDA, comm 'p2p' or 'nvls')")
                skip = tuple(self.opt_kwargs.get("adamw_names", ()))
                self.rs_idx = [i for i, p in enumerate(self.params) if p.dim() == 2 and not any(s_ in self.param_names[i] for s_ in skip)
                               and muon_sharded.supported(p.shape[0], p.shape[1], self.world)]
            rs = set(self.rs_idx)
            whole = [i for i in range(len(numels)) if i not in rs]
            sub = ownership.assign_tensors([numels[i] for i in whole], self.world)
            self.owner = [-1] * len(numels)
            for i, o in zip(whole, sub):
                self.owner[i] = o
            self.offsets, self.regions, self.total = ownership.grouped_layout(numels, self.owner, self.world)
            for i in self.rs_idx:                                     # row-sharded tensors follow the owned regions
                self.offsets[i] = self.total
                self.total += -(-numels[i] // 8) * 8
            if optimizer in _REDUCING and len(set(o for o in self.owner if o >= 0)) < self.world:
                # the element-wise optimizers combine global scalars (clip norm, Prodigy sums, ...) across the ranks from inside
                # their step; a rank without tensors would skip those collectives and the sequences would diverge
                raise ValueError(f"'{optimizer}' shards whole tensors: {len(numels)} parameter tensors cannot give each of "
                                 f"{self.world} ranks one; use fewer ranks, or 'adamw' / 'lion' / 'supergrok2'")
        self.my_begin, self.my_end = self.regions[self.rank]
        # (begin, end, offset into this rank's state) of every flat range this rank owns: one range, or one per bucket
        self.seg_push: Dict[int, bool] = {}                             # segment begin -> False when the all-gather is left to the first GEMM
        if self.overlap:
            self.segments = [(bk["mine"][0], bk["mine"][1], bk["state_off"]) for bk in self.buckets if bk["mine"][1] > bk["mine"][0]]
        elif self.gw_idx:
            self.segments, so = [], 0
            for i in self.gw_idx:                                        # this rank's rows of every row-owned weight
                per = numels[i] // self.world
                b = self.offsets[i] + self.rank * per
                self.segments.append((b, b + per, so))
                self.seg_push[b] = False
                so += per
            per = (self.total - self.rest_lo) // self.world               # an equal slice of everything else
            if per:
                self.segments.append((self.rest_lo + self.rank * per, self.rest_lo + (self.rank + 1) * per, so))
        else:
            self.segments = [(self.my_begin, self.my_end, 0)] if self.my_end > self.my_begin else []
        self.n_own = sum(e - b for b, e, _ in self.segments)
        self.pbuf = symm.alloc(self.total, param_dtype, self.device, group)
        self.gbuf = symm.alloc(self.total, param_dtype, self.device, group)
        with torch.no_grad():
            for p, off in zip(self.params, self.offsets):
                view = self.pbuf.tensor[off:off + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.gbuf.tensor[off:off + p.numel()].view(p.shape)
        # ---- signalling and small all-reduce scratch
        self.pads = symm.alloc(64, torch.int32, self.device, group)
        self.slots_n = 16384
        self.slots = symm.alloc(self.slots_n * max(self.world, 1), torch.float32, self.device, group)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch = 0
        self._calls = 0                                                  # steps started so far (start-up steps wait longer for their peers)
        self._sink_stream = None                                         # side stream of the weight-gradient GEMMs (see _fwd_bwd)
        # the status word is copied to pinned host memory after every step and looked at before the next one is launched
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory() if self.cuda else None
        self._status_event = None
        self.heartbeat = heartbeat
        # NVLS (in-switch reduction / replication through the multicast mapping) needs multicast addresses for both buffers
        self.nvls = self.comm == "nvls" and self.world > 1 and self.gbuf.multicast_ptr != 0 and self.pbuf.multicast_ptr != 0
        if self.comm == "nvls" and self.world > 1 and not self.nvls:
            import warnings
            warnings.warn("comm='nvls' requested but no multicast address is available; using plain peer loads / stores")
        # ---- owner state
        n_own = self.n_own
        self.master = (torch.cat([self.pbuf.tensor[b:e].float() for b, e, _ in self.segments]) if self.segments
                       else torch.zeros(0, dtype=torch.float32, device=self.device))       # fp32 master shard
        self.gred = torch.zeros(max(n_own, 1), dtype=torch.float32, device=self.device)    # reduced fp32 gradient shard
        self._build_optimizer()
        self.steps = 0
        self.launches = 0
        self.param_version = 0                                         # bumped by every step: a weight gathered at an older version is stale
        if self.gw_idx:
            from . import gather_linear
            gather_linear.install(self, self._gather_mods, self.gw_idx)
            self.use_graph = False            # the gathering GEMMs take their call number by value: forward is not replayed from a graph
        # In-kernel collectives with every per-step scalar in a device table: the whole step (barrier, reduce-scatter + optimizer +
        # all-gather, barrier) is a fixed launch sequence and is captured into the same CUDA graph as forward / backward.
        self.fused = self.cuda and self.comm != "nccl"
        self.device_step = self.fused and not self.overlap and (self.flat_mode or (self.name == "supergrok2" and self._sg2_native))
        if self.device_step:
            from ..ops import sg2 as sg2_ops
            if self.name == "supergrok2":
                self.dyn = sg2_ops.dyn_table(self.opt, len(self.own_idx), self.device)
            else:
                self.dyn = torch.zeros(sg2_ops.DYN_WORDS + 4, dtype=torch.float32, device=self.device)
        self._step_hp = None
        if self.overlap:
            import functools
            self.use_graph = False                    # epochs and bias corrections are host-side arguments of the bucket kernels
            self._ostream = torch.cuda.Stream(self.device) if self.cuda else None
            self._armed, self._next = False, 0
            for k, bk in enumerate(self.buckets):
                bk["pending"], bk["ready"], bk["handle"] = len(bk["params"]), False, None
                for i in bk["params"]:
                    self.params[i].register_post_accumulate_grad_hook(functools.partial(self._on_grad, k))

    # ------------------------------------------------------------------ construction
    def _owned(self):
        return [i for i, o in enumerate(self.owner) if o == self.rank]

    def _build_optimizer(self):
        kw = self.opt_kwargs
        if self.flat_mode:
            n = self.n_own
            self.m = torch.zeros(max(n, 8), dtype=torch.float32, device=self.device)
            self.v = torch.zeros(max(n, 8), dtype=torch.float32, device=self.device) if self.name == "adamw" else None
            self.hp = dict(lr=kw.get("lr", 1e-3 if self.name == "adamw" else 3e-4),
                           betas=kw.get("betas", (0.9, 0.999) if self.name == "adamw" else (0.9, 0.99)),
                           eps=kw.get("eps", 1e-8), weight_decay=kw.get("weight_decay", 1e-2 if self.name == "adamw" else 3.0))
            self.opt = None
            return
        own = self._owned()
        self.own_idx = own
        b = self.my_begin
        # the optimizer sees fp32 master views as its parameters; gradients are views of the reduced shard
        self.master_views = [torch.nn.Parameter(self.master[self.offsets[i] - b:self.offsets[i] - b + self.params[i].numel()]
                                                .view(self.params[i].shape), requires_grad=False) for i in own]
        self.grad_views = [self.gred[self.offsets[i] - b:self.offsets[i] - b + self.params[i].numel()].view(self.params[i].shape)
                           for i in own]
        cls = OPTIMIZERS[self.name]
        if self.name == "supergrok2":
            # v2 updates the low-precision parameter views directly and keeps the fp32 master beside them
            views = [torch.nn.Parameter(self.params[i].data, requires_grad=False) for i in own] or \
                    [torch.nn.Parameter(torch.zeros(0, device=self.device))]
            self.opt = cls(views, **kw)
            self.opt._external_recycle = True                         # recycling runs in step() below, after the counts are summed
            from ..ops import sg2 as sg2_ops
            self._sg2_native = self.cuda and sg2_ops.supports_native(self.opt.meta_net)
            if self.cuda:
                self.opt.meta_net.to(self.device)
            if own:
                self.opt._ensure_state()
                self.opt._flat_masters = [mv.data.reshape(-1) for mv in self.master_views]
                if self.cuda and self.comm != "nccl" and self._sg2_native:
                    # the first kernel of the v2 pipeline reads this rank's tensors out of every rank's gradient buffer itself
                    self.opt._pull_grads = [self.params[i].grad.reshape(-1) for i in own]
                else:
                    self.opt._grad_override = [g.reshape(-1) for g in self.grad_views]
                if self.cuda and self.world > 1 and self.comm != "nccl":
                    peers = [p for r, p in enumerate(self.pbuf.peer_ptrs) if r != self.rank]
                    self.opt._peer_push = (self.pbuf.peer_ptrs[self.rank], peers)
            self._fix_layer_schedules(own)
        elif self.name == "muon":
            # 2-D weights go to the Newton-Schulz group unless their name matches ``adamw_names`` (embeddings, output head)
            kw = dict(kw)
            skip = tuple(kw.pop("adamw_names", ()))
            is_mat = [mv.dim() == 2 and not any(s_ in self.param_names[i] for s_ in skip) for mv, i in zip(self.master_views, own)]
            p2 = [mv for mv, f in zip(self.master_views, is_mat) if f]
            p1 = [mv for mv, f in zip(self.master_views, is_mat) if not f]
            self.opt = cls(p2 or [torch.nn.Parameter(torch.zeros(8, 8, device=self.device))], p1, **kw)
            if self.rs_idx:
                self._build_row_sharded(kw)
        else:
            self.opt = cls(self.master_views or [torch.nn.Parameter(torch.zeros(0, device=self.device))], **kw)
            if hasattr(self.opt, "_flat_layer_beta1s"):
                self._fix_layer_schedules(own)

    def _build_row_sharded(self, kw):
        """State of the row-sharded matrices: this rank's rows of the fp32 master and of the momentum, and the fused
        Newton-Schulz object (its symmetric buffers are one allocation for all matrices)."""
        from ..ops import muon_sharded
        W, r = self.world, self.rank
        self.rs_hp = dict(lr=kw.get("lr", 0.02), momentum=kw.get("momentum", 0.95), weight_decay=kw.get("weight_decay", 1.0),
                          ns_steps=kw.get("ns_steps", 5))
        shapes = [tuple(self.params[i].shape) for i in self.rs_idx]
        sizes = [(R // W) * C for R, C in shapes]
        tot = sum(sizes)
        self.rs_master = torch.empty(tot, dtype=torch.float32, device=self.device)
        self.rs_mom = torch.zeros(tot, dtype=torch.float32, device=self.device)
        self.rs_gred = torch.zeros(tot, dtype=torch.float32, device=self.device)
        self.rs_views, pos = [], 0
        for i, (R, C), n in zip(self.rs_idx, shapes, sizes):
            lo = self.offsets[i] + r * n                              # this rank's rows are one contiguous range of the flat buffers
            self.rs_master[pos:pos + n].copy_(self.pbuf.tensor[lo:lo + n])
            self.rs_views.append(dict(flat_lo=lo, n=n, master=self.rs_master[pos:pos + n], mom=self.rs_mom[pos:pos + n],
                                      gred=self.rs_gred[pos:pos + n], shape=(R // W, C)))
            pos += n
        self.rs_ns = muon_sharded.RowShardedNewtonSchulz(shapes, self.device, self.group, status=self.status, timeout_s=self.timeout_s)
        C = _build.require()
        nb = C.mt_num_blocks(sizes)
        self.rs_partials = torch.empty(3 * max(nb, 1), dtype=torch.float32, device=self.device)
        self.rs_pt = torch.zeros(3 * len(sizes), dtype=torch.float32, device=self.device)
        self.rs_inv = torch.zeros(len(sizes), dtype=torch.float32, device=self.device)

    @torch.no_grad()
    def _step_row_sharded(self):
        """Muon on the row-sharded matrices: gradient rows pulled from every rank, momentum, norm of the whole matrix (partial
        sums combined over the ranks), five Newton-Schulz iterations whose GEMMs carry the collectives, update of the master
        rows, and the new low-precision rows stored into every rank's parameter buffer."""
        C = _build.require()
        hp, W, r = self.rs_hp, self.world, self.rank
        dt = _DT[self.pdtype]
        for v in self.rs_views:
            C.dist_pull_reduce(dt, self.nvls, self.gbuf.peer_ptrs, self.gbuf.multicast_ptr, r, v["flat_lo"], v["n"], 1.0 / W, v["gred"])
        grads, moms = [v["gred"] for v in self.rs_views], [v["mom"] for v in self.rs_views]
        C.mt_apply(C.ops["OP_MUON_MOMENTUM"], [[], grads, moms], [], [0, 0, 0, 0, 0, hp["momentum"]], partials=self.rs_partials,
                   per_tensor_out=self.rs_pt)
        self.all_reduce_small(self.rs_pt)                             # sum of squares of the WHOLE matrices
        C.scalar_finalize(C.ops["SC_MUON_NORMS"], self.rs_pt, len(self.rs_views), self.rs_inv, 0.0, 0.0, 0.0)
        outs = self.rs_ns.run([v["mom"].view(v["shape"]) for v in self.rs_views], hp["ns_steps"], scales=self.rs_inv)
        C.mt_apply(C.ops["OP_MUON_UPDATE"], [[v["master"] for v in self.rs_views], [o.view(-1) for o in outs]], [],
                   [0, 0, 0, 0, 0, 0, 0, 0, -0.2 * hp["lr"], 1.0 - hp["lr"] * hp["weight_decay"]])
        for v in self.rs_views:
            C.dist_cast_push(dt, self.pbuf.peer_ptrs, r, v["flat_lo"], v["n"], v["master"])
        self.launches += 4 * len(self.rs_views)

    def _fix_layer_schedules(self, own):
        """Layer-wise beta1 / alpha factors are functions of the parameter's index in the FULL model."""
        o = self.opt
        n_all = len(self.params)
        beta1 = o.param_groups[0]["betas"][0]
        for k, i in enumerate(own):
            o._flat_layer_beta1s[k] = beta1 * ((1.0 - o.gamma) ** i)
            o._flat_layer_alphas[k] = 1.0 if o.gamma_alpha == 0.0 else (1.0 - o.gamma_alpha) ** (max(n_all - 1, 1) - i)

    # ------------------------------------------------------------------ collectives
    def _wait_limit(self) -> float:
        """Seconds a device-side wait on a peer may last.  The first steps of a run see seconds of skew between the ranks that has
        nothing to do with a lost peer (lazy library initialisation, kernel loading, CUDA-graph capture and instantiation under
        whatever load the host has), so they get at least a minute; afterwards ``timeout_s`` applies (a captured barrier keeps
        the limit it was captured with, and capture happens after the start-up steps)."""
        if self.cuda and torch.cuda.is_current_stream_capturing():
            return self.timeout_s
        return max(self.timeout_s, 60.0) if self._calls <= self.graph_warmup + 1 else self.timeout_s

    def _barrier(self, site: int):
        if self.world == 1:
            return
        if self.cuda and self.comm != "nccl":
            self.epoch += 1
            _build.require().dist_barrier(self.pads.peer_ptrs, self.rank, self.epoch, self.status, self._wait_limit(), site)
            self.launches += 1
        else:
            import torch.distributed as dist
            dist.barrier(self.group)

    def _barrier_dyn(self, k: int, site: int):
        """Barrier k (1 or 2) of a device step: its epoch is the step's base epoch in the device table plus k, so the launch is
        the same every step and can be replayed from a CUDA graph."""
        if self.world > 1:
            _build.require().dist_barrier(self.pads.peer_ptrs, self.rank, k, self.status, self._wait_limit(), site, self.dyn)
            self.launches += 1

    def all_reduce_small(self, vec: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """In-place deterministic sum of a small fp32 vector over the ranks (bitwise identical everywhere)."""
        if self.world == 1:
            return vec.mul_(scale) if scale != 1.0 else vec
        if self.cuda and self.comm != "nccl":
            C = _build.require()
            n = vec.numel()
            assert n <= self.slots_n
            C.dist_scatter_slots(self.slots.peer_ptrs, self.rank, vec.contiguous())
            self._barrier(3)
            C.dist_reduce_slots(self.slots.tensor, self.world, vec, scale)
            self._barrier(4)            # slots may be overwritten only after everybody has read them
            self.launches += 2
            return vec
        import torch.distributed as dist
        dist.all_reduce(vec, group=self.group)
        return vec.mul_(scale) if scale != 1.0 else vec

    def _raise_timeout(self, s: int):
        self.status.zero_()
        raise CommTimeout(f"rank {self.rank}: wait on peer {(s >> 8) & 0xff} timed out at site {(s >> 16) & 0xff}")

    def check(self):
        """Raise if a device-side wait timed out since the last check (reads one int from the device)."""
        s = int(self.status.item())
        if s & 0xff:
            self._raise_timeout(s)

    def _poll_status(self):
        """Called before a step is launched: looks at the copy of the status word that the previous step left in pinned host
        memory.  Once a wait has timed out the kernels that update optimizer state return without touching it (they read the
        status word), so no state is corrupted between the timeout and this raise.  Also asks the heartbeat, when one is given,
        whether a peer stopped beating before any kernel that would wait for it is launched."""
        if self.heartbeat is not None:
            from .fault import guard_step
            guard_step(self.heartbeat)
        if self._status_event is not None and self._status_event.query():
            self._status_event = None
            s = int(self._status_host[0])
            if s & 0xff:
                self._raise_timeout(s)

    def _publish_status(self):
        if self.cuda and self.world > 1 and self._status_event is None:
            self._status_host.copy_(self.status, non_blocking=True)
            self._status_event = torch.cuda.Event()
            self._status_event.record()

    # ------------------------------------------------------------------ step
    def zero_grad(self):
        self.gbuf.tensor.zero_()

    # ------------------------------------------------------------------ flat optimizers (AdamW / Lion)
    def _flat_args(self, step_no: int) -> List[float]:
        b1, b2 = self.hp["betas"]
        return [self.hp["lr"], b1, b2, self.hp["eps"], self.hp["weight_decay"], 1 - b1 ** step_no, 1 - b2 ** step_no, 1.0 / self.world]

    def _flat_fused_segment(self, b: int, e: int, so: int, f: List[float], dyn=None):
        """Fused reduce-scatter + step + all-gather kernel on the owned flat range [b, e), whose state starts at ``so``."""
        nvls = self.nvls
        _build.require().dist_fused_flat_step(FLAT_OPTIMIZERS[self.name], _DT[self.pdtype], _DT[self.pdtype], self.gbuf.peer_ptrs,
                                              self.pbuf.peer_ptrs, self.rank, b, e - b, f, self.master[so:], self.m[so:],
                                              self.v[so:] if self.v is not None else None, nvls,
                                              self.gbuf.multicast_ptr if nvls else 0, self.pbuf.multicast_ptr if nvls else 0, dyn,
                                              self.seg_push.get(b, True))
        self.launches += 1

    def _flat_host_segment(self, b: int, e: int, so: int, step_no: int):
        """CPU / NCCL path: the gradient range is already summed over the ranks; step on the fp32 master, cast back."""
        n = e - b
        g = self.gred[so:so + n].copy_(self.gbuf.tensor[b:e])
        if self.world > 1:
            g.mul_(1.0 / self.world)
        b1, b2 = self.hp["betas"]
        mp = [self.master[so:so + n]]
        if self.name == "adamw":
            ew.adamw(mp, [g], [self.m[so:so + n]], [self.v[so:so + n]], [step_no], self.hp["lr"], b1, b2, self.hp["eps"], self.hp["weight_decay"])
        else:
            ew.lion(mp, [g], [self.m[so:so + n]], self.hp["lr"], b1, b2, self.hp["weight_decay"])
        self.pbuf.tensor[b:e].copy_(self.master[so:so + n])

    # ------------------------------------------------------------------ overlap with backward, bucket by bucket
    def _arm(self):
        """Called before the backward pass whose gradients complete the step: from now on finished buckets are issued."""
        for bk in self.buckets:
            bk["pending"], bk["ready"], bk["handle"] = len(bk["params"]), False, None
        self._next, self._armed = 0, True

    def _on_grad(self, k: int, _param):
        if not self._armed:
            return
        bk = self.buckets[k]
        bk["pending"] -= 1
        if bk["pending"] == 0:
            bk["ready"] = True
            while self._next < len(self.buckets) and self.buckets[self._next]["ready"]:     # strictly in order: same sequence on every rank
                self._issue_bucket(self._next)
                self._next += 1

    @torch.no_grad()
    def _issue_bucket(self, k: int):
        bk = self.buckets[k]
        if self.cuda and self.comm != "nccl":
            ev = torch.cuda.Event()
            ev.record()                                               # this bucket's gradients are complete at this point of backward
            with torch.cuda.stream(self._ostream):
                self._ostream.wait_event(ev)
                self._barrier(10)                                     # ... on every rank
                b, e = bk["mine"]
                if e > b:
                    self._flat_fused_segment(b, e, bk["state_off"], self._flat_args(self.steps + 1))
        elif self.world > 1:
            import torch.distributed as dist
            bk["handle"] = dist.all_reduce(self.gbuf.tensor[bk["lo"]:bk["hi"]], group=self.group, async_op=True)

    @torch.no_grad()
    def _finish_overlapped_step(self):
        while self._next < len(self.buckets):                         # buckets that no hook completed (unused parameters, manual backward)
            self._issue_bucket(self._next)
            self._next += 1
        self._armed = False
        self.steps += 1
        if self.cuda and self.comm != "nccl":
            ev = torch.cuda.Event()
            ev.record(self._ostream)
            torch.cuda.current_stream(self.device).wait_event(ev)
        else:
            import torch.distributed as dist
            for bk in self.buckets:
                if bk["handle"] is not None:
                    bk["handle"].wait()
                    bk["handle"] = None
                b, e = bk["mine"]
                if e > b:
                    self._flat_host_segment(b, e, bk["state_off"], self.steps)
            if self.world > 1:
                for bk in self.buckets:
                    for rr, (b, e) in enumerate(bk["slices"]):
                        if e > b:
                            dist.broadcast(self.pbuf.tensor[b:e], src=rr, group=self.group)
        self._barrier(2)                                              # every rank's parameters are complete

    # ------------------------------------------------------------------ device step: host part, kernel sequence, host part
    def _host_pre(self, metrics: dict):
        """Host side of a device step: schedules and counters, then ONE tiny kernel that writes this step's scalars (barrier
        epoch base, learning rate, weight decay, per-tensor bias corrections) into the device table."""
        from ..ops import sg2 as sg2_ops
        C = _build.require()
        self._calls += 1
        base = self.epoch
        if self.world > 1:
            self.epoch += 2                                           # the two barriers of the step use base + 1 and base + 2
        if self.flat_mode:
            self.steps += 1
            f = self._flat_args(self.steps)
            C.write_table(self.dyn, [base & 0xffffffff, 0, 0, 0, 0, 0, 0, 0], [f[0], f[4], 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, f[5], f[6]])
            self.launches += 1
            return
        if self.own_idx:
            idx, per, hp = self.opt._prepare_step(**metrics)
            self._step_hp = (idx, hp)
            sg2_ops.refresh_weights(self.opt, self.device)
            sg2_ops.write_scalars(self.opt, per, lr=hp["lr"], wd_eff=hp["wd_eff"], dev=self.device, epoch_base=base)
        else:
            self.opt._global_step += 1
            C.write_table(self.dyn, [base & 0xffffffff], [])
        self.launches += 1

    def _device_step(self, hook=None):
        """The kernels of a step, identical every step (safe to capture): barrier, sharded step with the reduce-scatter in its
        first kernel and the all-gather in its last, barrier."""
        stage = hook                                                  # None: the pipeline is enqueued without phase marks
        hook = hook or (lambda _n: None)
        self._barrier_dyn(1, 1)                                       # every rank's backward has written its gradients
        hook("barrier")
        if self.flat_mode:
            f = self._flat_args(1)
            for b, e, so in self.segments:
                self._flat_fused_segment(b, e, so, f, dyn=self.dyn)
            hook("reduce+step+gather")
        elif self.own_idx:
            from ..ops import sg2 as sg2_ops
            idx, hp = self._step_hp
            sg2_ops.launch(self.opt, idx, beta2=hp["beta2"], eps=hp["eps"], clip=hp["clip"],
                           pull=(self.gbuf.peer_ptrs, self.rank, 1.0 / self.world), status=self.status, stage_hook=stage)
        self._barrier_dyn(2, 2)                                       # every rank's parameters are complete
        hook("barrier2")

    def _host_post(self):
        self.param_version += 1
        if self.name == "supergrok2":
            if self.own_idx:
                self.opt._after_step()
            self._recycle_if_due()
        self._publish_status()

    def _recycle_if_due(self):
        """Expert recycling is driven here so that every rank does it at the same step on the same counts: each rank routed only
        the tensors it owns, so the 144 activation counts are summed over the ranks first (deterministic slot all-reduce)."""
        self._v2_steps = getattr(self, "_v2_steps", 0) + 1
        ri = self.opt.meta_net.recycle_interval
        if ri > 0 and self._v2_steps % ri == 0:
            counts = self.opt.meta_net.expert_counts
            if self.world > 1:
                cf = counts.float()
                self.all_reduce_small(cf)
                counts.copy_(cf.clamp_(max=2.0e9).to(counts.dtype))
            self.opt.recycle_dead_experts()

    @torch.no_grad()
    def step(self, **metrics):
        W, r = self.world, self.rank
        C = _build.require() if self.cuda else None
        n_own = self.n_own
        fused = self.cuda and self.comm != "nccl"
        if self.overlap:
            if not self._armed:                                       # step() after a backward that train_step did not drive
                self._arm()
            return self._finish_overlapped_step()
        if self.cuda:
            self._poll_status()
        if self.device_step:
            self._host_pre(metrics)
            self._device_step()
            self._host_post()
            return
        self._calls += 1
        self._barrier(1)                                              # every rank's backward has written its gradients
        # ---- reduce-scatter
        if fused:
            if n_own:
                C.dist_pull_reduce(_DT[self.pdtype], self.nvls, self.gbuf.peer_ptrs,
                                   self.gbuf.multicast_ptr, r, self.my_begin, n_own, 1.0 / W, self.gred)
                self.launches += 1
        else:
            if W > 1:
                import torch.distributed as dist
                dist.all_reduce(self.gbuf.tensor, group=self.group)
            if n_own:
                self.gred[:n_own].copy_(self.gbuf.tensor[self.my_begin:self.my_end])
                if W > 1:
                    self.gred.mul_(1.0 / W)
        # ---- sharded optimizer step
        if self.flat_mode:                                            # CPU / NCCL path of AdamW / Lion on the flat shard
            self.steps += 1
            for b, e, so in self.segments:
                self._flat_host_segment(b, e, so, self.steps)
        elif self.name == "supergrok2":
            if self.own_idx:
                self.opt.step(**metrics)
            else:
                self.opt._global_step += 1
            self._recycle_if_due()
        else:
            if getattr(self, "rs_idx", None):
                self._step_row_sharded()
            for mv, g in zip(self.master_views, self.grad_views):
                mv.grad = g
            ew.set_cross_rank_reducer(self.all_reduce_small if W > 1 else None)
            try:
                self.opt.step(**metrics) if metrics else self.opt.step()
            finally:
                ew.set_cross_rank_reducer(None)
            if n_own:
                if fused and self.nvls:
                    # cast into the local buffer, then one multimem.st per 16 bytes replicates it through the switch
                    self.pbuf.tensor[self.my_begin:self.my_end].copy_(self.master[:n_own])
                    es = self.pbuf.tensor.element_size()
                    C.dist_push(True, self.pbuf.peer_ptrs, self.pbuf.multicast_ptr, r, self.my_begin * es, n_own * es, self.pbuf.tensor)
                    self.launches += 1
                elif fused:
                    C.dist_cast_push(_DT[self.pdtype], self.pbuf.peer_ptrs, r, self.my_begin, n_own, self.master)
                    self.launches += 1
                else:
                    self.pbuf.tensor[self.my_begin:self.my_end].copy_(self.master[:n_own])
        # ---- all-gather (baseline path only: the fused paths pushed already)
        if W > 1 and not fused:
            import torch.distributed as dist
            for rr, (b, e) in enumerate(self.regions):
                if e > b:
                    dist.broadcast(self.pbuf.tensor[b:e], src=rr, group=self.group)
        self._barrier(2)                                              # every rank's parameters are complete
        self.param_version += 1
        self._publish_status()

    def _fwd_bwd(self, x: torch.Tensor, y: torch.Tensor, micro_batches: int) -> torch.Tensor:
        """Zero the flat gradient buffer, then forward + loss + backward of every micro-batch (gradients accumulate in the buffer)."""
        self.zero_grad()
        total = None
        chunks = list(zip(x.chunk(micro_batches), y.chunk(micro_batches)))
        # Parameter gradients are added to the flat buffer by the backward kernels themselves (no accumulation kernel per
        # parameter; weight-gradient GEMMs on a side stream).  Not with overlap: its buckets fire from autograd's accumulation hooks.
        sink = self.cuda and not self.overlap and os.environ.get("SG_GRAD_SINK", "1") != "0"
        if sink and self._sink_stream is None:
            self._sink_stream = torch.cuda.Stream(self.device)
        with nn_ops.grad_sink(sink, self._sink_stream if sink else None):
            for k, (xb, yb) in enumerate(chunks):
                if self.overlap and k == len(chunks) - 1:
                    self._arm()                                       # the gradients of this backward pass complete the step
                logits = self.model(xb)
                if logits.dim() == 3:                                 # language modelling: one target per position
                    logits, yb = logits.reshape(-1, logits.shape[-1]), yb.reshape(-1)
                if self.criterion is None:                            # reads the low-precision logits directly (fp32 arithmetic inside)
                    loss = nn_ops.cross_entropy(logits, yb)
                else:
                    loss = self.criterion(logits.float(), yb)
                if micro_batches > 1:
                    loss = loss / micro_batches
                loss.backward()
                total = loss.detach() if total is None else total + loss.detach()
        return total

    def _fwd_bwd_graphed(self, x: torch.Tensor, y: torch.Tensor, micro_batches: int, with_step: bool = False) -> torch.Tensor:
        """Forward + backward (and, ``with_step``, the kernels of the sharded step) through a CUDA graph captured per
        (shape, dtype, micro-batch count).  The first ``graph_warmup`` calls of a shape run eagerly (lazy initialisation,
        workspace growth); a capture that fails switches graphs off.  Every rank captures at the same call, and the barriers
        inside the graph take their epochs from the device table, so a replay is a complete step."""
        def body(xx, yy):
            total = self._fwd_bwd(xx, yy, micro_batches)
            if with_step:
                self._device_step()
            return total
        key = (tuple(x.shape), x.dtype, tuple(y.shape), y.dtype, micro_batches, self.model.training, with_step)
        entry = self._graphs.get(key)
        if entry is None:
            seen = self._graph_seen.get(key, 0)
            self._graph_seen[key] = seen + 1
            if seen < self.graph_warmup:
                return body(x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True))
            sx = torch.empty(x.shape, dtype=x.dtype, device=self.device)
            sy = torch.empty(y.shape, dtype=y.dtype, device=self.device)
            sx.copy_(x, non_blocking=True)
            sy.copy_(y, non_blocking=True)
            C = _build.require()
            try:
                torch.cuda.synchronize(self.device)
                g = torch.cuda.CUDAGraph()
                l0 = C.launch_count()
                with torch.cuda.graph(g):
                    total = body(sx, sy)
                entry = (g, sx, sy, total, C.launch_count() - l0)
                C.add_launches(-entry[4])                             # enqueued for the capture only; counted again at every replay
                self._graphs[key] = entry
            except Exception as exc:  # noqa: BLE001
                import warnings
                warnings.warn(f"CUDA graph capture of the step failed ({type(exc).__name__}: {exc}); running eagerly")
                self.use_graph = False
                torch.cuda.synchronize(self.device)
                return body(x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True))
        g, sx, sy, total, n_launch = entry
        sx.copy_(x, non_blocking=True)
        sy.copy_(y, non_blocking=True)
        g.replay()
        _build.require().add_launches(n_launch)
        return total.clone()                                          # the graph's own loss tensor is overwritten by the next replay

    # ------------------------------------------------------------------ the call a user makes
    def train_step(self, x: torch.Tensor, y: torch.Tensor, micro_batches: int = 1, **metrics) -> torch.Tensor:
        """Host (pinned) or device batch in, loss tensor out: H2D copy, forward, backward, sharded fused step.
        ``micro_batches`` > 1 splits the batch and accumulates gradients in the flat buffer (activation memory)."""
        if self.use_graph and self.cuda and self.device_step:
            # the whole step is one graph launch: host work is the schedule update and one table-writing kernel
            self._poll_status()
            self._host_pre(metrics)
            total = self._fwd_bwd_graphed(x, y, micro_batches, with_step=True)
            self._host_post()
            return total
        if self.use_graph and self.cuda:
            total = self._fwd_bwd_graphed(x, y, micro_batches)
        else:
            if x.device != self.device:
                x = x.to(self.device, non_blocking=True)
                y = y.to(self.device, non_blocking=True)
            total = self._fwd_bwd(x, y, micro_batches)
        self.step(**metrics)
        return total

    def profile_step(self, x: torch.Tensor, y: torch.Tensor, micro_batches: int = 1, **metrics) -> Dict[str, float]:
        """One eager step with CUDA events between its phases; returns milliseconds per phase on this rank.  The launches are
        queued behind a short device-side delay so that the phases run back to back, as they do when replayed from the graph
        (the host needs longer to enqueue the ~300 kernels of forward / backward than the GPU needs to run them)."""
        assert self.cuda and self.device_step, "per-phase timing covers the device step (in-kernel collectives)"
        from ..utils.timers import StepTimer
        timer = StepTimer()
        x, y = x.to(self.device), y.to(self.device)
        self._poll_status()
        self._host_pre(metrics)
        torch.cuda.synchronize(self.device)
        torch.cuda._sleep(int(3e7))
        timer.start()
        self._fwd_bwd(x, y, micro_batches)
        timer.mark("fwd+bwd")
        self._device_step(hook=timer.mark)
        self._host_post()
        return timer.finish()

    @torch.no_grad()
    def gather_params(self):
        """gather="gemm": make every rank's parameter buffer complete NOW (each owner stores its rows into the peers' buffers),
        for code that reads the weights outside a forward pass: evaluation through other modules, export, comparisons."""
        if not self.gw_idx or self.world == 1:
            return
        C = _build.require()
        es = self.pbuf.tensor.element_size()
        for b, e, _ in self.segments:
            if self.seg_push.get(b, True) is False:
                C.dist_push(False, self.pbuf.peer_ptrs, 0, self.rank, b * es, (e - b) * es, self.pbuf.tensor)
        self._barrier(5)
        for mod in self._gather_mods:
            mod._sg_gather.version = self.param_version

    # ------------------------------------------------------------------ introspection
    def state_bytes(self) -> int:
        n = self.master.numel() * 4 + self.gred.numel() * 4
        if self.opt is not None:
            for st in self.opt.state.values():
                n += sum(t.numel() * t.element_size() for t in st.values() if torch.is_tensor(t))
        return n

    def nvlink_bytes_per_step(self) -> Dict[str, int]:
        """Bytes over NVLink per step and rank on the fused path.  A rank pulls its shard of the gradients from the W - 1 peers
        and pushes its shard of the parameters to them; its INGRESS direction therefore carries its own pulls and the peers'
        pushes into its buffer (and the egress direction the mirror image), so every direction moves both amounts."""
        es = torch.tensor([], dtype=self.pdtype).element_size()
        n_shard = self.n_own + sum(v["n"] for v in getattr(self, "rs_views", []))
        pull = (self.world - 1) * n_shard * es
        pushed_to_me = (self.total - n_shard) * es if self.world > 1 else 0
        return {"rs_ingress": pull, "ag_egress": pull, "per_direction": pull + pushed_to_me}
