"""Newton-Schulz for matrices whose ROWS are sharded over the ranks, with every collective inside a tcgen05 GEMM kernel.

Rank r holds the row block ``X_r [R / W, C]`` of the normalised momentum of every matrix.  One iteration
``X <- a X + b (X X^T) X + c (X X^T)^2 X`` (reference csrc/ops.cpp:713-727, whole matrices on one GPU through ``torch::mm``) is
three kernels per matrix, each of which moves its operands over NVLink from inside the GEMM (``csrc/gemm_sm100.cu``):

  rows >= cols (right-Gram form, ``X (a I + b G + c G^2)``, ``G = X^T X = sum_r X_r^T X_r``):
    1. GEMM -> reduce-scatter   ``G_r``  = rows r of ``sum_r X_r^T X_r``: finished tiles go to their owner with peer stores, the
                                 owner adds the W partials in rank order in its own epilogue;
    2. all-gather -> GEMM       ``P_r``  = ``a I_r + b G_r + c G_r G``: copier CTAs pull the other ranks' ``G`` rows with peer loads
                                 while the MMA CTAs start on the local rows; the polynomial is the GEMM's epilogue;
    3. all-gather -> GEMM       ``X_r`` <- ``X_r P`` (``P`` gathered the same way), written in both layouts for the next step 1.
  rows < cols (left form, ``(a I + b A + c A^2) X``, ``A = X X^T``):
    1. all-gather -> GEMM       ``A_r``  = ``X_r X^T`` (the gather of ``X`` is the fused one; ``X`` stays in local memory for step 3);
    2. all-gather -> GEMM       ``B_r``  = ``a I_r + b A_r + c A_r A``;
    3. local GEMM               ``X_r`` <- ``B_r X``.

No rank ever forms a product it does not need: the work per rank is 1 / W of the whole iteration, and what crosses NVLink per
matrix and iteration is one square matrix twice (``G`` and ``P``, or ``X`` and ``A``).  All matrices of a step go through a phase
together, so the ranks meet at three barriers per iteration, not three per matrix.

Ordering: a shard is written by its owner's kernel, then every rank passes ``barrier()`` (stream-ordered: a rank signals after
its own kernels of the phase), then the kernels that gather it run.  Nothing here loads another GPU's memory through TMA: the
copiers use plain 16-byte peer loads into local memory and TMA reads local memory only.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

from .. import _build
from . import gemm as _gemm
from . import oracle

NS_COEFFS = oracle.NS_COEFFS


def supported(rows: int, cols: int, world: int) -> bool:
    """Shapes the fused kernels take: shard rows and gather groups must be whole tiles / 32-row groups and 16-byte rows."""
    if world < 1 or rows % world or cols % 8:
        return False
    if rows >= cols:
        return cols % (128 * world) == 0 and (rows // world) % 8 == 0
    return rows % (32 * world) == 0 and rows % 8 == 0


class SymmArena:
    """One symmetric (peer-mapped) allocation carved into buffers: a rendezvous per buffer would cost a collective each."""

    def __init__(self, nbytes: int, device, group=None):
        from ..parallel import symm
        self.buf = symm.alloc(max((nbytes + 255) // 256 * 256, 256), torch.uint8, device, group)
        self.rank, self.world = self.buf.rank, self.buf.world
        self.pos = 0

    def take(self, shape: Sequence[int], dtype: torch.dtype) -> Tuple[torch.Tensor, List[int]]:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        off = self.pos
        self.pos = (off + nbytes + 255) // 256 * 256
        assert self.pos <= self.buf.tensor.numel(), "symmetric arena too small"
        t = self.buf.tensor[off:off + nbytes].view(dtype).view(*shape)
        return t, [p + off for p in self.buf.peer_ptrs]


def arena_bytes(shapes: Sequence[Tuple[int, int]], world: int) -> int:
    total = 0
    for R, C in shapes:
        if R >= C:
            total += 2 * (C * C * 2 + 256)                                        # G, P
            total += 2 * world * (C // world) * C * 2 + 256                       # reduce-scatter slots [2][W][C/W][C]
            total += 2 * world * max(C // world // 128, 1) * 4 + 256              # reduce-scatter flags
        else:
            total += 2 * (R * C * 2 + 256) + R * R * 2 + 256                      # X (two parities), A
    return total + 4096


class _Mat:
    """Buffers and the three phases of one row-sharded matrix."""

    def __init__(self, R: int, C: int, arena: SymmArena, n_copy: int, it_dev: torch.Tensor):
        self.R, self.C, self.W, self.rank = R, C, arena.world, arena.rank
        self.it_dev = it_dev                                                      # device counter of Newton-Schulz iterations so far: the call
                                                                                  # number of every fused GEMM (one call per iteration each)
        W, r = self.W, self.rank
        self.Rl = R // W
        self.tall = R >= C
        dev = arena.buf.tensor.device
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.err = _gemm._err_flag(dev)
        self.n_copy = n_copy
        if self.tall:
            Cl = C // W
            self.X = [torch.empty(self.Rl, C, **bf) for _ in range(2)]
            self.XT = [torch.empty(C, self.Rl, **bf) for _ in range(2)]
            self.G, self.G_ptrs = arena.take((C, C), torch.bfloat16)
            self.P, self.P_ptrs = arena.take((C, C), torch.bfloat16)
            self.G_own, self.P_own = self.G[r * Cl:(r + 1) * Cl], self.P[r * Cl:(r + 1) * Cl]
            self.slots, self.slot_ptrs = arena.take((2 * W * Cl * C,), torch.bfloat16)
            self.flags, self.flag_ptrs = arena.take((2 * W * max(Cl // 128, 1),), torch.int32)
            self.flags.zero_()
            self.cnt_g = torch.zeros(2 + (C + 255) // 256, dtype=torch.int32, device=dev)
            self.cnt_p = torch.zeros(2 + (C + 255) // 256, dtype=torch.int32, device=dev)
            self.diag_off = r * Cl
        else:
            Xa, pa = arena.take((R, C), torch.bfloat16)
            Xb, pb = arena.take((R, C), torch.bfloat16)
            self.Xs, self.Xs_ptrs = [Xa, Xb], [pa, pb]
            self.X = [Xa[r * self.Rl:(r + 1) * self.Rl], Xb[r * self.Rl:(r + 1) * self.Rl]]
            self.A, self.A_ptrs = arena.take((R, R), torch.bfloat16)
            self.A_own = self.A[r * self.Rl:(r + 1) * self.Rl]
            self.B = torch.empty(self.Rl, R, **bf)
            self.cnt_x = torch.zeros(2 + (R + 255) // 256, dtype=torch.int32, device=dev)
            self.cnt_a = torch.zeros(2 + (R + 255) // 256, dtype=torch.int32, device=dev)
            self.diag_off = r * self.Rl
        self.out32 = torch.empty(self.Rl, C, dtype=torch.float32, device=dev)

    # ---- load the normalised shard (fp32 [R / W, C]) into the bf16 operands of iteration 0
    def load(self, x_shard: torch.Tensor, scale: Optional[torch.Tensor] = None):
        src = x_shard if scale is None else x_shard * scale
        self.X[0].copy_(src)
        if self.tall:
            self.XT[0].copy_(src.t())

    def phase1(self, it: int):
        C = _build.require()
        q = it & 1
        if self.tall:            # G_r = rows r of sum over ranks of X_r^T X_r      (GEMM -> reduce-scatter)
            C.gemm_tn_reducescatter(self.XT[q], self.XT[q], self.slot_ptrs, self.flag_ptrs, self.rank, self.G_own, 0, 10.0, self.err,
                                    epoch_dev=self.it_dev)
        else:                    # A_r = X_r X^T                                    (all-gather of X -> GEMM)
            C.gemm_tn_allgather(self.X[q], self.Xs_ptrs[q], self.rank, self.R, self.A_own, self.cnt_x, 0, self.n_copy, self.err,
                                epoch_dev=self.it_dev)

    def phase2(self, it: int, coeffs):
        C = _build.require()
        a, b, c = coeffs
        if self.tall:            # P_r = a I_r + b G_r + c G_r G                    (all-gather of G -> GEMM)
            C.gemm_tn_allgather(self.G_own, self.G_ptrs, self.rank, self.C, self.P_own, self.cnt_g, 0, self.n_copy, self.err,
                                alpha=c, beta=b, d=self.G_own, diag=a, diag_off=self.diag_off, epoch_dev=self.it_dev)
        else:                    # B_r = a I_r + b A_r + c A_r A                    (all-gather of A -> GEMM)
            C.gemm_tn_allgather(self.A_own, self.A_ptrs, self.rank, self.R, self.B, self.cnt_a, 0, self.n_copy, self.err,
                                alpha=c, beta=b, d=self.A_own, diag=a, diag_off=self.diag_off, epoch_dev=self.it_dev)

    def phase3(self, it: int, last: bool):
        C = _build.require()
        q = it & 1
        if self.tall:            # X_r <- X_r P                                     (all-gather of P -> GEMM), both layouts
            if last:
                C.gemm_tn_allgather(self.X[q], self.P_ptrs, self.rank, self.C, self.out32, self.cnt_p, 0, self.n_copy, self.err,
                                    epoch_dev=self.it_dev)
            else:
                C.gemm_tn_allgather(self.X[q], self.P_ptrs, self.rank, self.C, self.X[q ^ 1], self.cnt_p, 0, self.n_copy, self.err,
                                    out_t=self.XT[q ^ 1], epoch_dev=self.it_dev)
        else:                    # X_r <- B_r X                                     (X was gathered into local memory by phase 1)
            _gemm.gemm_tn(self.B, self.Xs[q], out=self.out32 if last else self.X[q ^ 1], b_t=True)


class RowShardedNewtonSchulz:
    """Newton-Schulz over a fixed list of row-sharded matrices.

    Everything a step needs lives on the device: the call number of the fused GEMMs (``it``, bumped by a one-thread kernel at
    the start of every iteration) and the epoch of the barriers between the phases (own signal pad; bumped the same way).  The
    launch sequence of a step is therefore identical every time, and from the third call with the same inputs on it is replayed
    from ONE CUDA graph (every rank captures at the same call): ~3 launches per matrix and iteration would otherwise be issued from
    Python, slower than the GPU runs them.  ``barrier``: a callable that orders the ranks on the current stream replaces the
    in-kernel barrier (and disables the graph); ``status``: the int32 status word that records a timed-out wait."""

    def __init__(self, shapes: Sequence[Tuple[int, int]], device, group=None, barrier: Optional[Callable[[], None]] = None,
                 n_copy_ctas: int = 16, status: Optional[torch.Tensor] = None, timeout_s: float = 20.0, graph: bool = True):
        from ..parallel import symm
        self.rank, self.world = symm.world_info(group)
        for R, C in shapes:
            if not supported(R, C, self.world):
                raise ValueError(f"row-sharded Newton-Schulz does not take a {R} x {C} matrix on {self.world} ranks")
        self.arena = SymmArena(arena_bytes(shapes, self.world), device, group)
        self.it = torch.zeros(1, dtype=torch.int32, device=device)
        self.mats = [_Mat(R, C, self.arena, n_copy_ctas, self.it) for R, C in shapes]
        self.user_barrier = barrier
        self.timeout_s = timeout_s
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=device)
        self.bar_epoch = torch.zeros(16, dtype=torch.int32, device=device)         # word 0: epoch of the next barrier
        self.pads = symm.alloc(64, torch.int32, device, group) if self.world > 1 and barrier is None else None
        self.use_graph = bool(graph) and barrier is None
        self._graphs, self._calls = {}, 0

    def barrier(self, site: int = 30):
        if self.world == 1:
            return
        if self.user_barrier is not None:
            return self.user_barrier()
        C = _build.require()
        C.dist_bump(self.bar_epoch)
        limit = self.timeout_s if torch.cuda.is_current_stream_capturing() or self._calls > 2 else max(self.timeout_s, 60.0)
        C.dist_barrier(self.pads.peer_ptrs, self.rank, 0, self.status, limit, site, self.bar_epoch.view(torch.float32))

    def _body(self, shards, steps, scales, coeffs):
        C = _build.require()
        for i, (m, x) in enumerate(zip(self.mats, shards)):
            m.load(x, None if scales is None else scales[i])
        self.barrier(30)                                 # wide form: every X_r is in place before anybody gathers it
        for it in range(steps):
            last = it == steps - 1
            C.dist_bump(self.it)
            for m in self.mats:
                m.phase1(it)
            self.barrier(31)
            for m in self.mats:
                m.phase2(it, coeffs)
            self.barrier(32)
            for m in self.mats:
                m.phase3(it, last)
            self.barrier(33)

    def run(self, shards: Sequence[torch.Tensor], steps: int, scales: Optional[torch.Tensor] = None, coeffs=NS_COEFFS) -> List[torch.Tensor]:
        """``shards[i]``: fp32 [R_i / W, C_i], this rank's rows of matrix i (``scales[i]``, a device scalar, is multiplied in:
        1 / (norm + eps) of the whole matrix).  Returns this rank's rows of the orthogonalised matrices (fp32, owned by this
        object and overwritten by the next call)."""
        self._calls += 1
        outs = [m.out32 for m in self.mats]
        if not self.use_graph or torch.cuda.is_current_stream_capturing():
            self._body(shards, steps, scales, coeffs)
            return outs
        key = (tuple(x.data_ptr() for x in shards), steps, None if scales is None else scales.data_ptr(), tuple(coeffs))
        ent = self._graphs.get(key, 0)
        if isinstance(ent, int) and ent < 2:              # two eager calls (lazy initialisation, both buffer parities), then capture
            self._graphs[key] = ent + 1
            self._body(shards, steps, scales, coeffs)
            return outs
        if isinstance(ent, int):
            try:
                torch.cuda.synchronize(shards[0].device)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._body(shards, steps, scales, coeffs)
                ent = self._graphs[key] = g
            except Exception as exc:  # noqa: BLE001
                import warnings
                warnings.warn(f"CUDA graph capture of the row-sharded Newton-Schulz failed ({type(exc).__name__}: {exc}); running eagerly")
                self.use_graph = False
                torch.cuda.synchronize(shards[0].device)
                self._body(shards, steps, scales, coeffs)
                return outs
        ent.replay()
        return outs

    def nvlink_bytes_per_iteration(self) -> int:
        """Bytes this rank receives per iteration: (W - 1) / W of two square matrices per matrix (bf16)."""
        W, n = self.world, 0
        for m in self.mats:
            side = m.C if m.tall else m.R
            first = side * side if m.tall else m.R * m.C
            n += (first + side * side) * 2 * (W - 1) // W
        return n
