"""GEMMs fused with their collective (``csrc/gemm_sm100.cu``): the transfer overlaps the tensor-core tiles inside ONE kernel.

``ShardedWeight``   a bf16 weight [N, K] whose rows are sharded over the ranks in symmetric memory.  ``matmul(x)`` computes
                    ``x @ W_full.T`` with the all-gather inside the GEMM: copier CTAs pull the remote shards over NVLink with plain
                    peer loads while the MMA CTAs start on the local shard; a tile's B operand is loaded (TMA, local memory) once its
                    row groups have arrived (release/acquire counters, bounded waits).  Every remote byte crosses NVLink once.

``ReduceScatterGemm``  ``a_r [M, K_r] @ b_r[N, K_r].T`` summed over the ranks, rank r keeping rows ``[r*M/W, (r+1)*M/W)``: the epilogue of
                    every tile sends it to its owner with peer stores, and the CTAs that run out of tiles reduce this rank's rows as
                    the blocks arrive (release/acquire counters across GPUs, bounded waits, fixed rank order: deterministic).

The reference keeps every parameter replicated and has no collective at all (its ``nn.Linear`` calls cuBLAS,
grokking_race_v2.py:310-331); this is the parameter all-gather of a ZeRO-3 / FSDP layout fused into the first consumer.

Ordering contract: the owner writes its shard, then every rank passes a barrier (``ZeroEngine`` uses its in-kernel barrier,
tests use ``dist.barrier``), then ``matmul`` may run; a second barrier is needed before the shards are overwritten again.
"""
from __future__ import annotations

import torch

from .. import _build
from ..ops import gemm as _gemm
from . import symm


class ShardedWeight:
    def __init__(self, n_rows: int, n_cols: int, device, group=None, n_copy_ctas: int = 24):
        self.rank, self.world = symm.world_info(group)
        if n_rows % (32 * self.world) or n_cols % 8:
            raise ValueError("ShardedWeight needs rows % (32 * world) == 0 and cols % 8 == 0")
        self.N, self.K = n_rows, n_cols
        self.buf = symm.alloc(n_rows * n_cols, torch.bfloat16, device, group)
        self.full = self.buf.tensor.view(n_rows, n_cols)                 # local [N, K] buffer: own rows valid, the rest is gather space
        self.rows = n_rows // self.world
        # [0:2] 64-bit tile ticket counter, [2:] per-tile arrival counters; all monotone over the calls, never reset
        self.counters = torch.zeros(2 + (n_rows + 255) // 256, dtype=torch.int32, device=device)
        self._m = None
        self.epoch = 0
        self.n_copy = n_copy_ctas

    @property
    def shard(self) -> torch.Tensor:
        """This rank's rows (the only ones it may write)."""
        return self.full[self.rank * self.rows:(self.rank + 1) * self.rows]

    def matmul(self, x: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
        """x [M, K] bf16 -> x @ W_full.T [M, N]; afterwards ``self.full`` holds the gathered weight (usable by later GEMMs)."""
        C = _build.require()
        if self._m not in (None, x.shape[0]):                            # the ticket arithmetic assumes one problem size per counter set
            torch.cuda.current_stream(x.device).synchronize()
            self.counters.zero_()
            self.epoch = 0
        self._m = x.shape[0]
        self.epoch += 1
        out = torch.empty(x.shape[0], self.N, dtype=out_dtype, device=x.device)
        C.gemm_tn_allgather(x, self.buf.peer_ptrs, self.rank, self.N, out, self.counters, self.epoch, self.n_copy, _gemm._err_flag(x.device))
        return out


class ReduceScatterGemm:
    """Row-parallel product with the reduce-scatter inside the GEMM kernel (one instance per problem shape)."""

    def __init__(self, M: int, N: int, device, group=None, timeout_s: float = 5.0):
        self.rank, self.world = symm.world_info(group)
        if M % (128 * self.world) or N % 64:
            raise ValueError("ReduceScatterGemm needs M % (128 * world) == 0 and N % 64 == 0")
        self.M, self.N, self.timeout_s = M, N, timeout_s
        mloc = M // self.world
        self.slots = symm.alloc(2 * self.world * mloc * N, torch.bfloat16, device, group)      # [parity][sender][M/W][N]
        self.flags = symm.alloc(2 * self.world * (mloc // 128), torch.int32, device, group)    # [parity][sender][128-row block]
        self.epoch = 0

    def __call__(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        C = _build.require()
        self.epoch += 1
        out = torch.empty(self.M // self.world, self.N, dtype=torch.bfloat16, device=a.device)
        C.gemm_tn_reducescatter(a, b, self.slots.peer_ptrs, self.flags.peer_ptrs, self.rank, out, self.epoch, self.timeout_s,
                                _gemm._err_flag(a.device))
        return out
