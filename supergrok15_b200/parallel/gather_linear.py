"""Linear layers whose weight rows are owned by the ranks in turn, with the parameter all-gather inside the first consuming GEMM.

``ZeroEngine(..., gather="gemm")`` keeps every such weight ``[N, K]`` in the engine's peer-mapped parameter buffer; after the
sharded optimizer step only the owner's rows are current.  The first forward use of the weight in a step runs
``gemm_tn_allgather`` (``csrc/gemm_sm100.cu``): copier CTAs pull the other ranks' rows with plain 16-byte peer loads into this
rank's buffer while the tcgen05 CTAs already multiply the local rows; a tile's weights are loaded by TMA (local memory) once
their rows have arrived.  Afterwards the local buffer holds the whole weight, so later uses in the same step (more
micro-batches, dgrad in backward) are ordinary GEMMs on local memory.  This replaces the parameter push at the end of the step
for these weights: every remote byte still crosses NVLink once, but hidden behind the GEMM that needs it.

Ordering: the engine's closing barrier of a step orders the owners' writes before any gather of the next forward, and its
opening barrier (after backward) orders every gather before the owners write again.
"""
from __future__ import annotations

from typing import List

import torch

from .. import _build
from ..ops import gemm as _gemm


class _State:
    """Per-weight bookkeeping: the peer addresses of the weight, its arrival counters and the version it was gathered at."""

    def __init__(self, engine, index: int, n_copy: int):
        p = engine.params[index]
        self.N, self.K = p.shape
        off_bytes = engine.offsets[index] * p.element_size()
        self.ptrs: List[int] = [base + off_bytes for base in engine.pbuf.peer_ptrs]
        self.counters = torch.zeros(2 + (self.N + 255) // 256, dtype=torch.int32, device=p.device)
        self.calls = 0                      # gathers so far (the kernel's epoch)
        self.version = -1                   # engine.param_version at the last gather
        self.m = None                       # rows of the activation at the last gather (one counter set serves one problem size)
        self.engine, self.n_copy = engine, n_copy


class _GatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, st: _State):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        eng = st.engine
        if st.version != eng.param_version and eng.world > 1:
            C = _build.require()
            if st.m not in (None, x2.shape[0]):                         # another activation size: restart the tile tickets
                torch.cuda.current_stream(x2.device).synchronize()
                st.counters.zero_()
                st.calls = 0
            st.m = x2.shape[0]
            st.calls += 1
            out = torch.empty(x2.shape[0], st.N, dtype=x2.dtype, device=x2.device)
            C.gemm_tn_allgather(x2, st.ptrs, eng.rank, st.N, out, st.counters, st.calls, st.n_copy, _gemm._err_flag(x2.device))
            st.version = eng.param_version
            eng.launches += 1
        else:
            out = torch.nn.functional.linear(x2, weight)
        if bias is not None:
            out = out + bias
        ctx.save_for_backward(x2, weight)
        ctx.has_bias, ctx.xshape = bias is not None, x.shape
        return out.view(*x.shape[:-1], st.N)

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = (dy2 @ weight).view(ctx.xshape)                             # the whole weight is in local memory by now
        dw = dy2.t() @ x2
        db = dy2.sum(0) if ctx.has_bias else None
        return dx, dw, db, None


def install(engine, modules, indices, n_copy: int = 24) -> None:
    """Route ``forward`` of the given ``nn.Linear`` modules through the gathering GEMM."""
    for mod, i in zip(modules, indices):
        st = _State(engine, i, n_copy)
        mod._sg_gather = st
        mod.forward = (lambda x, _m=mod, _st=st: _GatherLinear.apply(x, _m.weight, _m.bias, _st))
