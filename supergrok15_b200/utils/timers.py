"""Step timing on the device (CUDA events on the launching stream), NVTX ranges, and the max-over-ranks reduction."""
from __future__ import annotations

import contextlib
from collections import defaultdict
from typing import Dict, List

import torch


class StepTimer:
    """``with timer.phase("fwd"): ...`` records a CUDA-event pair per phase; ``summary()`` synchronises once and
    returns mean milliseconds per phase (max over ranks when a process group is initialised)."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._ev: Dict[str, List] = defaultdict(list)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        torch.cuda.nvtx.range_push(name)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        try:
            yield
        finally:
            e1.record()
            torch.cuda.nvtx.range_pop()
            self._ev[name].append((e0, e1))

    # ---- consecutive phases of one step: start(), mark(name) after each phase, finish() -> {name: ms} on this rank
    def start(self):
        self._marks = []
        if self.enabled:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._marks.append((None, e))

    def mark(self, name: str):
        if self.enabled:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._marks.append((name, e))

    def finish(self) -> Dict[str, float]:
        if not self.enabled or not getattr(self, "_marks", None):
            return {}
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        for (_, a), (name, b) in zip(self._marks[:-1], self._marks[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        self._marks = []
        return out

    def summary(self, reset: bool = True) -> Dict[str, float]:
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        out = {k: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1) for k, v in self._ev.items()}
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            keys = sorted(out)
            t = torch.tensor([out[k] for k in keys], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out = dict(zip(keys, t.tolist()))
        if reset:
            self._ev.clear()
        return out


@contextlib.contextmanager
def nvtx(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
