"""Replay an optimizer step as a CUDA graph (reference grokking_optimizers/cuda_graph_optimizer.py:56-168).

After ``warmup_steps`` eager steps the wrapped ``optimizer.step()`` is captured once with static
gradient buffers; later steps copy the live gradients into those buffers and replay the graph.
Keyword arguments to ``step`` (metrics for the SuperGrok schedules) force an eager step, a failed
capture falls back to eager for good, ``invalidate()`` or an age limit triggers a re-record.
Because the optimizers of this package keep their reductions on the device, steps that the
reference could not capture (global clip, Prodigy, Muon norms) capture here.  Per-step host scalars
(bias corrections) are baked into a capture, so use ``max_graph_age`` with schedules that change.
"""
from __future__ import annotations

import warnings
from typing import List, Optional

import torch


class CUDAGraphOptimizer:
    def __init__(self, optimizer: torch.optim.Optimizer, warmup_steps: int = 3, max_graph_age: int = 0):
        self.optimizer = optimizer
        self.warmup_steps = warmup_steps
        self.max_graph_age = max_graph_age
        self._step_count = 0
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._graph_age = 0
        self._static_grads: List[Optional[torch.Tensor]] = []
        self._params: List[torch.Tensor] = []
        self._capture_failed = False

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def state(self):
        return self.optimizer.state

    def _all_params(self):
        return [p for g in self.optimizer.param_groups for p in g["params"]]

    def _on_cuda(self) -> bool:
        ps = self._all_params()
        return bool(ps) and ps[0].is_cuda

    def step(self, closure=None, **kwargs):
        self._step_count += 1
        if (closure is not None or kwargs or self._capture_failed or not self._on_cuda()
                or self._step_count <= self.warmup_steps):
            if kwargs:
                self.invalidate()
            return self.optimizer.step(closure, **kwargs) if closure is not None else self.optimizer.step(**kwargs)
        if self._graph is not None and self.max_graph_age > 0 and self._graph_age >= self.max_graph_age:
            self.invalidate()
        if self._graph is None:
            self._record_graph()
            if self._graph is None:
                return self.optimizer.step()
            self._graph.replay()          # capturing records the work without running it
            return None
        self._swap_grads()
        self._graph.replay()
        self._graph_age += 1
        return None

    def _record_graph(self):
        self._params = self._all_params()
        self._static_grads = [p.grad.detach().clone() if p.grad is not None else None for p in self._params]
        live = [p.grad for p in self._params]
        for p, sg in zip(self._params, self._static_grads):
            p.grad = sg
        try:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.optimizer.step()
            self._graph, self._graph_age = g, 1
        except Exception as e:  # noqa: BLE001
            warnings.warn(f"CUDA graph capture of optimizer.step() failed, staying eager: {e}")
            self._graph, self._capture_failed = None, True
            for p, lg in zip(self._params, live):
                p.grad = lg

    def _swap_grads(self):
        for p, sg in zip(self._params, self._static_grads):
            if sg is None:
                continue
            if p.grad is not None and p.grad.data_ptr() != sg.data_ptr():
                sg.copy_(p.grad)
                p.grad = sg

    def invalidate(self):
        self._graph = None
        self._graph_age = 0

    def zero_grad(self, set_to_none: bool = False):
        # static gradient buffers must survive: zero in place while a graph is alive
        self.optimizer.zero_grad(set_to_none=set_to_none and self._graph is None)

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, sd):
        self.invalidate()
        return self.optimizer.load_state_dict(sd)
