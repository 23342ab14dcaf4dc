"""Muon step: momentum + per-matrix norm (multi-tensor kernel) and the Newton-Schulz chain.

The iteration is  X <- aX + b(XX^T)X + c(XX^T)^2 X  with (a,b,c) = (3.4445, -4.7750, 2.0315)
(reference csrc/ops.cpp:672-674, 713-727).  Since (XX^T)X = X(X^T X), a matrix with more rows
than columns is iterated in the algebraically equal right-Gram form  X <- X(aI + bG + cG^2),
G = X^T X, which needs cols^2 instead of rows^2 sized intermediates.  The reference always
uses the left form.
"""
from __future__ import annotations

from typing import List

import torch

from .. import _build
from . import elementwise as ew
from . import oracle

NS_COEFFS = oracle.NS_COEFFS


def newton_schulz_cuda(X: torch.Tensor, steps: int, precision: str = "bf16") -> torch.Tensor:
    """Newton-Schulz on the tcgen05 GEMM kernels.  X fp32 [r,c] (already normalised); returns fp32 [r,c]."""
    from . import gemm
    return gemm.newton_schulz(X, steps, NS_COEFFS, precision)


# Newton-Schulz chains captured as CUDA graphs, keyed by the momentum buffers they read: a step over 21 owned matrices is ~450
# short launches (15 GEMMs plus casts per matrix) that the host cannot issue as fast as the GPU runs them; replayed from a graph they
# are one launch.  The first call for a set of buffers runs eagerly (lazy initialisation), the second is captured.
_ns_graphs = {}


def _ns_all(bufs, inv, ns_steps, precision):
    return [newton_schulz_cuda(buf * inv[i], ns_steps, precision).contiguous() for i, buf in enumerate(bufs)]   # device scalar, no host sync


def _ns_graphed(bufs, inv, ns_steps, precision):
    import os
    if os.environ.get("SG_MUON_GRAPH", "1") == "0" or torch.cuda.is_current_stream_capturing():
        return _ns_all(bufs, inv, ns_steps, precision)
    key = (tuple((b.data_ptr(), tuple(b.shape)) for b in bufs), inv.data_ptr(), ns_steps, precision)
    ent = _ns_graphs.get(key)
    if ent is None:
        _ns_graphs[key] = "warm"
        return _ns_all(bufs, inv, ns_steps, precision)
    if ent == "warm":
        try:
            torch.cuda.synchronize(bufs[0].device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                xs = _ns_all(bufs, inv, ns_steps, precision)
            ent = _ns_graphs[key] = (g, xs)
        except Exception as exc:  # noqa: BLE001
            import warnings
            warnings.warn(f"CUDA graph capture of the Newton-Schulz chains failed ({type(exc).__name__}: {exc}); running eagerly")
            _ns_graphs[key] = ent = "eager"
    if ent == "eager":
        return _ns_all(bufs, inv, ns_steps, precision)
    ent[0].replay()
    return ent[1]


def muon_step(params: List[torch.Tensor], grads, bufs, lr: float, momentum: float, wd: float, ns_steps: int,
              precision: str = "bf16") -> None:
    if not params[0].is_cuda:
        return oracle.muon_(params, grads, bufs, lr, momentum, wd, ns_steps)
    C = _build.require()
    dev = params[0].device
    n = len(params)
    nb = C.mt_num_blocks([int(p.numel()) for p in params])
    partials = ew.workspace(dev, "partials", 3 * nb)
    pt = ew.workspace(dev, "pt_muon", 3 * n)
    C.mt_apply(C.ops["OP_MUON_MOMENTUM"], [[], grads, bufs], [], [0, 0, 0, 0, 0, momentum], partials=partials,
               per_tensor_out=pt)
    inv = ew.workspace(dev, "muon_inv", n)
    C.scalar_finalize(C.ops["SC_MUON_NORMS"], pt, n, inv, 0.0, 0.0, 0.0)
    xs = _ns_graphed(list(bufs), inv, ns_steps, precision)
    C.mt_apply(C.ops["OP_MUON_UPDATE"], [params, xs], [], [0, 0, 0, 0, 0, 0, 0, 0, -0.2 * lr, 1.0 - lr * wd])
