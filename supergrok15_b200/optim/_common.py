"""Shared helpers of the optimizers: closure handling, fp32 state creation, reference-compat switch."""
from __future__ import annotations

from typing import Callable, Optional

import torch


def run_closure(closure: Optional[Callable]):
    if closure is None:
        return None
    with torch.enable_grad():
        return closure()


def zeros_state(p: torch.Tensor) -> torch.Tensor:
    """fp32 state shaped like the parameter (state is fp32 for every parameter dtype)."""
    return torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
