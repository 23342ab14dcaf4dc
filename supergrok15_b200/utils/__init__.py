"""Timers, NVTX ranges and roofline bookkeeping."""
from .roofline import fraction, peaks
from .timers import StepTimer, nvtx

__all__ = ["StepTimer", "nvtx", "fraction", "peaks"]
