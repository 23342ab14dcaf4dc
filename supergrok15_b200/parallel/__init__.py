"""ZeRO-sharded data parallelism with in-kernel collectives over NVLink / NVSwitch."""
from .engine import CommTimeout, ZeroEngine
from .ownership import assign_tensors, flat_ranges, grouped_layout, imbalance

__all__ = ["CommTimeout", "ZeroEngine", "assign_tensors", "flat_ranges", "grouped_layout", "imbalance"]
