"""Roofline bookkeeping against MEASURED peaks (``MEASURED_PEAKS.json`` at the repository root when present, otherwise
the fallback figures 6.65 TB/s and 1.59 PFLOP/s) and the measured NVLink references (770 GB/s peer copy per direction)."""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NVLINK_GBS_PER_DIRECTION = 770.0


def peaks(path: Optional[str] = None) -> Dict[str, float]:
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    except Exception:  # noqa: BLE001
        return dict(FALLBACK)


def fraction(ms: float, *, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0, sustained: bool = False,
             pk: Optional[Dict[str, float]] = None) -> Dict[str, float]:
    """Achieved fraction of the roofline: target time = max(FLOPs / GEMM peak, HBM bytes / copy bandwidth,
    NVLink bytes per direction / link bandwidth); fraction = target / measured."""
    pk = pk or peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    t_c = flops / tf if flops else 0.0
    t_m = hbm_bytes / (pk["hbm_gbs"] * 1e9) if hbm_bytes else 0.0
    t_l = nvlink_bytes / (NVLINK_GBS_PER_DIRECTION * 1e9) if nvlink_bytes else 0.0
    target = max(t_c, t_m, t_l)
    bound = "compute" if target == t_c else ("hbm" if target == t_m else "nvlink")
    return {"target_ms": target * 1e3, "measured_ms": ms, "fraction": (target * 1e3 / ms) if ms > 0 else 0.0, "bound": bound,
            "peaks": pk["source"]}
