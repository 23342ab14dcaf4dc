"""Sharded optimizer-step sweep: every optimizer's ZeRO step (gradient reduce-scatter + step + parameter all-gather)
on a flat fp32 model of square tensors, reported as milliseconds per 10^9 parameters.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m supergrok15_b200.parallel.bench_sweep \
        --params 1e9 --steps 5 --warmup 3 [--optimizers lion,adamw,...] [--comm p2p|nccl]

Model: tensors of shape 4096x4096, the last one trimmed so the total is exactly ``--params``.  Gradients are N(0, 1e-3)
with 1 % of the entries scaled by 100 (seeded per rank), written straight into the engine's gradient buffer.
Timing: CUDA events around ``engine.step()``, max over ranks, after warm-up; one JSON line per optimizer on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn as nn

ALL = ["lion", "grokfast", "grokadamw", "prodigy", "looksam", "neuralgrok", "supergrok11", "supergrok15", "supergrok2", "muon", "adamw"]


class FlatModel(nn.Module):
    def __init__(self, total: int, side: int = 4096, dtype=torch.float32, device="cuda"):
        super().__init__()
        per = side * side
        n_full, rem = divmod(total, per)
        shapes = [(side, side)] * n_full
        if rem:
            rows = rem // side
            if rows:
                shapes.append((rows, side))
        self.ws = nn.ParameterList([nn.Parameter(torch.empty(s, dtype=dtype, device=device).normal_(0, 0.02)) for s in shapes])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=float, default=1e9)
    ap.add_argument("--side", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--optimizers", default="all")
    ap.add_argument("--comm", default="p2p")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--muon-sharding", default="tensors", choices=["tensors", "rows"])
    ap.add_argument("--pg-timeout", type=int, default=180, help="seconds before a stuck NCCL bootstrap collective aborts the job")
    ap.add_argument("--progress-dir", dest="log", default=None, help="directory for per-rank progress logs")
    a = ap.parse_args()
    import torch.distributed as dist
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=a.pg_timeout))
    from supergrok15_b200.parallel import ZeroEngine
    dt = torch.float32 if a.dtype == "fp32" else torch.bfloat16
    names = ALL if a.optimizers == "all" else a.optimizers.split(",")
    logf = open(os.path.join(a.log, f"sweep_rank{rank}.log"), "w") if a.log else None

    def note(msg):
        if logf:
            logf.write(msg + "\n")
            logf.flush()

    for name in names:
        note(f"begin {name}")
        torch.manual_seed(0)
        model = FlatModel(int(a.params), a.side, dt)
        n_params = sum(p.numel() for p in model.parameters())
        kw = {}
        if name in ("supergrok2", "supergrok15", "supergrok11"):
            kw = dict(warmup_steps=0, warmup_ramp=1)
        if name == "muon":
            kw = dict(sharding=a.muon_sharding)
        try:
            eng = ZeroEngine(model, name, kw, comm=a.comm, param_dtype=dt)
            g = torch.Generator(device="cuda").manual_seed(1234 + rank)
            gb = eng.gbuf.tensor
            gb.normal_(0, 1e-3, generator=g)
            mask = torch.rand(gb.shape, device="cuda", generator=g) < 0.01
            gb[mask] *= 100.0
            del mask
            note("  engine built")
            for _ in range(a.warmup):
                eng.step()
            torch.cuda.synchronize()
            eng.check()
            note("  warm-up done")
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.steps):
                eng.step()
            e1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device="cuda")
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            eng.check()
            ok = all(bool(torch.isfinite(p).all()) for p in eng.params[:2])
            nv = eng.nvlink_bytes_per_step()
            if rank == 0:
                print(json.dumps({"optimizer": name, "n_gpus": world, "params": n_params, "ms_per_step": float(ms),
                                  "ms_per_1e9_params": float(ms) * 1e9 / n_params, "comm": eng.comm, "dtype": a.dtype, "finite": ok,
                                  "nvlink_bytes_per_direction_per_rank": nv["per_direction"],
                                  "nvlink_floor_ms": nv["per_direction"] / 770e9 * 1e3,
                                  "nvlink_fraction": (nv["per_direction"] / 770e9 * 1e3) / float(ms) if float(ms) > 0 else None}), flush=True)
        except Exception as e:  # noqa: BLE001
            note(f"  FAILED {type(e).__name__}: {str(e)[:300]}")
            if rank == 0:
                print(json.dumps({"optimizer": name, "n_gpus": world, "error": f"{type(e).__name__}: {str(e)[:300]}"}), flush=True)
        del model
        eng = None
        torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
