#!/usr/bin/env python
"""Headline benchmark: train tokens/s of ZeRO-2 SuperGrok v2 on the modular-division transformer.

Config (the ZeRO-2 configuration of the baseline spec): modular division mod 113, all pairs with b != 0,
30 % train split; 6-layer post-LN decoder, d_model 512, 8 heads, MLP 2048, sequence length 4; bf16 model
with fp32 master weights; global batch 8192 sequences, split evenly over the ranks (strong scaling);
one step = forward + backward + gradient reduce-scatter + SuperGrok v2 step + parameter all-gather.
Inputs are synthetic: batches are drawn (seeded) from the 3,797-row train split; weights are random-init.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...             # the reference from baseline/_ref (own model,
                                                              # own optimizer, DistributedDataParallel for N>1)

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with inputs resident
on the device; ``e2e`` times the public call ``ZeroEngine.train_step`` on pinned host batches, including the
host-to-device copy and the device-to-host read of the loss every step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

P_MOD, FRAC_TRAIN, SEQ = 113, 0.3, 4
NL, D, H = 6, 512, 8
GLOBAL_BATCH = 8192
NTOK = P_MOD + 2
BASELINE_VALUE = None          # the reference publishes no throughput number
# identical in both arms; what differs between the arms is reported under "arm"
CONFIG = {"model": "6-layer post-LN decoder d512 h8 mlp2048 (19.0M params)", "global_batch": GLOBAL_BATCH, "seq_len": SEQ,
          "l2": "per-step working set (optimizer state + sort/scan workspace, > 1 GB per rank) exceeds the 126 MB L2"}


def dist_setup(n):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def make_division_data(p, frac, seed):
    """All (a, b != 0) pairs of a / b mod p as [a, p, b, p+1]; python-random shuffle; int(len*frac) train rows."""
    import random
    import torch
    rng = random.Random(seed)
    rows = []
    for a in range(p):
        for b in range(1, p):
            rows.append(([a, p, b, p + 1], (a * pow(b, p - 2, p)) % p))
    rng.shuffle(rows)
    n = int(len(rows) * frac)
    x = torch.tensor([r[0] for r in rows], dtype=torch.long)
    y = torch.tensor([r[1] for r in rows], dtype=torch.long)
    return x[:n], y[:n], x[n:], y[n:]


def batches(tx, ty, n_steps, per_rank, rank, seed):
    """Seeded synthetic batches: each step draws per_rank rows (with replacement) from the train split."""
    import torch
    g = torch.Generator().manual_seed(seed * 1000 + rank)
    out = []
    for _ in range(n_steps):
        idx = torch.randint(0, tx.shape[0], (per_rank,), generator=g)
        out.append((tx[idx].pin_memory(), ty[idx].pin_memory()))
    return out


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi (rank 0 only).  The query loop is started before the warm-up steps so
    that it is in steady state when the timed region begins; only samples that arrived between ``mark_begin()`` and ``stop()``
    (the device-timed loop and the end-to-end loop) are reported."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0, period_ms=100):
        self.proc, self.lines, self.gpu, self.period_ms, self.t0 = None, [], gpu_index, period_ms, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def mark_begin(self):
        self.t0 = time.monotonic()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t1 = time.monotonic()
        time.sleep(0.25)                                   # a query that started under load may still be printing
        self.proc.terminate()
        t0 = self.t0 if self.t0 is not None else 0.0
        sm, mx, reasons = [], [], set()
        for t, l in self.lines:
            if t < t0 or t > t1 + 0.25:
                continue
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "window_s": round(t1 - t0, 3)}


def timed_loop(step_fn, K, world):
    """barrier + sync, K steps between CUDA events, sync + barrier; returns max-over-ranks ms per step."""
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        step_fn(i)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.barrier()
    return float(ms.item()) / K


def wall_loop(step_fn, K, world):
    import torch
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(K):
        step_fn(i)
    torch.cuda.synchronize()
    dt = torch.tensor([time.perf_counter() - t0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        dist.barrier()
    return float(dt.item()) * 1e3 / K


# ------------------------------------------------------------------------------------------------ this framework
def correctness_probe(rank, world, local, comm):
    """Sharded == unsharded on a small fp32 problem at this world size (outside every timed region): two steps of the engine
    (one rank per GPU, in-kernel collectives, each rank a slice of a 64-row batch) against two steps of the plain
    optimizer on the whole batch in one process.  Returns the largest absolute parameter difference and whether every rank
    ends with bitwise identical parameters."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from supergrok15_b200 import optim as O
    from supergrok15_b200.models import Transformer
    from supergrok15_b200.parallel import ZeroEngine
    dev = torch.device("cuda", local)
    kw = dict(warmup_steps=0, warmup_ramp=1, eps=1e-3)

    def problem():
        torch.manual_seed(0)
        m = Transformer(1, 32, 2).to(dev)
        g = torch.Generator().manual_seed(5)
        return m, torch.randint(0, 97, (64, 4), generator=g).to(dev), torch.randint(0, 97, (64,), generator=g).to(dev)
    m, x, y = problem()
    eng = ZeroEngine(m, "supergrok2", kw, comm=comm, param_dtype=torch.float32, graph=False)
    per = 64 // world
    for _ in range(2):
        eng.train_step(x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per])
    eng.check()
    flat = torch.cat([p.detach().float().reshape(-1) for p in eng.params])
    m2, x2, y2 = problem()
    opt = O.SuperGrok2(m2.parameters(), **kw)
    for _ in range(2):
        opt.zero_grad()
        F.cross_entropy(m2(x2), y2).backward()
        opt.step()
    ref = torch.cat([p.detach().float().reshape(-1) for p in m2.parameters()])
    diff = (flat - ref).abs().max()
    lo, hi = flat.clone(), flat.clone()
    if world > 1:
        dist.all_reduce(diff, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return {"what": "2 steps of ZeRO SuperGrok v2 on a 1-layer d32 fp32 decoder, 64 rows split over the ranks, vs the unsharded "
                    "optimizer on the whole batch in one process", "max_abs_param_diff": float(diff),
            "ref_abs_max": float(ref.abs().max()), "replicas_bitwise_equal": bool(torch.equal(lo, hi))}


def median(v):
    v = sorted(v)
    return v[len(v) // 2]


def phase_times(eng, batch, world, n=3):
    """Per-phase device times of a step (CUDA events, median of n eager steps, max over ranks)."""
    import torch
    import torch.distributed as dist
    runs = [eng.profile_step(*batch) for _ in range(n)]
    keys = list(runs[0])
    t = torch.tensor([median([r[k] for r in runs]) for k in keys], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {k: round(v, 4) for k, v in zip(keys, t.tolist())}


def run_ours(args, rank, world, local):
    import torch
    from supergrok15_b200 import _build
    from supergrok15_b200.models import Transformer
    from supergrok15_b200.parallel import ZeroEngine
    _build.require()
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    model = Transformer(NL, D, H, NTOK, SEQ).to(dev)
    eng = ZeroEngine(model, "supergrok2", dict(lr=1e-3, betas=(0.9, 0.98), weight_decay=1.0), comm=args.comm,
                     param_dtype=torch.bfloat16)
    tx, ty, _, _ = make_division_data(P_MOD, FRAC_TRAIN, 0)
    per_rank = GLOBAL_BATCH // world
    W, K = args.warmup, args.steps
    host = batches(tx, ty, W + 2 * K, per_rank, rank, 1)
    dev_batches = [(x.to(dev), y.to(dev)) for x, y in host[:W + K]]
    # steps before the W warm-up steps: lazy initialisation and the capture of the forward/backward CUDA graph (the engine runs
    # its first calls of a batch shape eagerly, then captures), so that neither falls into the warm-up or the timed region
    for i in range(eng.graph_warmup + 2):
        eng.train_step(*dev_batches[i % len(dev_batches)])
    try:                                             # diagnostics never take the measurement down with them
        probe = correctness_probe(rank, world, local, args.comm)
    except Exception as e:  # noqa: BLE001
        probe = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()                                  # query loop up and running before the warm-up ends
    for i in range(W):
        eng.train_step(*dev_batches[i])
    eng.check()
    C = _build.require()
    R = max(1, args.repeats)
    sampler.mark_begin()
    l0 = C.launch_count()
    ms_runs = [timed_loop(lambda i: eng.train_step(*dev_batches[W + i]), K, world) for _ in range(R)]
    launches_region = (C.launch_count() - l0) // R    # kernels of this package enqueued inside one timed region of K steps
    ms = median(ms_runs)
    losses = []

    def e2e_step(i):
        x, y = host[W + K + i]
        losses.append(float(eng.train_step(x, y).item()))       # H2D of the batch, D2H of the loss, every step
    e2e_ms = median([wall_loop(e2e_step, K, world) for _ in range(R)])
    clocks = sampler.stop() if rank == 0 else None
    eng.check()
    try:
        phases = phase_times(eng, dev_batches[W], world)
        eng.check()
    except Exception as e:  # noqa: BLE001
        phases = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
    # every rank must hold bitwise identical bf16 parameters after the run (the all-gather is part of the step)
    import torch.distributed as dist
    pb = eng.pbuf.tensor.view(torch.int16).to(torch.int32)
    lo, hi = pb.clone(), pb.clone()
    if world > 1:
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    probe["flagship_replicas_bitwise_equal"] = bool(torch.equal(lo, hi))
    tokens = GLOBAL_BATCH * SEQ
    # roofline of the two phases that cross NVLink: each rank pulls its tensors' gradients from W-1 peers and pushes its updated
    # parameters to W-1 peers; every link direction carries both one rank's pulls and another rank's pushes
    from supergrok15_b200.utils import roofline
    link_bytes = 2 * (world - 1) * eng.n_own * 2
    fr = {}
    if world > 1 and "error" not in phases:
        fr["reduce+prep"] = roofline.fraction(phases.get("reduce+prep", 0.0), nvlink_bytes=link_bytes / 2, hbm_bytes=eng.n_own * 22)
        fr["elem+push"] = roofline.fraction(phases.get("elem+push", 0.0), nvlink_bytes=link_bytes / 2, hbm_bytes=eng.n_own * 130)
    return {
        "metric": "train tokens/s (max over ranks), ZeRO-2 SuperGrok v2", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": (tokens / (ms * 1e-3) / BASELINE_VALUE) if BASELINE_VALUE else None, "dtype": "bf16",
        "data": "synthetic: seeded batches drawn from the mod-113 division train split; random-init weights",
        "config": dict(CONFIG, parallelism=f"dp{world}"),
        "arm": {"parallelism": f"zero2-dp{world}", "optimizer": "SuperGrok v2 (fp32 master, bf16 model)", "comm": eng.comm,
                "whole_step_cuda_graph": bool(eng.use_graph and eng.device_step)},
        "repeats": R, "ms_per_step_runs": [round(m, 4) for m in ms_runs],
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": per_rank * SEQ * 8 + per_rank * 8, "d2h_bytes_per_step": 4,
                "api": "supergrok15_b200.parallel.ZeroEngine.train_step(pinned_x, pinned_y).item()"},
        "gpu_launches": launches_region, "phases_ms": phases, "phase_roofline": fr, "correctness": probe,
        "final_loss": losses[-1] if losses else None, "impl": "ours",
    }


# ------------------------------------------------------------------------------------------------ Muon on the Llama-style 1.3B model
def run_llama_muon(args, rank, world, local):
    """Secondary benchmark (``--config llama_muon``): Llama-style 1.3 B decoder, bf16, sequence 2048, global batch 256 sequences,
    Muon (5 Newton-Schulz iterations on the tcgen05 GEMM) for the block matrices, AdamW for embedding / head / norms, ZeRO-sharded."""
    import torch
    from supergrok15_b200 import _build
    from supergrok15_b200.models import LLAMA_1P3B, Llama, LlamaConfig
    from supergrok15_b200.parallel import ZeroEngine
    C = _build.require()
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    cfg = LLAMA_1P3B if not args.small else LlamaConfig(n_layers=4, d_model=1024, n_heads=8, d_ff=2752, vocab=32000, max_seq=2048)
    with torch.device(dev):
        model = Llama(cfg).to(torch.bfloat16)
    eng = ZeroEngine(model, "muon", dict(lr=0.02, momentum=0.95, weight_decay=0.01, adamw_lr=1e-3, adamw_names=("embed", "lm_head"),
                                         sharding=args.muon_sharding),
                     comm=args.comm, param_dtype=torch.bfloat16, graph=False)     # GPU-bound step: nothing to gain from a graph
    seq, gb = 2048, args.global_batch or 256
    per_rank = gb // world
    micro = max(1, per_rank // args.micro_seqs)
    g = torch.Generator().manual_seed(100 + rank)
    W, K = args.warmup, args.steps
    host = [(torch.randint(0, cfg.vocab, (per_rank, seq), generator=g).pin_memory(),) for _ in range(W + K)]

    def step(i):
        ids = host[i][0].to(dev, non_blocking=True)
        return eng.train_step(ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), micro_batches=micro)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(W):
        step(i)
    eng.check()
    l0 = C.launch_count()
    sampler.mark_begin()
    losses = []
    ms = timed_loop(lambda i: losses.append(step(W + i)), K, world)
    clocks = sampler.stop() if rank == 0 else None
    eng.check()
    opt_ms = timed_loop(lambda i: eng.step(), 5, world)       # the sharded optimizer step alone (reduce-scatter, Muon / AdamW, all-gather)
    eng.check()
    from supergrok15_b200.ops import gemm as _g
    _g.check(dev)
    tokens = gb * seq
    n_params = sum(p.numel() for p in model.parameters())
    return {"metric": "train tokens/s (max over ranks), Muon on Llama-style decoder", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: uniform-random token ids; random-init weights",
            "config": {"model": f"llama {cfg.n_layers}L d{cfg.d_model} h{cfg.n_heads} ff{cfg.d_ff} vocab{cfg.vocab} ({n_params / 1e9:.3f}B params)",
                       "global_batch": gb, "seq_len": seq, "parallelism": f"zero2-dp{world}, Muon matrices " + ("split by rows over the ranks (collectives inside the Newton-Schulz GEMMs)"
                                                                          if getattr(eng, "rs_idx", None) else "owned whole by one rank each"),
                       "row_sharded_matrices": len(getattr(eng, "rs_idx", []) or []),
                       "micro_batches": micro, "l2": "inputs and weights far exceed the 126 MB L2"},
            "clocks": clocks, "gpu_launches": C.launch_count() - l0, "final_loss": float(losses[-1]) if losses else None,
            "model_flops_per_step": 6.0 * n_params * tokens, "impl": "ours", "optimizer_step_ms": opt_ms,
            "optimizer_step_ms_per_1e9_params": opt_ms * 1e9 / n_params,
            "h2d_bytes_per_step": per_rank * seq * 8}


# ------------------------------------------------------------------------------------------------ reference arm
def run_reference(args, rank, world, local):
    """The unmodified reference: its own Transformer (grokking_race_v2.py:321-331), its own SuperGrok2 optimizer through
    grokking_optimizers (stock batched CUDA path), bf16 autocast over fp32 parameters, DDP over NCCL when N > 1."""
    import types
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "grokking_optimizers")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref of the reference)"}
    sys.path.insert(0, ref_dir)
    sys.modules.pop("grokking_optimizers", None)
    for name in ("matplotlib", "matplotlib.pyplot"):            # the driver imports matplotlib at module level for its plots
        try:
            __import__(name)
        except Exception:  # noqa: BLE001
            m = types.ModuleType(name)
            m.use = lambda *a, **k: None
            sys.modules[name] = m
    import ctypes
    import torch
    import torch.nn.functional as F
    try:
        shim = os.path.join(ref_dir, "libref_shim.so")       # one PyTorch symbol the reference needs (baseline/ref_shim.cpp)
        if os.path.exists(shim):
            ctypes.CDLL(shim, mode=ctypes.RTLD_GLOBAL)
        import grokking_optimizers as go
        import grokking_race_v2 as ref
    except Exception as e:  # noqa: BLE001
        return {"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {str(e)[:160]}"}
    if "baseline/_ref" not in os.path.abspath(go.__file__).replace("\\", "/"):
        return {"impl": "reference", "unavailable": "grokking_optimizers resolved outside baseline/_ref"}
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    model = ref.Transformer(NL, D, H, NTOK, SEQ).to(dev)
    opt = go.SuperGrok2(model.parameters(), lr=1e-3, betas=(0.9, 0.98), weight_decay=1.0)
    opt.meta_net.to(dev)
    fwd = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        fwd = DDP(model, device_ids=[local])
    tx, ty, _, _ = ref.make_data(P_MOD, FRAC_TRAIN, 0)
    per_rank = GLOBAL_BATCH // world
    W, K = args.warmup, args.steps
    host = batches(tx, ty, W + 2 * K, per_rank, rank, 1)
    dev_batches = [(x.to(dev), y.to(dev)) for x, y in host[:W + K]]

    def train_step(x, y):
        if x.device != dev:
            x, y = x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = F.cross_entropy(fwd(x).float(), y)
        loss.backward()
        opt.step()
        return loss.detach()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(W):
        train_step(*dev_batches[i])
    sampler.mark_begin()
    ms = timed_loop(lambda i: train_step(*dev_batches[W + i]), K, world)
    losses = []
    e2e_ms = wall_loop(lambda i: losses.append(float(train_step(*host[W + K + i]).item())), K, world)
    clocks = sampler.stop() if rank == 0 else None
    tokens = GLOBAL_BATCH * SEQ
    return {
        "metric": "train tokens/s (max over ranks), ZeRO-2 SuperGrok v2", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded batches drawn from the mod-113 division train split; random-init weights",
        "config": dict(CONFIG, parallelism=f"dp{world}"),
        "arm": {"parallelism": f"ddp{world} (the reference has no sharding; replicated optimizer)",
                "optimizer": "reference SuperGrok2, fp32 parameters, bf16 autocast"},
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": per_rank * SEQ * 8 + per_rank * 8, "d2h_bytes_per_step": 4},
        "gpu_launches": None, "final_loss": losses[-1] if losses else None, "impl": "reference",
        "build_note": "built from an unmodified source copy; only the copy's setup.py changed (GPU check dropped, gencode sm_100)",
    }


def main():
    import faulthandler
    faulthandler.enable()                            # a fatal signal in any rank leaves the Python stack of every thread in the log
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="the K-step timed loop is run this many times; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default=None, choices=[None, "p2p", "nvls", "nccl"])
    ap.add_argument("--config", default="zero2_sg2", choices=["zero2_sg2", "llama_muon"])
    ap.add_argument("--small", action="store_true", help="llama_muon: 4-layer d1024 model for quick checks")
    ap.add_argument("--global-batch", type=int, default=0)
    ap.add_argument("--micro-seqs", type=int, default=4, help="llama_muon: sequences per micro-batch")
    ap.add_argument("--muon-sharding", default="tensors", choices=["tensors", "rows"],
                    help="llama_muon: whole matrices per rank, or rows of every matrix over the ranks (fused collectives in the NS GEMMs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    import torch
    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device in this process"}))
            return
        raise SystemExit("bench.py needs a CUDA device")
    rank, world, local = dist_setup(args.gpus)
    try:
        if args.config == "llama_muon":
            res = ({"impl": "reference", "unavailable": "the reference ships no Llama model and no data-parallel Muon"} if args.impl == "reference"
                   else run_llama_muon(args, rank, world, local))
        else:
            res = run_reference(args, rank, world, local) if args.impl == "reference" else run_ours(args, rank, world, local)
    except Exception as e:  # noqa: BLE001
        if args.impl == "reference":
            res = {"impl": "reference", "unavailable": f"reference run failed: {type(e).__name__}: {str(e)[:200]}"}
        else:
            raise
    if rank == 0:
        print(json.dumps(res), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        # Nobody leaves while another rank still computes or prints; then every rank ends WITHOUT interpreter finalisation.
        # At interpreter exit the destructors of CUDA graphs, side streams, peer mappings and NCCL communicators run in no
        # defined order across the processes: one of four 8-GPU runs lost a rank to SIGSEGV there, after its work was done, and
        # the launcher then killed rank 0 before it had printed its line.  The driver frees everything when the process ends.
        import torch.distributed as dist
        try:
            torch.cuda.synchronize()
            dist.barrier()
        except Exception:  # noqa: BLE001
            pass
        os._exit(0)


if __name__ == "__main__":
    main()
