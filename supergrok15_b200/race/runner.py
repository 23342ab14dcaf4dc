"""Pipelines of the race: one (split, architecture, scale) cell = every optimizer x every seed; multi-GPU runs hand the
(optimizer, seed) jobs to one worker process per GPU through a queue (reference grokking_race_v2.py:1076-1356)."""
from __future__ import annotations

import copy
import json
import os
import subprocess
import time
import traceback
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import status
from .config import ALL_OPTIMIZERS, COMMON, DEFAULT_CONFIG, DISPLAY_NAMES, MODEL_LABELS, MODEL_SCALES, SEEDS, TRAIN_SPLITS, merged
from .data import make_data_for_task
from .train import OPTIMIZER_REGISTRY, TrainResult, get_init_state


def _git_hash() -> Optional[str]:
    try:
        return subprocess.check_output(["git", "rev-parse", "--short", "HEAD"], stderr=subprocess.DEVNULL, text=True,
                                       cwd=os.path.dirname(os.path.abspath(__file__))).strip()
    except Exception:  # noqa: BLE001
        return None


def _run_one(name, seed, base_cfg, device, progress=None) -> TrainResult:
    c = merged(base_cfg, name, {"seed": seed})
    tx, ty, vx, vy = (t.to(device) for t in make_data_for_task(c, seed))
    init = get_init_state(c, device)
    return OPTIMIZER_REGISTRY[name](c, init, tx, ty, vx, vy, device, 0, progress)


def _gpu_worker(gpu: int, tasks, results, base_cfg):
    """Worker process: owns one GPU, pulls (optimizer, seed) jobs until the poison pill."""
    dev = torch.device("cuda", gpu) if gpu >= 0 and torch.cuda.is_available() else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    while True:
        job = tasks.get()
        if job is None:
            break
        name, seed = job
        try:
            results.put((name, seed, _run_one(name, seed, base_cfg, dev), None))
        except Exception as e:  # noqa: BLE001
            results.put((name, seed, None, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-800:]}"))


def run_pipeline(base_cfg: Optional[dict] = None, optimizers: Sequence[str] = ALL_OPTIMIZERS, seeds: Sequence[int] = (42,),
                 device: str = "auto", gpus: Optional[List[int]] = None, save_dir: Optional[str] = "results", plot: bool = True,
                 verbose: bool = True, result_timeout: float = 7200.0, resume: bool = False) -> Dict[str, List[TrainResult]]:
    """``resume``: every finished (optimizer, seed) job is appended to ``<save_dir>/progress_<model>_ft<pct>.json`` as soon as it
    ends; a later call with ``resume=True`` and the same cell (model type, split) takes those results from the file and runs only
    the jobs that are missing (a race of 11 optimizers x 5 seeds x 20,000 steps that was interrupted does not start over)."""
    c = copy.deepcopy(DEFAULT_CONFIG)
    c.update(COMMON)
    c.update(base_cfg or {})
    t0 = time.time()
    tasks = [(n, s) for n in optimizers for s in seeds]
    rbo: Dict[str, List[TrainResult]] = {n: [] for n in optimizers}
    prog_path = os.path.join(save_dir, f"progress_{c.get('model_type', 'decoder')}_ft{int(c.get('frac_train', 0.5) * 100)}.json") if save_dir else None
    done: Dict[str, dict] = {}
    if resume and prog_path and os.path.exists(prog_path):
        with open(prog_path) as f:
            done = json.load(f)
        for n, s in tasks:
            if f"{n}/{s}" in done:
                rbo[n].append(TrainResult.from_dict(n, done[f"{n}/{s}"]))
        tasks = [(n, s) for n, s in tasks if f"{n}/{s}" not in done]
        if verbose:
            print(f"  resuming: {len(done)} finished jobs found in {prog_path}, {len(tasks)} to run", flush=True)
    elif prog_path and os.path.exists(prog_path):
        os.remove(prog_path)                                    # a fresh run does not inherit an older run's jobs

    def record(name, seed, res):
        if prog_path is None or res is None:
            return
        os.makedirs(save_dir, exist_ok=True)
        done[f"{name}/{seed}"] = res.to_dict()
        tmp = prog_path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(done, f)
        os.replace(tmp, prog_path)
    status.reset(len(tasks))
    multi = gpus is not None and len(gpus) > 1 and torch.cuda.is_available()
    if multi:
        import torch.multiprocessing as mp
        ctx = mp.get_context("spawn")
        tq, rq = ctx.Queue(), ctx.Queue()
        for t in tasks:
            tq.put(t)
        for _ in gpus:
            tq.put(None)
        procs = [ctx.Process(target=_gpu_worker, args=(g, tq, rq, c), daemon=True) for g in gpus]
        for p in procs:
            p.start()
        for _ in tasks:
            try:
                name, seed, res, err = rq.get(timeout=result_timeout)
            except Exception:  # noqa: BLE001
                status.job_done("?", -1, error="timed out waiting for a worker result")
                break
            if res is not None:
                rbo[name].append(res)
                record(name, seed, res)
            status.job_done(name, seed, {"grok": res.grokking_step} if res else None, err)
        for p in procs:
            p.join(60)
            if p.is_alive():
                p.terminate()
    else:
        if device == "auto":
            device = "cuda" if torch.cuda.is_available() else "cpu"
        dev = torch.device(device if gpus is None or not torch.cuda.is_available() else f"cuda:{gpus[0]}")
        for name, seed in tasks:
            try:
                res = _run_one(name, seed, c, dev, status.update)
                rbo[name].append(res)
                record(name, seed, res)
                status.job_done(name, seed, {"grok": res.grokking_step})
                if verbose:
                    print(f"  {DISPLAY_NAMES.get(name, name):<14} seed {seed:<5} steps {res.total_steps:>6} grok {res.grokking_step} "
                          f"val {res.final_val_acc:.3f} {res.step_ms:.2f} ms/step", flush=True)
            except Exception as e:  # noqa: BLE001
                status.job_done(name, seed, error=f"{type(e).__name__}: {e}")
                if verbose:
                    print(f"  {name} seed {seed} FAILED: {type(e).__name__}: {e}", flush=True)
    total = time.time() - t0
    rbo = {k: v for k, v in rbo.items() if v}
    if verbose:
        print_summary(rbo, total, c.get("model_type", "decoder"), c.get("frac_train", 0.5))
    if save_dir:
        save_json(rbo, save_dir, total, c.get("model_type", "decoder"), c.get("frac_train", 0.5), config=c)
        if plot:
            from .plots import plot_comparison
            plot_comparison(rbo, save_dir, f"_{c.get('model_type', 'decoder')}_ft{int(c.get('frac_train', 0.5) * 100)}")
    return rbo


def print_summary(rbo, total_wall=None, model_type="decoder", frac_train=0.5):
    w = 105
    print("\n" + "=" * w)
    print(f"  GROKKING RACE - {MODEL_LABELS.get(model_type, model_type)} | split={frac_train * 100:.0f}/{(1 - frac_train) * 100:.0f}")
    print("=" * w)
    ranked = sorted(rbo.items(), key=lambda kv: np.mean([r.grokking_wall or 1e9 for r in kv[1]]))
    print(f"  {'#':>2} {'Optimizer':<14} {'Grok Wall (s)':>14} {'Grok Steps':>12} {'Total Steps':>12} {'Val Acc':>9} {'Status':>8} {'Seeds':>6}")
    print("  " + "-" * (w - 2))
    medals = ["1.", "2.", "3."] + ["  "] * 20
    for rank, (name, runs) in enumerate(ranked):
        gw = [r.grokking_wall or r.wall_time for r in runs]
        nogrok = any(r.grokking_wall is None for r in runs)
        print(f"  {medals[rank]} {DISPLAY_NAMES.get(name, name):<14} {np.mean(gw):>14.2f} "
              f"{np.mean([r.grokking_step or r.total_steps for r in runs]):>12,.0f} {np.mean([r.total_steps for r in runs]):>12,.0f} "
              f"{np.mean([r.final_val_acc for r in runs]):>9.4f} {'DNF' if nogrok else 'GROK':>8} {len(runs):>6}")
    print("  " + "-" * (w - 2))
    if total_wall:
        print(f"  Pipeline wall: {total_wall:.1f}s")
    print("=" * w)


def save_json(rbo, save_dir="results", total_wall=None, model_type="decoder", frac_train=0.5, config=None):
    """Reference schema (``_meta`` + one list of runs per optimizer) with the config, seeds and git hash added to ``_meta``."""
    os.makedirs(save_dir, exist_ok=True)
    d = {"_meta": {"total_wall": total_wall, "model_type": model_type, "frac_train": frac_train, "git": _git_hash(),
                   "config": {k: v for k, v in (config or {}).items() if isinstance(v, (int, float, str, bool, type(None)))}}}
    for name, runs in rbo.items():
        d[name] = [r.to_dict() for r in runs]
    path = os.path.join(save_dir, f"results_{model_type}_ft{int(frac_train * 100)}.json")
    with open(path, "w") as f:
        json.dump(d, f, indent=2)
    return path


def _grok_table(cells: Dict) -> Dict[str, Dict[str, float]]:
    """{row label: {optimizer: mean steps to grok (total steps when a run did not grok)}}."""
    return {str(k): {n: float(np.mean([r.grokking_step or r.total_steps for r in runs])) for n, runs in rbo.items()} for k, rbo in cells.items()}


def run_multi_split(base_cfg=None, splits=TRAIN_SPLITS, **kw):
    out = {}
    for ft in splits:
        c = dict(base_cfg or {}, frac_train=ft)
        out[ft] = run_pipeline(c, **kw)
    if kw.get("save_dir") and kw.get("plot", True):
        from .plots import plot_grouped_bars
        plot_grouped_bars(_grok_table({f"{int(ft * 100)}% train": r for ft, r in out.items()}), "steps to grok by train split",
                          os.path.join(kw["save_dir"], "split_comparison.png"))
    return out


def run_architecture_comparison(base_cfg=None, archs=("decoder", "vit", "mamba"), **kw):
    out = {a: run_pipeline(dict(base_cfg or {}, model_type=a), **kw) for a in archs}
    if kw.get("save_dir") and kw.get("plot", True):
        from .plots import plot_grouped_bars
        plot_grouped_bars(_grok_table({MODEL_LABELS.get(a, a): r for a, r in out.items()}), "steps to grok by architecture",
                          os.path.join(kw["save_dir"], "architecture_comparison.png"))
    return out


def run_scale_comparison(base_cfg=None, scales=("small", "medium", "large"), **kw):
    return {s: run_pipeline(dict(base_cfg or {}, **MODEL_SCALES[s]), save_dir=os.path.join(kw.pop("save_dir", "results") or "results", s), **kw)
            for s in scales}


def run_full_sweep(base_cfg=None, archs=("decoder", "vit", "mamba"), splits=TRAIN_SPLITS, **kw):
    """Every architecture x every train split x every optimizer x every seed; also writes the sweep heat map."""
    table = {}
    save_dir = kw.get("save_dir", "results") or "results"
    for a in archs:
        for ft in splits:
            rbo = run_pipeline(dict(base_cfg or {}, model_type=a, frac_train=ft), **kw)
            for name, runs in rbo.items():
                table.setdefault(name, {})[f"{a}@{int(ft * 100)}"] = float(np.mean([r.grokking_step or r.total_steps for r in runs]))
    from .plots import plot_heatmap
    plot_heatmap(table, "steps to grok", os.path.join(save_dir, "full_sweep.png"))
    with open(os.path.join(save_dir, "full_sweep.json"), "w") as f:
        json.dump(table, f, indent=2)
    return table


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="Grokking race driver")
    ap.add_argument("--setup", action="store_true", help="check the environment (no network install is attempted)")
    ap.add_argument("--ntfy", default=None, help="ntfy.sh topic for notifications (optional)")
    ap.add_argument("--port", type=int, default=8765, help="port of the /status HTTP server")
    ap.add_argument("--no-status-server", action="store_true")
    ap.add_argument("--gpus", default="auto", help='"auto" or a comma-separated list of GPU ids')
    ap.add_argument("--mode", default="A", choices=list("ABCDE"),
                    help="A single pipeline, B multi-split, C architectures, D full sweep, E model scales")
    ap.add_argument("--optimizers", default="all")
    ap.add_argument("--seeds", default="42")
    ap.add_argument("--model-scale", default="small", choices=list(MODEL_SCALES))
    ap.add_argument("--model-type", default="decoder", choices=["decoder", "decoder_preln", "vit", "mamba"])
    ap.add_argument("--task", default="division", choices=["division", "addition"])
    ap.add_argument("--frac-train", type=float, default=0.5)
    ap.add_argument("--max-steps", type=int, default=20_000)
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16", "fp16"])
    ap.add_argument("--reference-compat", action="store_true", help="reproduce the reference's SAM / bias-correction / amplifier quirks")
    ap.add_argument("--cuda-graph", action="store_true")
    ap.add_argument("--compile-model", action="store_true", help="wrap the model in torch.compile (reference grokking_race_v2.py:432-443); off by default")
    ap.add_argument("--save-dir", default="results")
    ap.add_argument("--resume", action="store_true", help="skip the (optimizer, seed) jobs already recorded in the save directory's progress file")
    a = ap.parse_args(argv)
    if a.setup:
        from .. import _build
        print("torch", torch.__version__, "cuda", torch.cuda.is_available(), "native extension", _build.native_available())
        return 0
    if a.gpus == "auto":
        gpus = list(range(torch.cuda.device_count())) if torch.cuda.is_available() else None
    else:
        gpus = [int(g) for g in a.gpus.split(",") if g != ""]
    opts = list(ALL_OPTIMIZERS) if a.optimizers == "all" else [o.strip() for o in a.optimizers.split(",")]
    seeds = SEEDS if a.seeds == "all" else [int(s) for s in a.seeds.split(",")]
    base = dict(MODEL_SCALES[a.model_scale], model_type=a.model_type, task=a.task, frac_train=a.frac_train, max_steps=a.max_steps,
                use_amp=a.dtype != "fp32", amp_dtype=a.dtype, reference_compat=a.reference_compat, use_cuda_graph=a.cuda_graph, compile_model=a.compile_model)
    if not a.no_status_server:
        try:
            status.start_status_server(a.port)
        except OSError:
            pass
    status.start_ntfy_listener(a.ntfy)
    status.ntfy(a.ntfy, f"race started: mode {a.mode}, {len(opts)} optimizers, {len(seeds)} seeds")
    kw = dict(optimizers=opts, seeds=seeds, gpus=gpus if gpus and len(gpus) > 1 else None, save_dir=a.save_dir, resume=a.resume)
    if a.mode == "A":
        run_pipeline(base, **kw)
    elif a.mode == "B":
        run_multi_split(base, **kw)
    elif a.mode == "C":
        run_architecture_comparison(base, **kw)
    elif a.mode == "D":
        run_full_sweep(base, **kw)
    else:
        run_scale_comparison(base, **kw)
    status.ntfy(a.ntfy, "race finished")
    return 0
