"""SuperGrok v2 optimizer-step and bilevel-step latency on one GPU.

Config: the pre-LN bias-free decoder at d_model 256, 4 layers (3,174,144 parameters in 26 tensors), gradients drawn
from N(0, 1e-3) (seeded), meta-net defaults (d_model 8, d_inner 16, d_state 16, GRU 4, 4 heads, 144 experts of 1-16-1),
``bilevel_checkpoint_interval=32``.  Reports milliseconds per ``step()`` and per ``bilevel_step()`` (CUDA events, after
warm-up), for this package or for the reference installed under baseline/_ref (``--impl reference``).

    python -m supergrok15_b200.optim.bench_step [--impl reference] [--steps 20] [--scale medium|large]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn as nn


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--scale", default="medium", choices=["small", "medium", "large"])
    ap.add_argument("--no-bilevel", action="store_true")
    ap.add_argument("--kernels", action="store_true", help="also print the device time of every kernel of one step (torch.profiler)")
    ap.add_argument("--engine", default="none", choices=["none", "fp32", "bf16"],
                    help="run the step through ZeroEngine on this one GPU (world of one) with parameters of that dtype and fp32 masters: "
                         "the path of the data-parallel benchmark (gradient pull fused into the first kernel, device table of step scalars)")
    a = ap.parse_args()
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    from supergrok15_b200.models import MODEL_SCALES, PreLNTransformer
    sc = MODEL_SCALES[a.scale]
    dev = torch.device("cuda")
    torch.manual_seed(0)
    model = PreLNTransformer(sc["num_layers"], sc["dim_model"], sc["num_heads"], 99, 4).to(dev)
    if a.impl == "reference":
        import ctypes
        ref = os.path.join(root, "baseline", "_ref")
        sys.path.insert(0, ref)
        sys.modules.pop("grokking_optimizers", None)
        shim = os.path.join(ref, "libref_shim.so")
        if os.path.exists(shim):
            ctypes.CDLL(shim, mode=ctypes.RTLD_GLOBAL)
        try:
            import grokking_optimizers as go
            assert "baseline/_ref" in go.__file__.replace("\\", "/")
            opt = go.SuperGrok2(model.parameters(), bilevel_checkpoint_interval=32)
        except Exception as e:  # noqa: BLE001
            print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:200]}"}))
            return
    elif a.engine != "none":
        from supergrok15_b200.parallel import ZeroEngine
        dt = torch.float32 if a.engine == "fp32" else torch.bfloat16
        eng = ZeroEngine(model, "supergrok2", {}, param_dtype=dt, graph=False)
        ge = torch.Generator(device="cuda").manual_seed(1)

        def eng_step():
            eng.gbuf.tensor.copy_((torch.randn(eng.gbuf.tensor.shape, device=dev, generator=ge) * 1e-3).to(dt))
            eng.step()
        for _ in range(a.warmup):
            eng_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            eng_step()
        e1.record()
        torch.cuda.synchronize()
        n_params = sum(p.numel() for p in model.parameters())
        print(json.dumps({"impl": "ours", "engine": a.engine, "scale": a.scale, "params": n_params,
                          "step_ms_including_gradient_fill": e0.elapsed_time(e1) / a.steps}))
        return
    else:
        from supergrok15_b200.optim import SuperGrok2
        opt = SuperGrok2(model.parameters(), bilevel_checkpoint_interval=32)
    opt.meta_net.to(dev)
    g = torch.Generator(device="cuda").manual_seed(1)
    n_params = sum(p.numel() for p in model.parameters())

    def set_grads():
        for p in model.parameters():
            p.grad = torch.randn(p.shape, device=dev, generator=g) * 1e-3

    def timeit(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    set_grads()
    for _ in range(a.warmup):
        opt.step()
    step_ms = timeit(opt.step, a.steps)
    out = {"impl": a.impl, "scale": a.scale, "params": n_params, "tensors": len(list(model.parameters())), "step_ms": step_ms,
           "step_ms_per_1e9_params": step_ms * 1e9 / n_params}
    if a.kernels:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(3):
                opt.step()
            torch.cuda.synchronize()
        rows = sorted((e for e in prof.key_averages() if e.device_time_total > 0), key=lambda e: -e.device_time_total)
        tot = sum(e.device_time_total for e in rows)
        import re

        def short(name):                                   # "void ns::(anonymous namespace)::kernel<3>(args)" -> "kernel<3>"
            m = re.search(r"([A-Za-z_]\w*(?:<[^()]*>)?)\(", name.replace("(anonymous namespace)", ""))
            return (m.group(1) if m else name)[:48]
        out["kernels_us_per_step"] = [[short(e.key), round(e.device_time_total / 3, 1), e.count // 3,
                                       round(100 * e.device_time_total / tot, 1)] for e in rows[:12]]
    if not a.no_bilevel:
        x = torch.randint(0, 97, (512, 4), device=dev)
        y = torch.randint(0, 97, (512,), device=dev)
        crit = nn.CrossEntropyLoss()
        mopt = torch.optim.Adam(opt.meta_net.parameters(), lr=1e-4)

        def bilevel():
            set_grads()
            opt.bilevel_step(model, x, y, x, y, crit, mopt)
        try:
            for _ in range(2):
                bilevel()
            out["bilevel_ms"] = timeit(bilevel, max(3, a.steps // 4))
            if a.kernels:
                from torch.profiler import ProfilerActivity, profile
                with profile(activities=[ProfilerActivity.CUDA]) as prof:
                    bilevel()
                    torch.cuda.synchronize()
                rows = sorted((e for e in prof.key_averages() if e.device_time_total > 0), key=lambda e: -e.device_time_total)
                tot = sum(e.device_time_total for e in rows)
                out["bilevel_device_ms"] = round(tot / 1e3, 3)
                out["bilevel_kernels_us"] = [[e.key.replace("(anonymous namespace)::", "")[:56], round(e.device_time_total, 1), e.count,
                                              round(100 * e.device_time_total / tot, 1)] for e in rows[:16]]
        except Exception as e:  # noqa: BLE001
            out["bilevel_error"] = f"{type(e).__name__}: {str(e)[:200]}"
    print(json.dumps(out))


if __name__ == "__main__":
    main()
