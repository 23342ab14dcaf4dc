#!/usr/bin/env python
"""Steps-to-grok parity: the reference's own training loops (from ``baseline/_ref``) next to this package's race, same seeds.

    python baseline/parity_race.py --optimizers adamw,grokadamw,lion,supergrok15,supergrok2 --seeds 42,123 --max-steps 5000 \
        --out parity.json

For every (optimizer, seed) the reference arm calls ``OPTIMIZER_REGISTRY[name](cfg, init, tx, ty, vx, vy, device, 0)`` of the
reference's ``grokking_race_v2.py`` (its own ``Transformer``, ``make_data``, optimizer and native kernels, reference
grokking_race_v2.py:940-947), and this package's arm calls the same registry key of ``supergrok15_b200.race`` with
``reference_compat=True`` (bias correction frozen at step 1, SAM failure semantics, stale amplifier weights: the behaviours of the
reference that shape its curve).  Both arms start from the same initial weights (the reference's ``get_init_state`` and this
package's build the same ``nn.Module`` layout from the same seed; the state dict of one is loaded into the other and checked).
Output: grok step, final accuracies and the validation-accuracy curve of both arms, and their differences.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import time
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def import_reference():
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "grokking_optimizers")):
        raise RuntimeError("baseline/_ref is not installed (python baseline/build_reference.py <reference source>)")
    for name in ("matplotlib", "matplotlib.pyplot"):
        try:
            __import__(name)
        except Exception:  # noqa: BLE001
            m = types.ModuleType(name)
            m.use = lambda *a, **k: None
            sys.modules[name] = m
    import torch  # noqa: F401  (libtorch must be loaded before the reference's extension)
    shim = os.path.join(ref_dir, "libref_shim.so")
    if os.path.exists(shim):
        ctypes.CDLL(shim, mode=ctypes.RTLD_GLOBAL)
    # the reference's modules are imported under private names so that this package's own grokking_optimizers stays importable
    import importlib.util
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "grokking_optimizers" or k.startswith("grokking_optimizers.")
             or k == "grokking_race_v2"}
    sys.path.insert(0, ref_dir)
    try:
        import grokking_optimizers as ref_go                 # noqa: F401  (resolved from baseline/_ref: it is first on the path)
        import grokking_race_v2 as ref_race
        assert "baseline/_ref" in os.path.abspath(ref_race.__file__).replace("\\", "/")
    finally:
        sys.path.remove(ref_dir)
    ref_modules = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "grokking_optimizers" or k.startswith("grokking_optimizers.")
                   or k == "grokking_race_v2"}
    sys.modules.update(saved)
    return ref_race, ref_modules


def curve(res):
    return {"steps": list(res.steps), "val_acc": [round(float(v), 4) for v in res.val_accs], "train_acc": [round(float(v), 4) for v in res.train_accs]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--optimizers", default="adamw,grokadamw,lion,supergrok15,supergrok2")
    ap.add_argument("--seeds", default="42,123")
    ap.add_argument("--max-steps", type=int, default=5000)
    ap.add_argument("--frac-train", type=float, default=0.5)
    ap.add_argument("--out", default="parity.json")
    ap.add_argument("--skip-reference", action="store_true")
    a = ap.parse_args()
    import torch
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    from supergrok15_b200.race import config as cfg_mod
    from supergrok15_b200.race import runner
    from supergrok15_b200.race.train import OPTIMIZER_REGISTRY as OURS
    names = [n.strip() for n in a.optimizers.split(",")]
    seeds = [int(s) for s in a.seeds.split(",")]
    ref_race = None
    if not a.skip_reference:
        ref_race, ref_modules = import_reference()
    out = {"config": {"scale": "small (d128, 2 layers, 4 heads)", "task": "division mod 97", "frac_train": a.frac_train, "max_steps": a.max_steps,
                      "reference_compat": True, "device": str(dev)}, "runs": []}
    for name in names:
        for seed in seeds:
            base = dict(cfg_mod.DEFAULT_CONFIG)
            base.update(cfg_mod.COMMON)
            base.update(cfg_mod.MODEL_SCALES["small"])
            base.update(cfg_mod.OPTIMIZER_CONFIGS.get(name, {}))
            base.update(max_steps=a.max_steps, frac_train=a.frac_train, seed=seed, compile_model=False, use_amp=False)
            rec = {"optimizer": name, "seed": seed}
            # ---- this package, reference_compat
            c = dict(base, reference_compat=True)
            torch.manual_seed(seed)
            from supergrok15_b200.race.data import make_data_for_task
            from supergrok15_b200.race.train import get_init_state
            tx, ty, vx, vy = (t.to(dev) for t in make_data_for_task(c, seed))
            init = get_init_state(c, dev)
            t0 = time.time()
            r = OURS[name](c, init, tx, ty, vx, vy, dev, 0, None)
            rec["ours"] = {"grok_step": r.grokking_step, "total_steps": r.total_steps, "final_val_acc": r.final_val_acc,
                           "final_train_acc": r.final_train_acc, "wall_s": round(time.time() - t0, 1), "events": r.events[:5], **curve(r)}
            # ---- the reference
            if ref_race is not None:
                saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "grokking_optimizers" or k.startswith("grokking_optimizers.")}
                sys.modules.update({k: v for k, v in ref_modules.items() if k != "grokking_race_v2"})
                try:
                    rc = dict(base)
                    torch.manual_seed(seed)
                    rtx, rty, rvx, rvy = (t.to(dev) for t in ref_race.make_data_for_task(rc, seed))
                    assert torch.equal(rtx, tx) and torch.equal(rvy, vy), "the two data generators disagree"
                    rinit = ref_race.get_init_state(rc, dev)
                    shared = [k for k in rinit if k in init]
                    same_init = bool(shared) and all(torch.equal(rinit[k], init[k]) for k in shared)
                    same_keys = set(rinit) == set(init)
                    t0 = time.time()
                    rr = ref_race.OPTIMIZER_REGISTRY[name](rc, rinit, rtx, rty, rvx, rvy, dev, 0)
                    rec["reference"] = {"grok_step": rr.grokking_step, "total_steps": rr.total_steps, "final_val_acc": rr.final_val_acc,
                                        "final_train_acc": rr.final_train_acc, "wall_s": round(time.time() - t0, 1), "same_init_values": bool(same_init), "same_state_dict_keys": bool(same_keys),
                                        **curve(rr)}
                except Exception as e:  # noqa: BLE001
                    rec["reference"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
                finally:
                    for k in [k for k in sys.modules if k == "grokking_optimizers" or k.startswith("grokking_optimizers.")]:
                        sys.modules.pop(k)
                    sys.modules.update(saved)
                ro, rf = rec["ours"], rec.get("reference", {})
                if "val_acc" in rf:
                    n = min(len(ro["val_acc"]), len(rf["val_acc"]))
                    rec["max_val_acc_gap_common_prefix"] = round(max((abs(x - y) for x, y in zip(ro["val_acc"][:n], rf["val_acc"][:n])), default=0.0), 4)
                    if ro["grok_step"] and rf["grok_step"]:
                        rec["grok_step_ratio_ours_over_reference"] = round(ro["grok_step"] / rf["grok_step"], 3)
            out["runs"].append(rec)
            print(json.dumps({k: v for k, v in rec.items() if k not in ("ours", "reference")} |
                             {"ours_grok": rec["ours"]["grok_step"], "ref_grok": rec.get("reference", {}).get("grok_step"),
                              "ref_error": rec.get("reference", {}).get("error")}), flush=True)
            with open(a.out, "w") as f:
                json.dump(out, f)
    return 0


if __name__ == "__main__":
    sys.exit(main())
