"""Sharded checkpoints of a ``ZeroEngine`` (the reference has no checkpointing at all).

Layout of a checkpoint directory:
    manifest.json   world size, optimizer name, layout mode, tensor sizes, ownership map, dtype, per-shard SHA-256
    rank_<k>.pt     what rank k owns: fp32 master tensors, optimizer state per tensor (or flat ranges), optimizer extras

``save`` is collective (every rank writes its own file, rank 0 writes the manifest).  ``load`` accepts a checkpoint
written with ANY world size: the ownership map is a pure function of (tensor sizes, world size), so a rank simply reads
the tensors it owns under the new map from whichever files hold them.  ``consolidate`` rebuilds one unsharded dictionary
(per-tensor state in the model's parameter order) without needing a process group.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, List, Optional

import torch


def _sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def _barrier(engine):
    if engine.world > 1:
        import torch.distributed as dist
        dist.barrier(engine.group)


def _per_tensor_state(engine) -> Dict[int, dict]:
    """{global tensor index: {"master": fp32 tensor, "state": {...}}} for the tensors this rank owns."""
    out = {}
    b = engine.my_begin
    if engine.flat_mode:
        return out
    opt = engine.opt
    if hasattr(opt, "_sync_steps_to_state") and getattr(opt, "_state_initialized", False):
        opt._sync_steps_to_state()
    handles = engine.master_views if engine.name != "supergrok2" else list(opt._flat_params)
    for k, i in enumerate(engine.own_idx):
        n = engine.params[i].numel()
        master = engine.master[engine.offsets[i] - b: engine.offsets[i] - b + n].detach().cpu().clone()
        st = {}
        key = handles[k] if k < len(handles) else None
        if key is not None and key in opt.state:
            for name, v in opt.state[key].items():
                st[name] = v.detach().cpu().clone() if torch.is_tensor(v) else v
        out[i] = {"master": master, "state": st}
    return out


def _payload_digest(payload: dict) -> str:
    """SHA-256 over the fp32 master values a shard file holds (tensor order, or the flat range)."""
    if "flat" in payload:
        return _sha(payload["flat"]["master"])
    parts = [payload["tensors"][i]["master"].reshape(-1) for i in sorted(payload["tensors"])]
    return _sha(torch.cat(parts)) if parts else _sha(torch.zeros(0))


def save(engine, path: str) -> None:
    os.makedirs(path, exist_ok=True)
    payload = {"rank": engine.rank, "world": engine.world, "tensors": _per_tensor_state(engine), "steps": engine.steps}
    if engine.flat_mode:
        # the flat ranges this rank owns (one, or one per bucket when the step overlaps backward) and their state, concatenated
        n = engine.n_own
        payload["flat"] = {"segments": [[b, e] for b, e, _ in engine.segments], "master": engine.master[:n].cpu().clone(),
                           "m": engine.m[:n].cpu().clone(), "v": engine.v[:n].cpu().clone() if engine.v is not None else None}
    elif engine.opt is not None:
        sd = engine.opt.state_dict()
        payload["extra"] = sd.get("extra")
        payload["param_groups"] = [{k: v for k, v in g.items() if k != "params"} for g in sd["param_groups"]]
    f = os.path.join(path, f"rank_{engine.rank}.pt")
    torch.save(payload, f)
    digest = _payload_digest(payload)
    if engine.world > 1:
        import torch.distributed as dist
        digests = [None] * engine.world
        dist.all_gather_object(digests, digest, group=engine.group)
    else:
        digests = [digest]
    if engine.rank == 0:
        man = {"world": engine.world, "optimizer": engine.name, "flat_mode": engine.flat_mode, "numels": [p.numel() for p in engine.params],
               "owner": engine.owner, "total": engine.total, "param_dtype": str(engine.pdtype), "master_sha256": digests,
               "format": 1}
        with open(os.path.join(path, "manifest.json"), "w") as fh:
            json.dump(man, fh, indent=1)
    _barrier(engine)


def _read_manifest(path: str) -> dict:
    with open(os.path.join(path, "manifest.json")) as fh:
        return json.load(fh)


def verify(path: str) -> List[int]:
    """Ranks whose shard cannot be read or whose master values do not match the manifest checksum (empty = intact)."""
    man = _read_manifest(path)
    bad = []
    for r in range(man["world"]):
        try:
            p = torch.load(os.path.join(path, f"rank_{r}.pt"), weights_only=False)
            if _payload_digest(p) != man["master_sha256"][r]:
                bad.append(r)
        except Exception:  # noqa: BLE001
            bad.append(r)
    return bad


def consolidate(path: str) -> dict:
    """Unsharded view: {"masters": [fp32 tensor per parameter], "state": {index: {...}}, "extra": ..., "manifest": ...}."""
    man = _read_manifest(path)
    n = len(man["numels"])
    masters: List[Optional[torch.Tensor]] = [None] * n
    state: Dict[int, dict] = {}
    extra = None
    flat_parts = []
    for r in range(man["world"]):
        p = torch.load(os.path.join(path, f"rank_{r}.pt"), weights_only=False)
        for i, rec in p["tensors"].items():
            masters[int(i)] = rec["master"]
            state[int(i)] = rec["state"]
        if p.get("extra") is not None and extra is None:
            extra = p["extra"]
        if "flat" in p:
            flat_parts.append(p["flat"])
    out = {"masters": masters, "state": state, "extra": extra, "manifest": man}
    if flat_parts:
        # scatter every rank's segments back to their positions of the flat buffer (positions do not depend on the world size)
        total = int(man["total"])
        full = {k: (torch.zeros(total) if flat_parts[0][k] is not None else None) for k in ("master", "m", "v")}
        for d in flat_parts:
            segs = d["segments"] if "segments" in d else [[d["begin"], d["end"]]]
            pos = 0
            for b, e in segs:
                for k in ("master", "m", "v"):
                    if full[k] is not None:
                        full[k][b:e] = d[k][pos:pos + e - b]
                pos += e - b
        out["flat"] = full
    return out


def load(engine, path: str) -> None:
    """Restore an engine from a checkpoint of any world size (collective; re-shards when the world size differs)."""
    man = _read_manifest(path)
    assert man["optimizer"] == engine.name and man["numels"] == [p.numel() for p in engine.params], "checkpoint does not match the model"
    full = consolidate(path)
    b = engine.my_begin
    with torch.no_grad():
        if engine.flat_mode:
            fl = full["flat"]
            if fl["master"].numel() < engine.total:                # a larger world pads the flat buffer further
                pad = engine.total - fl["master"].numel()
                fl = {k: (torch.cat([t, torch.zeros(pad)]) if t is not None else None) for k, t in fl.items()}
            for b, e, so in engine.segments:
                engine.master[so:so + e - b].copy_(fl["master"][b:e])
                engine.m[so:so + e - b].copy_(fl["m"][b:e])
                if engine.v is not None:
                    engine.v[so:so + e - b].copy_(fl["v"][b:e])
            p0 = torch.load(os.path.join(path, "rank_0.pt"), weights_only=False)
            engine.steps = int(p0.get("steps", 0))
            engine.pbuf.tensor.copy_(fl["master"][: engine.total].to(engine.pdtype))
        else:
            opt = engine.opt
            if hasattr(opt, "_ensure_state"):
                opt._ensure_state()
            handles = engine.master_views if engine.name != "supergrok2" else list(opt._flat_params)
            for k, i in enumerate(engine.own_idx):
                num = engine.params[i].numel()
                engine.master[engine.offsets[i] - b: engine.offsets[i] - b + num].copy_(full["masters"][i])
                st = opt.state[handles[k]]
                for name, v in full["state"].get(i, {}).items():
                    if torch.is_tensor(v) and name in st and torch.is_tensor(st[name]):
                        st[name].copy_(v.to(st[name].device))
                    else:
                        st[name] = v.to(engine.device) if torch.is_tensor(v) else v
                if hasattr(opt, "_flat_steps") and "step" in full["state"].get(i, {}):
                    opt._flat_steps[k] = int(full["state"][i]["step"])
            if full["extra"] is not None and hasattr(opt, "_load_extra_state"):
                ex = dict(full["extra"])
                ex.pop("flat_steps", None)               # per-tensor steps were restored above in this rank's own numbering
                opt._load_extra_state(ex)
            # every rank rebuilds the full low-precision parameter buffer from the consolidated masters
            for i, p in enumerate(engine.params):
                p.data.copy_(full["masters"][i].view(p.shape).to(engine.pdtype))
    _barrier(engine)
