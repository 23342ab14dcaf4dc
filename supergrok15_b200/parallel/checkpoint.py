"""Sharded checkpoints of a ``ZeroEngine`` (the reference has no checkpointing at all).

Layout of a checkpoint directory:
    latest                  name of the newest complete save (one line of text)
    save_<n>/manifest.json  world size, optimizer name, layout mode, tensor sizes, ownership map, dtype, per-shard SHA-256
    save_<n>/rank_<k>.pt    what rank k owns: fp32 master tensors, optimizer state per tensor (or flat ranges), optimizer extras

``save`` is collective and atomic: every rank first checks that no device-side wait timed out since the last check (a step that
ran on incomplete gradients is never persisted), writes its shard to a temporary name, flushes it to disk and renames it; rank 0
writes the manifest the same way, only after every shard is in place, and then flips ``latest`` to the new save.  Every save goes
into a sub-directory of its own; the previous one is kept until the next save has completed (older ones are removed), so a rank
that dies anywhere inside ``save`` leaves ``latest`` pointing at a complete older save.  The per-shard SHA-256 covers every tensor of the payload (masters, moments, optimizer state, extras).  ``load`` accepts a checkpoint
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


def _row_shards(engine) -> Dict[int, dict]:
    """Muon with the rows of its matrices split over the ranks: this rank's rows of the fp32 master and of the momentum."""
    out = {}
    for i, v in zip(getattr(engine, "rs_idx", None) or [], getattr(engine, "rs_views", None) or []):
        rl, c = v["shape"]
        out[i] = {"rows": [engine.rank * rl, (engine.rank + 1) * rl], "master": v["master"].view(rl, c).detach().cpu().clone(),
                  "momentum_buffer": v["mom"].view(rl, c).detach().cpu().clone()}
    return out


def _walk(obj, prefix, out):
    if torch.is_tensor(obj):
        out.append((prefix, obj))
    elif isinstance(obj, dict):
        for k in sorted(obj, key=str):
            _walk(obj[k], f"{prefix}/{k}", out)
    elif isinstance(obj, (list, tuple)):
        for k, v in enumerate(obj):
            _walk(v, f"{prefix}/{k}", out)
    else:
        out.append((prefix, repr(obj)))


def _payload_digest(payload: dict) -> str:
    """SHA-256 over EVERY entry of a shard's payload: names, dtypes, shapes and bytes of all tensors (master weights, moments,
    optimizer state, extras) and the repr of every other leaf, in a fixed order."""
    leaves: list = []
    _walk(payload, "", leaves)
    h = hashlib.sha256()
    for name, v in leaves:
        h.update(name.encode())
        if torch.is_tensor(v):
            t = v.detach().cpu().contiguous()
            h.update(f"{t.dtype}{tuple(t.shape)}".encode())
            h.update(t.reshape(-1).view(torch.uint8).numpy().tobytes())
        else:
            h.update(v.encode())
    return h.hexdigest()


def _atomic_write(path: str, write) -> None:
    """``write(file_object)`` into ``path + '.tmp'``, flush to disk, rename over ``path``: a reader never sees a partial file."""
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        write(fh)
        fh.flush()
        os.fsync(fh.fileno())
    os.replace(tmp, path)


def _latest(path: str) -> Optional[str]:
    try:
        with open(os.path.join(path, "latest")) as fh:
            name = fh.read().strip()
        return name if name and os.path.isdir(os.path.join(path, name)) else None
    except OSError:
        return None


def resolve(path: str) -> str:
    """Directory that holds the newest complete save under ``path`` (``path`` itself for a directory written without ``latest``)."""
    name = _latest(path)
    return os.path.join(path, name) if name else path


def save(engine, path: str, keep: int = 2) -> str:
    """Collective.  Returns the directory of the new save.  ``keep``: complete saves left under ``path`` afterwards."""
    if hasattr(engine, "check"):
        engine.check()                                     # raises CommTimeout: state that saw a timed-out step is not persisted
    os.makedirs(path, exist_ok=True)
    prev = _latest(path)
    save_id = (int(prev.split("_")[1]) + 1) if prev else 1
    if engine.world > 1:                                   # every rank must write into the same sub-directory
        import torch.distributed as dist
        ids = [None] * engine.world
        dist.all_gather_object(ids, save_id, group=engine.group)
        save_id = max(ids)
    name = f"save_{save_id:06d}"
    d = os.path.join(path, name)
    os.makedirs(d, exist_ok=True)
    payload = {"rank": engine.rank, "world": engine.world, "tensors": _per_tensor_state(engine), "steps": engine.steps, "save_id": save_id}
    rows = _row_shards(engine)
    if rows:
        payload["row_shards"] = rows
    if engine.flat_mode:
        # the flat ranges this rank owns (one, or one per bucket when the step overlaps backward) and their state, concatenated
        n = engine.n_own
        payload["flat"] = {"segments": [[b, e] for b, e, _ in engine.segments], "master": engine.master[:n].cpu().clone(),
                           "m": engine.m[:n].cpu().clone(), "v": engine.v[:n].cpu().clone() if engine.v is not None else None}
    elif engine.opt is not None:
        sd = engine.opt.state_dict()
        payload["extra"] = sd.get("extra")
        payload["param_groups"] = [{k: v for k, v in g.items() if k != "params"} for g in sd["param_groups"]]
    _atomic_write(os.path.join(d, f"rank_{engine.rank}.pt"), lambda fh: torch.save(payload, fh))
    digest = _payload_digest(payload)
    if engine.world > 1:
        import torch.distributed as dist
        digests = [None] * engine.world
        dist.all_gather_object(digests, digest, group=engine.group)      # also the barrier: every shard is in place
    else:
        digests = [digest]
    _before_manifest(engine)
    if engine.rank == 0:
        man = {"world": engine.world, "optimizer": engine.name, "flat_mode": engine.flat_mode, "numels": [p.numel() for p in engine.params],
               "owner": engine.owner, "total": engine.total, "param_dtype": str(engine.pdtype), "sha256": digests, "save_id": save_id,
               "format": 2}
        _atomic_write(os.path.join(d, "manifest.json"), lambda fh: fh.write(json.dumps(man, indent=1).encode()))
        _atomic_write(os.path.join(path, "latest"), lambda fh: fh.write(name.encode()))   # the save exists from here on
        import shutil
        old = sorted(n for n in os.listdir(path) if n.startswith("save_") and n < name and os.path.isdir(os.path.join(path, n)))
        for n in old[:max(0, len(old) - (keep - 1))]:
            shutil.rmtree(os.path.join(path, n), ignore_errors=True)
    _barrier(engine)
    return d


def _before_manifest(engine) -> None:
    """Hook between the shard writes and the manifest write (tests stop a save here to model a rank dying mid-save)."""


def _read_manifest(path: str) -> dict:
    with open(os.path.join(path, "manifest.json")) as fh:
        return json.load(fh)


def _load_shard(path: str, r: int) -> dict:
    """A shard holds tensors, numbers, strings and containers of them only, so the restricted unpickler suffices; checkpoints
    whose optimizer extras hold other objects (a generator state is a tensor, so none of this package's do) need the full one."""
    f = os.path.join(path, f"rank_{r}.pt")
    try:
        return torch.load(f, weights_only=True)
    except Exception:  # noqa: BLE001
        return torch.load(f, weights_only=False)


def verify(path: str) -> List[int]:
    """Ranks whose shard cannot be read, belongs to another save than the manifest, or does not match the manifest checksum
    (empty = intact)."""
    path = resolve(path)
    man = _read_manifest(path)
    bad = []
    for r in range(man["world"]):
        try:
            p = _load_shard(path, r)
            if p.get("save_id", 0) != man.get("save_id", 0) or _payload_digest(p) != man["sha256"][r]:
                bad.append(r)
        except Exception:  # noqa: BLE001
            bad.append(r)
    return bad


def consolidate(path: str) -> dict:
    """Unsharded view: {"masters": [fp32 tensor per parameter], "state": {index: {...}}, "extra": ..., "manifest": ...}."""
    path = resolve(path)
    man = _read_manifest(path)
    n = len(man["numels"])
    masters: List[Optional[torch.Tensor]] = [None] * n
    state: Dict[int, dict] = {}
    extra = None
    flat_parts = []
    row_parts: Dict[int, list] = {}
    for r in range(man["world"]):
        p = _load_shard(path, r)
        for i, rec in p["tensors"].items():
            masters[int(i)] = rec["master"]
            state[int(i)] = rec["state"]
        if p.get("extra") is not None and extra is None:
            extra = p["extra"]
        if "flat" in p:
            flat_parts.append(p["flat"])
        for i, rec in p.get("row_shards", {}).items():
            row_parts.setdefault(int(i), []).append(rec)
    for i, parts in row_parts.items():                      # matrices stored as row blocks: put the blocks back together
        parts.sort(key=lambda rec: rec["rows"][0])
        masters[i] = torch.cat([rec["master"] for rec in parts], 0).reshape(-1)
        state[i] = {"momentum_buffer": torch.cat([rec["momentum_buffer"] for rec in parts], 0)}
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
    """Restore an engine from the newest complete save under ``path``, written with any world size (collective; re-shards when
    the world size differs)."""
    path = resolve(path)
    man = _read_manifest(path)
    assert man["optimizer"] == engine.name and man["numels"] == [p.numel() for p in engine.params], "checkpoint does not match the model"
    bad = verify(path)
    if bad:
        raise RuntimeError(f"checkpoint {path}: shards of ranks {bad} are missing, from another save than the manifest, or corrupted")
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
            p0 = _load_shard(path, 0)
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
            for i, v in zip(getattr(engine, "rs_idx", None) or [], getattr(engine, "rs_views", None) or []):
                rl, c = v["shape"]
                lo = engine.rank * rl
                v["master"].copy_(full["masters"][i].view(-1, c)[lo:lo + rl].reshape(-1))
                mom = full["state"].get(i, {}).get("momentum_buffer")
                if mom is not None:
                    v["mom"].copy_(mom.reshape(-1, c)[lo:lo + rl].reshape(-1))
            # every rank rebuilds the full low-precision parameter buffer from the consolidated masters
            for i, p in enumerate(engine.params):
                p.data.copy_(full["masters"][i].view(p.shape).to(engine.pdtype))
    _barrier(engine)
