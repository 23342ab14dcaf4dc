"""Sharded checkpoint round-trip / re-shard, heartbeat failure detection and the simulated signal pad (CPU only)."""
import os
import socket
import subprocess
import sys
import tempfile
import threading
import time

import pytest
import torch

from supergrok15_b200.parallel import ZeroEngine, checkpoint
from supergrok15_b200.parallel.fault import Heartbeat, PeerLost, SimSignalPad, guard_step
from supergrok15_b200.utils import fraction, peaks

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import dist_worker  # noqa: E402


def _engine(opt):
    m, x, y = dist_worker.make_problem()
    return ZeroEngine(m, opt, dist_worker.OPT_KW.get(opt, {}), param_dtype=torch.float32), x, y


@pytest.mark.parametrize("opt", ["supergrok2", "adamw", "grokadamw"])
def test_checkpoint_round_trip_world1(opt, tmp_path):
    e1, x, y = _engine(opt)
    for _ in range(2):
        e1.train_step(x, y)
    checkpoint.save(e1, str(tmp_path))
    e1.train_step(x, y)
    e2, _, _ = _engine(opt)
    checkpoint.load(e2, str(tmp_path))
    e2.train_step(x, y)
    for p, q in zip(e1.params, e2.params):
        assert torch.allclose(p, q, rtol=0, atol=0, equal_nan=True)
    full = checkpoint.consolidate(str(tmp_path))
    assert full["manifest"]["world"] == 1 and (opt in ("adamw",) or all(m is not None for m in full["masters"]))


def test_flat_checkpoint_moves_between_bucketed_and_plain_layouts(tmp_path):
    """AdamW state saved by an engine whose step overlaps backward (one owned range per bucket) loads into a plain engine and back."""
    def eng(overlap):
        m, x, y = dist_worker.make_problem()
        return ZeroEngine(m, "adamw", dist_worker.OPT_KW["adamw"], param_dtype=torch.float32, overlap=overlap, bucket_numel=3000), x, y
    e1, x, y = eng(True)
    assert len(e1.buckets) >= 3 and len(e1.segments) == len(e1.buckets)
    for _ in range(2):
        e1.train_step(x, y)
    checkpoint.save(e1, str(tmp_path / "a"))
    assert checkpoint.verify(str(tmp_path / "a")) == []
    e2, _, _ = eng(False)
    checkpoint.load(e2, str(tmp_path / "a"))
    e1.train_step(x, y)
    e2.train_step(x, y)
    for p, q in zip(e1.params, e2.params):
        assert torch.equal(p, q)
    checkpoint.save(e2, str(tmp_path / "b"))
    e3, _, _ = eng(True)
    checkpoint.load(e3, str(tmp_path / "b"))
    e2.train_step(x, y)
    e3.train_step(x, y)
    for p, q in zip(e2.params, e3.params):
        assert torch.equal(p, q)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, {here!r}); sys.path.insert(0, os.path.dirname({here!r}))
import dist_worker
from supergrok15_b200.parallel import ZeroEngine, checkpoint
rank, world, port, mode, path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5]
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
dist.init_process_group("gloo")
m, x, y = dist_worker.make_problem()
eng = ZeroEngine(m, "supergrok2", dist_worker.OPT_KW["supergrok2"], comm="nccl", param_dtype=torch.float32)
per = x.shape[0] // world
xs, ys = x[rank*per:(rank+1)*per], y[rank*per:(rank+1)*per]
if mode == "save":
    eng.train_step(xs, ys); eng.train_step(xs, ys)
    checkpoint.save(eng, path)
else:
    checkpoint.load(eng, path)
eng.train_step(xs, ys)
if rank == 0:
    torch.save(torch.cat([p.detach().reshape(-1) for p in eng.params]), os.path.join(path, mode + "_final.pt"))
dist.barrier(); dist.destroy_process_group()
'''


@pytest.mark.dist
def test_checkpoint_reshard_2_to_1(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(WORKER.format(here=HERE))
    port = str(_free_port())
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", port, "save", str(tmp_path)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    ref = torch.load(tmp_path / "save_final.pt")
    # reload on ONE rank with the full batch: same parameters after the same third step
    m, x, y = dist_worker.make_problem()
    eng = ZeroEngine(m, "supergrok2", dist_worker.OPT_KW["supergrok2"], param_dtype=torch.float32)
    checkpoint.load(eng, str(tmp_path))
    eng.train_step(x, y)
    got = torch.cat([p.detach().reshape(-1) for p in eng.params])
    assert torch.allclose(got, ref, rtol=2e-4, atol=2e-6)


def test_truncated_shard_is_detected(tmp_path):
    e1, x, y = _engine("grokadamw")
    e1.train_step(x, y)
    checkpoint.save(e1, str(tmp_path))
    assert checkpoint.verify(str(tmp_path)) == []
    f = __import__("pathlib").Path(checkpoint.resolve(str(tmp_path))) / "rank_0.pt"
    payload = torch.load(f, weights_only=False)
    next(iter(payload["tensors"].values()))["master"][0] += 1.0        # silent corruption of one value
    torch.save(payload, f)
    assert checkpoint.verify(str(tmp_path)) == [0]
    f.write_bytes(f.read_bytes()[:100])                                # truncated file
    assert checkpoint.verify(str(tmp_path)) == [0]


def test_save_interrupted_before_the_manifest_keeps_the_previous_checkpoint(tmp_path, monkeypatch):
    """A rank that dies between its shard and the manifest (modelled by an exception at that point of ``save``) leaves ``latest``
    on the previous, complete save; its m / v / optimizer state are covered by the checksum, not only the master weights."""
    e1, x, y = _engine("grokadamw")
    e1.train_step(x, y)
    d1 = checkpoint.save(e1, str(tmp_path))
    want = torch.cat([p.detach().reshape(-1).clone() for p in e1.params])
    e1.train_step(x, y)

    def die(_engine):
        raise KeyboardInterrupt("rank killed mid-save")
    monkeypatch.setattr(checkpoint, "_before_manifest", die)
    with pytest.raises(KeyboardInterrupt):
        checkpoint.save(e1, str(tmp_path))
    monkeypatch.undo()
    assert checkpoint.resolve(str(tmp_path)) == d1 and checkpoint.verify(str(tmp_path)) == []
    e2, _, _ = _engine("grokadamw")
    checkpoint.load(e2, str(tmp_path))
    assert torch.equal(torch.cat([p.detach().reshape(-1) for p in e2.params]), want)
    # a flipped value in an optimizer moment (not a master weight) is caught
    f = __import__("pathlib").Path(d1) / "rank_0.pt"
    payload = torch.load(f, weights_only=False)
    st = next(iter(payload["tensors"].values()))["state"]
    st["exp_avg"].view(-1)[0] += 1.0
    torch.save(payload, f)
    assert checkpoint.verify(str(tmp_path)) == [0]
    with pytest.raises(RuntimeError, match="corrupted"):
        checkpoint.load(e2, str(tmp_path))


def test_a_timed_out_step_is_not_followed_by_a_save(tmp_path):
    """The status word of the collectives says that a wait on a peer ran out: ``save`` raises before it writes anything, and
    the next step raises before it launches anything."""
    from supergrok15_b200.parallel import CommTimeout
    e1, x, y = _engine("supergrok2")
    e1.train_step(x, y)
    e1.status.fill_(1 | (1 << 8) | (2 << 16))
    with pytest.raises(CommTimeout, match="peer 1"):
        checkpoint.save(e1, str(tmp_path))
    assert not any(tmp_path.iterdir())
    e1.train_step(x, y)                                            # the raise cleared the word: training can go on after a reload


def test_heartbeat_on_a_real_store_reports_a_rank_that_never_joined_at_once():
    """``TCPStore.get`` blocks until the key exists; the heartbeat must not: a peer that never joined is reported within its timeout."""
    from datetime import timedelta
    import torch.distributed as dist
    store = dist.TCPStore("127.0.0.1", _free_port(), 1, True, timeout=timedelta(seconds=30))
    a = Heartbeat(store, 0, 2, interval_s=0.05).start()
    t0 = time.time()
    assert a.dead_peers(timeout_s=0.3) == [1]
    assert time.time() - t0 < 5.0
    b = Heartbeat(store, 1, 2, interval_s=0.05).start()
    time.sleep(0.2)
    assert a.dead_peers(timeout_s=0.5) == []
    a.stop(); b.stop()


class _DictStore:
    def __init__(self):
        self.d, self.lock = {}, threading.Lock()

    def set(self, k, v):
        with self.lock:
            self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        with self.lock:
            return self.d[k]


def test_heartbeat_detects_silent_rank():
    store = _DictStore()
    a = Heartbeat(store, 0, 3, interval_s=0.05).start()
    b = Heartbeat(store, 1, 3, interval_s=0.05).start()
    time.sleep(0.2)
    assert a.dead_peers(timeout_s=0.5) == [2]                      # rank 2 never joined
    b.stop()                                                       # rank 1 exits between steps
    time.sleep(0.4)
    assert a.dead_peers(timeout_s=0.3) == [1, 2]
    with pytest.raises(PeerLost):
        guard_step(a, timeout_s=0.3)
    a.stop()


def test_sim_signal_pad_barrier_and_dropped_flag():
    pad = SimSignalPad(3)
    res = [None] * 3
    ts = [threading.Thread(target=lambda r=r: res.__setitem__(r, pad.barrier(r, 1, 2.0))) for r in range(3)]
    [t.start() for t in ts]; [t.join() for t in ts]
    assert res == [0, 0, 0]
    pad = SimSignalPad(2, drop=lambda src, dst, epoch: src == 1 and dst == 0)      # rank 1's flag to rank 0 is lost
    res = [None] * 2
    ts = [threading.Thread(target=lambda r=r: res.__setitem__(r, pad.barrier(r, 1, 0.3))) for r in range(2)]
    [t.start() for t in ts]; [t.join() for t in ts]
    assert res[0] == (1 | (1 << 8)) and res[1] == 0                # rank 0 reports WHICH peer it gave up on


def test_roofline_helpers():
    pk = peaks()
    assert pk["hbm_gbs"] > 1000 and pk["bf16_tflops"] > 100
    f = fraction(1.0, flops=1e12, hbm_bytes=1e9, pk={"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1400.0, "source": "measured"})
    assert f["bound"] == "compute" and abs(f["fraction"] - 0.625) < 1e-6
