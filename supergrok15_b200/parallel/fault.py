"""Failure detection for the data-parallel engine, exercised without ever faulting a GPU.

* ``Heartbeat``: every rank stamps a key in the process group's key-value store from a daemon thread; before launching
  a step a rank can ask which peers have gone silent (``dead_peers``) and refuse to launch kernels that would wait for them.
* Device-side waits are bounded (``csrc/comm.cuh``): a wait that runs out writes STATUS_TIMEOUT | peer | site into the
  engine's status word and returns; ``ZeroEngine.check()`` turns it into ``CommTimeout`` and the CUDA context stays usable.
* ``SimSignalPad`` restates the epoch-flag barrier protocol in host memory so that dropped flag writes and late ranks can
  be injected in unit tests (threads stand in for ranks).
* Recovery model: abort the step, reload the last sharded checkpoint (``parallel/checkpoint.py``), possibly with fewer ranks.

A device-side fault injector (a kernel that traps, hangs or touches a bad address) is deliberately not part of this package.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, List, Optional


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.5, prefix: str = "hb"):
        self.store, self.rank, self.world, self.interval, self.prefix = store, rank, world, interval_s, prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self):
        self.store.set(self._key(self.rank), str(time.time()))

    def start(self):
        self.beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self.beat()
            except Exception:  # noqa: BLE001  (store gone: the job is shutting down)
                return

    def stop(self):
        self._stop.set()

    def last_seen(self, r: int) -> Optional[float]:
        """Time of rank r's last beat, or None if it never beat.  A ``torch.distributed`` store blocks in ``get`` until the key
        exists (up to the store's timeout, minutes by default), so the key is looked up with ``check`` first where the store
        has it: a peer that never joined is reported at once."""
        try:
            check = getattr(self.store, "check", None)
            if check is not None and not check([self._key(r)]):
                return None
            v = self.store.get(self._key(r))
            return float(v.decode() if isinstance(v, (bytes, bytearray)) else v)
        except Exception:  # noqa: BLE001
            return None

    def dead_peers(self, timeout_s: float = 3.0) -> List[int]:
        now = time.time()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            t = self.last_seen(r)
            if t is None or now - t > timeout_s:
                dead.append(r)
        return dead


class PeerLost(RuntimeError):
    pass


def guard_step(hb: Heartbeat, timeout_s: float = 3.0) -> None:
    """Raise before launching a step if a peer's heartbeat is stale (its kernels would never signal)."""
    dead = hb.dead_peers(timeout_s)
    if dead:
        raise PeerLost(f"rank {hb.rank}: peers {dead} silent for more than {timeout_s}s; aborting before the next launch")


class SimSignalPad:
    """Host-memory model of the device barrier: pads[r][s] is slot s of rank r's pad.  ``drop`` decides whether a
    given (src, dst, epoch) flag write is lost."""

    def __init__(self, world: int, drop: Optional[Callable[[int, int, int], bool]] = None):
        self.world = world
        self.pads = [[0] * world for _ in range(world)]
        self.drop = drop or (lambda src, dst, epoch: False)
        self.lock = threading.Lock()

    def barrier(self, rank: int, epoch: int, timeout_s: float = 1.0) -> int:
        """Returns 0, or STATUS_TIMEOUT | (peer << 8) for the first peer that never showed up."""
        for dst in range(self.world):
            if not self.drop(rank, dst, epoch):
                with self.lock:
                    self.pads[dst][rank] = max(self.pads[dst][rank], epoch)
        t0 = time.time()
        for src in range(self.world):
            while True:
                with self.lock:
                    if self.pads[rank][src] >= epoch:
                        break
                if time.time() - t0 > timeout_s:
                    return 1 | (src << 8)
                time.sleep(0.001)
        return 0
