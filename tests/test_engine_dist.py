"""Sharded (ZeRO) step == unsharded step.  CPU: two gloo ranks.  GPU: NCCL bootstrap + in-kernel collectives."""
import os
import socket
import subprocess
import sys
import tempfile

import pytest
import torch

from supergrok15_b200.parallel import assign_tensors, flat_ranges, grouped_layout, imbalance

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import dist_worker  # noqa: E402


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _launch(world, optimizer, device, comm, steps, dtype="f32", timeout=600):
    port = _free_port()
    out = os.path.join(tempfile.mkdtemp(), "out.pt")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "dist_worker.py"), str(r), str(world), str(port), optimizer, out,
                               device, comm, str(steps), dtype], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(world)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        logs.append(o)
    assert all(p.returncode == 0 for p in procs), "\n".join(l[-3000:] for l in logs)
    return torch.load(out)


def test_ownership_is_deterministic_and_balanced():
    numels = [786432, 1536, 262144, 512, 512, 512, 1048576, 2048, 1048576, 512, 512, 512] * 6 + [50688, 2048, 512, 512, 50688, 99]
    own = assign_tensors(numels, 8)
    assert own == assign_tensors(list(numels), 8)
    assert imbalance(numels, own, 8) < 1.15
    offs, regions, total = grouped_layout(numels, own, 8)
    assert all(o % 8 == 0 for o in offs) and regions[0][0] == 0 and regions[-1][1] == total
    for r, (b, e) in enumerate(regions):
        mine = [i for i, o in enumerate(own) if o == r]
        assert all(b <= offs[i] and offs[i] + numels[i] <= e for i in mine)
    fr = flat_ranges(1000 * 8, 8)
    assert fr[0] == (0, 1000) and fr[-1] == (7000, 8000)


@pytest.mark.dist
@pytest.mark.parametrize("optimizer", ["supergrok2", "adamw", "grokadamw", "lion"])
def test_sharded_equals_unsharded_cpu_gloo(optimizer):
    steps = 2
    res = _launch(2, optimizer, "cpu", "nccl", steps)
    ref = dist_worker.reference_run(optimizer, steps)
    for got in res["params"]:
        assert torch.allclose(got, ref, rtol=2e-4, atol=2e-6), (got - ref).abs().max()
    assert torch.equal(res["params"][0], res["params"][1])            # every rank holds the same parameters
    assert len(set(res["owner"])) == (1 if optimizer in ("adamw", "lion") else 2)


@pytest.mark.gpu
@pytest.mark.dist
@pytest.mark.parametrize("comm", ["p2p", "nccl", "nvls"])
@pytest.mark.parametrize("optimizer", ["supergrok2", "adamw", "grokadamw"])
def test_sharded_equals_unsharded_gpu(optimizer, comm):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    steps = 2
    res = _launch(2, optimizer, "cuda", comm, steps)
    ref = dist_worker.reference_run(optimizer, steps, device="cuda")
    for got in res["params"]:
        assert torch.allclose(got, ref, rtol=5e-4, atol=5e-6), (got - ref).abs().max()
    assert torch.equal(res["params"][0], res["params"][1])
