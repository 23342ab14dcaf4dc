"""Row-sharded Newton-Schulz (collectives inside the tcgen05 GEMMs) against the fp32 iteration on the whole matrix."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

from test_engine_dist import _free_port

HERE = os.path.dirname(os.path.abspath(__file__))


def test_supported_shapes():
    from supergrok15_b200.ops.muon_sharded import arena_bytes, supported
    assert supported(2048, 2048, 8) and supported(5504, 2048, 8) and supported(2048, 5504, 8)       # the 1.3 B decoder's block matrices
    assert supported(4096, 4096, 8) and supported(4096, 4096, 2)
    assert not supported(2048, 1000, 8) and not supported(100, 2048, 8) and not supported(2048, 2048, 3)
    assert arena_bytes([(2048, 2048)], 8) > 2 * 2048 * 2048 * 2


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(512, 256), (256, 256), (256, 640)])
def test_row_sharded_newton_schulz_world_of_one(shape):
    """One rank holds all rows: the same three fused kernels per iteration run without peers."""
    from supergrok15_b200.ops import gemm, oracle
    from supergrok15_b200.ops.muon_sharded import RowShardedNewtonSchulz
    torch.manual_seed(2)
    X = torch.randn(shape, device="cuda")
    X = X / (X.norm() + 1e-7)
    ns = RowShardedNewtonSchulz([shape], X.device)
    for _ in range(4):                                   # eager, eager, captured into one CUDA graph, replayed
        out = ns.run([X], 5)[0]
    torch.cuda.synchronize()
    assert len(ns._graphs) == 1 and not isinstance(next(iter(ns._graphs.values())), int)
    gemm.check()
    ref = oracle.newton_schulz(X.double(), 5).float()
    assert (out - ref).norm() / ref.norm() < 0.06
    k = min(shape)
    Q = out @ out.t() if shape[0] <= shape[1] else out.t() @ out
    Qr = ref @ ref.t() if shape[0] <= shape[1] else ref.t() @ ref
    assert (Q - Qr).norm() / k ** 0.5 < 0.1


@pytest.mark.gpu
@pytest.mark.dist
@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_sharded_newton_schulz_equals_whole_matrix(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = _free_port()
    out = os.path.join(tempfile.mkdtemp(), "out.pt")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "muon_sharded_worker.py"), str(r), str(world), str(port), out], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=400)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        logs.append(o)
    assert all(p.returncode == 0 for p in procs), "\n".join(l[-3000:] for l in logs)
    res = torch.load(out)
    assert len(res) == 12
    for key, e in res.items():
        assert e["rel_vs_fp32"] < 0.06 and e["orth_vs_fp32"] < 0.1 and e["rel_vs_whole_bf16"] < 0.06, (key, e)


def _run_engine(world, sharding, steps=3):
    port = _free_port()
    out = os.path.join(tempfile.mkdtemp(), "out.pt")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "llama_engine_worker.py"), str(r), str(world), str(port), out, sharding, str(steps)],
                              env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=400)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        logs.append(o)
    assert all(p.returncode == 0 for p in procs), "\n".join(l[-3000:] for l in logs)
    return torch.load(out)


@pytest.mark.gpu
@pytest.mark.dist
def test_engine_muon_row_sharded_matches_whole_matrix_ownership():
    """ZeroEngine with Muon: block matrices split by rows over two ranks (collectives inside the Newton-Schulz GEMMs) against the same
    run with every matrix owned whole by one rank.  Both iterate in bf16; the parameters agree to a fraction of the update."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    rows = _run_engine(2, "muon/rows")
    whole = _run_engine(2, "muon/tensors")
    assert rows["row_sharded"] == 7 and whole["row_sharded"] == 0          # wq wk wv wo w1 w3 (tall / square), w2 (wide)
    assert all(torch.equal(rows["params"][0], p) for p in rows["params"])   # every rank ends with the same parameters
    # bf16 parameters: the two runs may round an update to neighbouring bf16 values (one unit in the last place of the largest
    # parameter); anything beyond that, or more than a few such elements, would be a real difference
    a, b = rows["params"][0], whole["params"][0]
    ulp = 2.0 ** -7 * float(b.abs().max())
    assert float((a - b).abs().max()) <= ulp, (float((a - b).abs().max()), ulp)
    moved = (b - whole["init"]).abs()
    assert float(((a - b).abs() > 0.25 * moved.max()).float().mean()) < 0.01
    assert rows["losses"][-1] < rows["losses"][0]


@pytest.mark.gpu
@pytest.mark.dist
def test_engine_allgather_inside_the_first_gemm_matches_the_push_path():
    """AdamW on two ranks: Linear weights whose rows are owned in turn and gathered inside the first consuming GEMM of the next
    forward, against the path that pushes every updated parameter at the end of the step.  Every rank must end with the same
    parameters, and the two paths must agree to bf16 rounding (their forward GEMMs are different kernels)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    fused = _run_engine(2, "adamw/gemm", steps=4)
    push = _run_engine(2, "adamw/push", steps=4)
    assert fused["gathered_in_gemm"] == 8 and push["gathered_in_gemm"] == 0          # 7 block matrices + the output head
    assert all(torch.equal(fused["params"][0], p) for p in fused["params"])
    # the forward GEMM differs (own tcgen05 kernel vs the library one), so the runs agree to bf16 rounding, not bitwise
    a, b = fused["params"][0], push["params"][0]
    ulp = 2.0 ** -7 * float(b.abs().max())
    assert float((a - b).abs().max()) <= 2 * ulp, float((a - b).abs().max())
    assert fused["losses"][-1] < fused["losses"][0] and abs(fused["losses"][-1] - push["losses"][-1]) < 0.05
