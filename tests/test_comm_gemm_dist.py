"""All-gather and reduce-scatter fused into the tcgen05 GEMM: results against fp32 references on 2 GPUs."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

from test_engine_dist import _free_port

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.dist
def test_fused_comm_gemms_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world, port = 2, _free_port()
    out = os.path.join(tempfile.mkdtemp(), "out.pt")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "comm_gemm_worker.py"), str(r), str(world), str(port), out], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        logs.append(o)
    assert all(p.returncode == 0 for p in procs), "\n".join(l[-3000:] for l in logs)
    res = torch.load(out)
    for shape, errs in res.items():
        assert max(errs) < 2e-2, (shape, errs)


@pytest.mark.gpu
def test_allgather_gemm_single_rank_is_plain_gemm():
    """World of one: no copier CTAs, no waits; the fused entry point must equal the plain GEMM."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from supergrok15_b200.ops import gemm
    from supergrok15_b200.parallel.comm_gemm import ShardedWeight
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    w = ShardedWeight(512, 256, dev)
    w.shard.copy_((torch.randn(512, 256, device=dev) * 0.05).to(torch.bfloat16))
    x = torch.randn(300, 256, device=dev).to(torch.bfloat16)
    y = w.matmul(x)
    torch.cuda.synchronize()
    gemm.check(dev)
    ref = x.float() @ w.full.float().t()
    assert float((y.float() - ref).abs().max() / ref.abs().max()) < 2e-2


@pytest.mark.gpu
def test_reducescatter_gemm_single_rank_is_plain_gemm():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from supergrok15_b200.ops import gemm
    from supergrok15_b200.parallel.comm_gemm import ReduceScatterGemm
    dev = torch.device("cuda:0")
    torch.manual_seed(1)
    a = torch.randn(384, 320, device=dev).to(torch.bfloat16)
    b = (torch.randn(192, 320, device=dev) * 0.05).to(torch.bfloat16)
    op = ReduceScatterGemm(384, 192, dev)
    for _ in range(3):
        y = op(a, b)
    torch.cuda.synchronize()
    gemm.check(dev)
    ref = a.float() @ b.float().t()
    assert float((y.float() - ref).abs().max() / ref.abs().max()) < 2e-2
