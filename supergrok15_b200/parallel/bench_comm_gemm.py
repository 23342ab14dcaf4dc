"""Timing of the GEMMs fused with their collective against "NCCL collective + cuBLAS", one process per GPU.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m supergrok15_b200.parallel.bench_comm_gemm

Cases: all-gather -> GEMM  x[16384, 2048] . W[N, 2048]^T with W row-sharded (N = 2048, 8192); GEMM -> reduce-scatter  M = 16384 with K
sharded (N = 2048 / K = 5504 per world, N = 8192 / K = 2048).  CUDA events on the launching stream, 3 warm-up + 10 timed calls, max over
ranks; rank 0 prints one JSON line per case with the roofline fraction: target = max(FLOPs / measured bf16 peak, bytes that must cross
NVLink per direction / 770 GB/s).
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist


def timed(fn, dev, it=10):
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(it):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / it], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from supergrok15_b200.ops import gemm
    from supergrok15_b200.parallel.comm_gemm import ReduceScatterGemm, ShardedWeight
    from supergrok15_b200.utils import roofline
    for (M, N, K) in [(16384, 2048, 2048), (16384, 8192, 2048)]:
        w = ShardedWeight(N, K, dev)
        w.shard.copy_((torch.randn(w.rows, K, device=dev) * 0.05).to(torch.bfloat16))
        x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier()
        gathered = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        shard = w.shard.clone()

        def baseline():
            dist.all_gather_into_tensor(gathered, shard)
            return x @ gathered.t()
        t_fused = timed(lambda: w.matmul(x), dev)
        rec = dict(case="allgather->gemm", M=M, N=N, K=K, n_gpus=world, fused_ms=t_fused, nccl_allgather_plus_cublas_ms=timed(baseline, dev),
                   own_gemm_only_ms=timed(lambda: gemm.gemm_tn(x, w.full), dev), cublas_only_ms=timed(lambda: x @ gathered.t(), dev),
                   roofline=roofline.fraction(t_fused, flops=2.0 * M * N * K, nvlink_bytes=(world - 1) / world * N * K * 2))
        gemm.check(dev)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        del w
    for (M, N, K) in [(16384, 2048, 5504 // world // 8 * 8), (16384, 8192, 2048)]:
        op = ReduceScatterGemm(M, N, dev)
        a = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
        b = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        full = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        outb = torch.empty(M // world, N, dtype=torch.bfloat16, device=dev)

        def baseline_rs():
            torch.matmul(a, b.t(), out=full)
            dist.reduce_scatter_tensor(outb, full)
        t_fused = timed(lambda: op(a, b), dev)
        rec = dict(case="gemm->reducescatter", M=M, N=N, K_per_rank=K, n_gpus=world, fused_ms=t_fused,
                   cublas_plus_nccl_reducescatter_ms=timed(baseline_rs, dev), own_gemm_only_ms=timed(lambda: gemm.gemm_tn(a, b), dev),
                   cublas_only_ms=timed(lambda: torch.matmul(a, b.t(), out=full), dev),
                   roofline=roofline.fraction(t_fused, flops=2.0 * M * N * K, nvlink_bytes=(world - 1) / world * M * N * 2))
        gemm.check(dev)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        del op
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
