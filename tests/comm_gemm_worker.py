"""One rank of the fused all-gather / reduce-scatter GEMM test: argv = rank world port out_path."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, port, out_path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from supergrok15_b200.ops import gemm
    from supergrok15_b200.parallel.comm_gemm import ShardedWeight
    res = {}
    for (M, N, K) in [(512, 1024, 512), (1000, 2048, 1024)]:
        w = ShardedWeight(N, K, dev)
        errs = []
        for call in range(2):                                    # second call: new shard contents, same counters (epoch 2)
            g = torch.Generator(device="cpu").manual_seed(100 * call + 7)
            w_full = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
            x = (torch.randn(M, K, generator=torch.Generator().manual_seed(rank + 10 * call)) * 0.5).to(torch.bfloat16).to(dev)
            w.full.fill_(float("nan"))                            # gather space must be overwritten by the kernel
            w.shard.copy_(w_full[rank * w.rows:(rank + 1) * w.rows].to(dev))
            torch.cuda.synchronize()
            dist.barrier()
            y = w.matmul(x)
            torch.cuda.synchronize()
            gemm.check(dev)
            ref = x.float() @ w_full.to(dev).float().t()
            errs.append(float((y.float() - ref).abs().max() / ref.abs().max()))
            assert torch.equal(w.full.cpu(), w_full), "gathered weight differs"
            dist.barrier()
        res[(M, N, K)] = errs
        del w
    from supergrok15_b200.parallel.comm_gemm import ReduceScatterGemm
    for (M, N, K) in [(256 * world, 512, 256), (1024 * world, 1024 + 64, 512)]:
        op = ReduceScatterGemm(M, N, dev)
        errs = []
        for call in range(3):                                    # three calls: both parities and the reuse of the first
            gen = torch.Generator().manual_seed(1000 * call + rank)
            a = (torch.randn(M, K, generator=gen) * 0.5).to(torch.bfloat16).to(dev)
            b = (torch.randn(N, K, generator=gen) * 0.05).to(torch.bfloat16).to(dev)
            y = op(a, b)
            torch.cuda.synchronize()
            gemm.check(dev)
            part = (a.float() @ b.float().t()).to(torch.bfloat16).float()        # partials travel as bf16
            dist.all_reduce(part)
            mloc = M // world
            ref = part[rank * mloc:(rank + 1) * mloc]
            errs.append(float((y.float() - ref).abs().max() / ref.abs().max()))
        res[("rs", M, N, K)] = errs
        del op
    if rank == 0:
        torch.save(res, out_path)
        print(res)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
