"""Worker of the row-sharded Newton-Schulz test: one process per GPU; every rank holds its row block of each matrix."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = [(2048, 1024), (1024, 1024), (512, 1280)]


def main():
    rank, world, port, out_path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from supergrok15_b200.ops import gemm, oracle
    from supergrok15_b200.ops.muon_sharded import RowShardedNewtonSchulz
    g = torch.Generator().manual_seed(7)
    full = []
    for R, C in SHAPES:
        X = torch.randn(R, C, generator=g)
        full.append((X / (X.norm() + 1e-7)).to(dev))
    ns = RowShardedNewtonSchulz(SHAPES, dev)
    res = {}
    for rep in range(4):                                  # two eager calls, the capture of the whole step into one CUDA graph, one replay
        shards = [X[rank * (X.shape[0] // world):(rank + 1) * (X.shape[0] // world)].contiguous() for X in full]
        outs = ns.run(shards, 5)
        torch.cuda.synchronize()
        gemm.check(dev)
        for (R, C), X, o in zip(SHAPES, full, outs):
            parts = [torch.empty_like(o) for _ in range(world)]
            dist.all_gather(parts, o.contiguous())
            got = torch.cat(parts, 0)
            ref = oracle.newton_schulz(X.double(), 5).float()
            whole = gemm.newton_schulz(X, 5, oracle.NS_COEFFS)
            k = min(R, C)
            Q = got @ got.t() if R <= C else got.t() @ got
            Qr = ref @ ref.t() if R <= C else ref.t() @ ref
            res[f"{R}x{C}/{rep}"] = {"rel_vs_fp32": float((got - ref).norm() / ref.norm()), "orth_vs_fp32": float((Q - Qr).norm() / k ** 0.5),
                                     "rel_vs_whole_bf16": float((got - whole).norm() / whole.norm())}
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
