"""Worker run by the multi-process tests (one process per rank; gloo on CPU, nccl on GPUs)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_problem(seed=0, n=64):
    from supergrok15_b200.models import Transformer
    torch.manual_seed(seed)
    m = Transformer(1, 32, 2)
    x = torch.randint(0, 97, (n, 4))
    y = torch.randint(0, 97, (n,))
    return m, x, y


def run(rank, world, port, optimizer, out_path, device, comm, steps, dtype):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    if device == "cuda":
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        dev = torch.device("cuda", rank)
    else:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")
    from supergrok15_b200.parallel import ZeroEngine
    m, x, y = make_problem()
    # "adamw+overlap": the sharded step is issued bucket by bucket from gradient hooks (several buckets on this small model);
    # "adamw+overlap2": the same with two micro-batches (only the last backward pass issues buckets)
    optimizer, _, flag = optimizer.partition("+")
    eng = ZeroEngine(m.to(dev), optimizer, OPT_KW.get(optimizer, {}), comm=comm, param_dtype=dtype, timeout_s=10.0,
                     overlap=flag.startswith("overlap"), bucket_numel=3000)
    per = x.shape[0] // world
    xs, ys = x[rank * per:(rank + 1) * per].to(dev), y[rank * per:(rank + 1) * per].to(dev)
    losses = []
    for _ in range(steps):
        losses.append(float(eng.train_step(xs, ys, micro_batches=2 if flag == "overlap2" else 1)))
    if dev.type == "cuda":
        eng.check()
    flat = torch.cat([p.detach().float().reshape(-1).cpu() for p in eng.params])
    gathered = [torch.zeros_like(flat) for _ in range(world)] if rank == 0 else None
    if device == "cuda":
        fl = flat.to(dev)
        gl = [torch.zeros_like(fl) for _ in range(world)]
        dist.all_gather(gl, fl)
        gathered = [g.cpu() for g in gl]
    else:
        dist.gather(flat, gathered, dst=0)
    if rank == 0:
        torch.save({"params": gathered, "losses": losses, "owner": eng.owner, "buckets": len(eng.buckets), "graphs": len(eng._graphs),
                    "device_step": bool(getattr(eng, "device_step", False))}, out_path)
    dist.barrier()
    dist.destroy_process_group()


# eps is large on purpose: with the default 1e-8 the first Adam steps are sign-like and amplify fp32 rounding differences
# between "mean of two half-batch gradients" and "full-batch gradient" far beyond any useful tolerance
OPT_KW = {"supergrok2": dict(warmup_steps=0, warmup_ramp=1, eps=1e-3), "grokadamw": dict(grad_clip=0.05, eps=1e-3),
          "supergrok15": dict(gradient_clipping=0.05, eps=1e-3), "adamw": dict(lr=1e-2, weight_decay=0.1, eps=1e-3),
          "lion": dict(lr=1e-3)}


def reference_run(optimizer, steps, device="cpu", dtype=torch.float32):
    """Single process, full batch, the plain (unsharded) optimizer on fp32 parameters."""
    from supergrok15_b200 import optim as O
    from supergrok15_b200.parallel.engine import OPTIMIZERS
    m, x, y = make_problem()
    m = m.to(device)
    x, y = x.to(device), y.to(device)
    cls = OPTIMIZERS[optimizer]
    kw = OPT_KW.get(optimizer, {})
    if optimizer == "muon":
        opt = cls([p for p in m.parameters() if p.dim() == 2], [p for p in m.parameters() if p.dim() != 2], **kw)
    else:
        opt = cls(m.parameters(), **kw)
    for _ in range(steps):
        opt.zero_grad()
        F.cross_entropy(m(x), y).backward()
        opt.step()
    return torch.cat([p.detach().float().reshape(-1).cpu() for p in m.parameters()])


if __name__ == "__main__":
    rank, world, port, optimizer, out_path, device, comm, steps, dtype = sys.argv[1:10]
    run(int(rank), int(world), int(port), optimizer, out_path, device, comm, int(steps),
        {"f32": torch.float32, "bf16": torch.bfloat16}[dtype])
