"""Worker of the Llama-style engine tests: a small decoder trained for a few steps, one process per GPU.
argv: rank world port out_path mode steps, mode one of
  muon/rows, muon/tensors   Muon with the block matrices split by rows over the ranks / owned whole by one rank each
  adamw/gemm, adamw/push    AdamW with the parameter all-gather inside the first consuming GEMM / pushed at the end of the step
Rank 0 saves every rank's final parameters."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, port, out_path, mode, steps = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5], int(sys.argv[6])
    optimizer, variant = mode.split("/")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    from supergrok15_b200.models.llama import Llama, LlamaConfig
    from supergrok15_b200.parallel import ZeroEngine
    cfg = LlamaConfig(n_layers=1, d_model=256, n_heads=4, d_ff=512, vocab=512, max_seq=64)
    torch.manual_seed(0)
    model = Llama(cfg).to(dev)
    init = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()]).cpu()
    if optimizer == "muon":
        eng = ZeroEngine(model, "muon", dict(lr=0.02, momentum=0.95, weight_decay=0.01, adamw_lr=1e-3, adamw_names=("embed", "lm_head"),
                                             sharding=variant), comm="p2p", param_dtype=torch.bfloat16, graph=False)
    else:
        eng = ZeroEngine(model, "adamw", dict(lr=3e-3, weight_decay=0.01), comm="p2p", param_dtype=torch.bfloat16, graph=False, gather=variant)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab, (8 * world, 33), generator=g)[rank * 8:(rank + 1) * 8].to(dev)
    losses = []
    for _ in range(steps):
        losses.append(float(eng.train_step(ids[:, :-1].contiguous(), ids[:, 1:].contiguous())))
    eng.gather_params()
    eng.check()
    from supergrok15_b200.ops import gemm
    gemm.check(dev)
    flat = torch.cat([p.detach().float().reshape(-1) for p in eng.params])
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat)
    if rank == 0:
        torch.save({"params": [p.cpu() for p in parts], "init": init, "losses": losses, "row_sharded": len(getattr(eng, "rs_idx", [])),
                    "gathered_in_gemm": len(eng.gw_idx)}, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
