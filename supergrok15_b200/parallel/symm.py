"""Symmetric (peer-mapped) buffers for the in-kernel collectives.

On CUDA with an initialised NCCL process group the buffers come from PyTorch's symmetric-memory allocator
(CUDA VMM allocations whose handles are exchanged over the process group's store); the rendezvous yields
the address of every peer's copy in this process's address space and, when the GPUs sit behind an
NVSwitch with NVLS, one multicast address.  ``torch.distributed`` is used for this bootstrap only; the
hot path issues no NCCL call.  With a world of one (or no process group) a buffer is ordinary device
memory and the peer table has a single entry.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass
class SymmBuffer:
    tensor: torch.Tensor            # the local copy
    peer_ptrs: List[int]            # address of rank r's copy, as seen from this process
    multicast_ptr: int              # NVLS multicast address, 0 if unavailable
    rank: int
    world: int
    handle: object = None           # keeps the rendezvous alive


def world_info(group=None):
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def alloc(numel: int, dtype: torch.dtype, device, group=None, zero: bool = True) -> SymmBuffer:
    rank, world = world_info(group)
    if world == 1 or torch.device(device).type != "cuda":
        t = torch.zeros(numel, dtype=dtype, device=device) if zero else torch.empty(numel, dtype=dtype, device=device)
        return SymmBuffer(t, [t.data_ptr()], 0, 0, 1)
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    t = symm_mem.empty(numel, dtype=dtype, device=device)
    if zero:
        t.zero_()
    gname = (group or dist.group.WORLD).group_name
    try:
        hdl = symm_mem.rendezvous(t, group=gname)
    except Exception:  # noqa: BLE001  (older API wants the group enabled first)
        symm_mem.enable_symm_mem_for_group(gname)
        hdl = symm_mem.rendezvous(t, group=gname)
    mc = 0
    try:
        mc = int(hdl.multicast_ptr or 0)
    except Exception:  # noqa: BLE001
        mc = 0
    torch.cuda.synchronize()
    dist.barrier(group)             # every copy is zeroed before anybody touches a peer
    return SymmBuffer(t, [int(p) for p in hdl.buffer_ptrs], mc, rank, world, hdl)
