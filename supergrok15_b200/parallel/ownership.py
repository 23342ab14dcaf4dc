"""Who owns what under ZeRO sharding.  Pure functions of (tensor sizes, world size): every rank computes the
same map without communicating, and a checkpoint can be re-sharded to another world size at load time.

* tensor-granular (SuperGrok v2, v1.1, v1.5, Muon, ...): whole tensors are assigned by greedy
  longest-processing-time bin packing on numel.  The per-tensor sort / scan / GRU state of v2 and the
  2-D semantics of Muon stay local to one rank.
* flat-range (AdamW, Lion): the flat buffer is cut into equal ranges of a multiple of 8 elements.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def assign_tensors(numels: Sequence[int], world: int) -> List[int]:
    """owner[i] for every tensor; deterministic (ties broken by index, then by lowest rank)."""
    order = sorted(range(len(numels)), key=lambda i: (-int(numels[i]), i))
    load = [0] * world
    owner = [0] * len(numels)
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += int(numels[i])
    return owner


def imbalance(numels: Sequence[int], owner: Sequence[int], world: int) -> float:
    """max load / mean load (1.0 = perfect)."""
    load = [0] * world
    for n, o in zip(numels, owner):
        load[o] += int(n)
    mean = sum(load) / world
    return max(load) / mean if mean else 1.0


def flat_ranges(total: int, world: int, align: int = 8) -> List[Tuple[int, int]]:
    """[begin, end) of every rank in a flat buffer of ``total`` elements (already padded to world*align)."""
    per = -(-total // (world * align)) * align
    return [(min(r * per, total), min((r + 1) * per, total)) for r in range(world)]


def grouped_layout(numels: Sequence[int], owner: Sequence[int], world: int, align: int = 8):
    """Flat-buffer layout with the tensors of each owner contiguous: returns (offset per tensor,
    (begin, end) of every owner's region, total length).  Offsets are multiples of ``align`` elements."""
    offsets = [0] * len(numels)
    regions = []
    pos = 0
    for r in range(world):
        begin = pos
        for i, n in enumerate(numels):
            if owner[i] == r:
                offsets[i] = pos
                pos += -(-int(n) // align) * align
        regions.append((begin, pos))
    return offsets, regions, pos


def reverse_buckets(offsets: Sequence[int], numels: Sequence[int], bucket_numel: int, align: int = 8):
    """Buckets of consecutive parameters for overlapping the sharded step with backward: [(lo, hi, [tensor indices])].

    Backward produces the gradients of the last parameters first, so bucket 0 holds the LAST parameters of the flat buffer.
    A bucket is closed once it holds at least ``bucket_numel`` elements; [lo, hi) is its range of the flat buffer (``offsets``
    are the aligned flat offsets of the tensors, in parameter order)."""
    out, cur, hi = [], [], None
    for i in range(len(numels) - 1, -1, -1):
        end = int(offsets[i]) + -(-int(numels[i]) // align) * align
        if hi is None:
            hi = end
        cur.append(i)
        if hi - int(offsets[i]) >= bucket_numel or i == 0:
            out.append((int(offsets[i]), hi, cur))
            cur, hi = [], None
    return out


def bucket_slices(lo: int, hi: int, world: int, align: int = 8) -> List[Tuple[int, int]]:
    """Every rank's [begin, end) of the flat range [lo, hi): equal slices of a multiple of ``align`` elements (the last may be short or empty)."""
    per = -(-(hi - lo) // (world * align)) * align
    return [(min(lo + r * per, hi), min(lo + (r + 1) * per, hi)) for r in range(world)]
