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
    """owner[i] for every tensor; deterministic (ties broken by index, then by lowest rank), so every rank computes the same map.
    Longest-processing-time greedy first, then a local search: while it lowers the largest load, move one tensor off the
    heaviest rank or swap one of its tensors with a smaller one of another rank.  The sharded step ends at a barrier, so the
    heaviest rank sets its duration; greedy alone leaves e.g. 2.62 M of 19.0 M elements on one of eight ranks (mean 2.38 M) for the
    6-layer d512 decoder, the search brings that to 2.42 M."""
    n = [int(x) for x in numels]
    order = sorted(range(len(n)), key=lambda i: (-n[i], i))
    load = [0] * world
    owner = [0] * len(n)
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += n[i]
    for _ in range(4 * len(n) + 16):                    # every accepted step lowers (max load, number of ranks at max): terminates
        hi = max(range(world), key=lambda k: (load[k], -k))
        best = None                                       # (new pair maximum, i, j or -1, target rank)
        for i in order:
            if owner[i] != hi:
                continue
            for r in range(world):
                if r == hi:
                    continue
                cand = max(load[hi] - n[i], load[r] + n[i])                     # move i to r
                if cand < load[hi] and (best is None or cand < best[0]):
                    best = (cand, i, -1, r)
            for j in order:
                r = owner[j]
                if r == hi or n[j] >= n[i]:
                    continue
                d = n[i] - n[j]
                cand = max(load[hi] - d, load[r] + d)                           # swap i (heaviest rank) with the smaller j of rank r
                if cand < load[hi] and (best is None or cand < best[0]):
                    best = (cand, i, j, r)
        if best is None:
            break
        _, i, j, r = best
        owner[i] = r
        load[hi] -= n[i]
        load[r] += n[i]
        if j >= 0:
            owner[j] = hi
            load[r] -= n[j]
            load[hi] += n[j]
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
