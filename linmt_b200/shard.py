"""Sentence sharding across the GPUs of one box.

Sentences are independent (src/decoder.h:1780-1840 keeps no state between calls), so the
only multi-GPU structure is: split the work, decode locally on a replica, gather the
hypotheses once at the end.  No collective runs inside the step loop.
"""
from __future__ import annotations

from typing import Dict, List


def batches_by_length(sents, batch: int) -> List[List[int]]:
    """Sentence indices sorted by step count (longest first) and cut into batches, so the
    sentences of a batch need similar numbers of steps."""
    order = sorted(range(sents.n), key=lambda i: (-int(sents.steps[i]), i))
    return [order[i:i + batch] for i in range(0, len(order), batch)]


def partition(sents, world: int, batch: int) -> List[List[int]]:
    """Deals length-bucketed batches to ranks, heaviest first, always to the least loaded rank
    (load of a batch = its longest sentence's decoder forwards, max T_i + 1, times its rows: a batch
    runs as long as its longest member)."""
    bl = batches_by_length(sents, batch)
    cost = [(max(int(sents.steps[i]) for i in b) + 1) * len(b) for b in bl]
    load = [0] * world
    parts: List[List[int]] = [[] for _ in range(world)]
    for bi in sorted(range(len(bl)), key=lambda j: -cost[j]):
        r = min(range(world), key=lambda x: (load[x], x))
        parts[r].extend(bl[bi])
        load[r] += cost[bi]
    return parts


def gather_results(local: Dict[int, object], dst: int = 0):
    """One gather of the per-sentence results to rank ``dst`` (the only collective of a job)."""
    parts = gather_parts(local, dst)
    if parts is None:
        return None
    merged = {}
    for part in parts:
        merged.update(part)
    return merged


def gather_parts(local, dst: int = 0):
    """The same gather for any picklable per-rank result (e.g. a tuple of numpy arrays: sentence indices,
    padded token rows, lengths, scores): the list of every rank's part on rank ``dst``, None elsewhere."""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return [local]
    out = [None] * dist.get_world_size() if dist.get_rank() == dst else None
    dist.gather_object(local, out, dst=dst)
    return out if dist.get_rank() == dst else None
