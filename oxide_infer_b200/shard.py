"""Partition of independent sequences across the GPUs of one box (replicas, no collective).

Sequences own their KV cache, conv state and table rows, so a decode step never exchanges
data between GPUs; the only multi-GPU decision is which GPU serves which sequence.  The
reference runs one GPU only (its engine opens device 0, server.rs:212); this is the
host-side policy the 8-GPU serving mix uses."""
from __future__ import annotations

from typing import List, Sequence


def assign_sequences(seq_lens: Sequence[int], world_size: int) -> List[List[int]]:
    """Longest-processing-time assignment: sequences sorted by length (descending, ties by
    index) go one by one to the rank with the fewest keys so far (ties to the lowest rank,
    then to the rank with fewer sequences).  Deterministic, so every rank computes the same
    partition from the same lengths without communicating.  Returns, per rank, the indices
    of its sequences in ascending order."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i))
    load = [0] * world_size
    count = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (load[j], count[j], j))
        out[r].append(i)
        load[r] += int(seq_lens[i])
        count[r] += 1
    return [sorted(x) for x in out]


def shard_keys(seq_lens: Sequence[int], parts: List[List[int]]) -> List[int]:
    """Total keys (the HBM-traffic proxy of a decode step) per rank."""
    return [sum(int(seq_lens[i]) for i in p) for p in parts]
