"""Multi-GPU host logic on CPU: two gloo ranks partition the serving mix without
exchanging data on the decode path, and their shards form an exact, balanced cover."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oxide_infer_b200.shard import assign_sequences, shard_keys


def _lens(n=1024, seed=0):
    rng = np.random.default_rng(seed)
    return np.clip(np.round(np.exp(rng.normal(np.log(2048), 1.0, n))), 16, 32768 - 64).astype(np.int64)


def test_assignment_is_exact_cover_and_balanced():
    lens = _lens()
    for world in (1, 2, 4, 8):
        parts = assign_sequences(lens, world)
        flat = sorted(i for p in parts for i in p)
        assert flat == list(range(len(lens)))
        keys = shard_keys(lens, parts)
        assert max(keys) - min(keys) <= lens.max()          # LPT bound
        assert max(keys) <= 1.02 * sum(keys) / world or world == 1
    assert assign_sequences([], 4) == [[], [], [], []]
    assert assign_sequences([5, 5, 5], 2) == [[0, 2], [1]]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens = _lens()
        mine = assign_sequences(lens, world)[rank]          # computed locally, no communication
        # a replica's "step": touch only its own sequences (stand-in for the per-rank decode step)
        local_keys = torch.tensor([int(lens[mine].sum()), len(mine)], dtype=torch.int64)
        gathered = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, local_keys)               # measurement plumbing only
        owned = torch.zeros(len(lens), dtype=torch.int64)
        owned[mine] = 1
        dist.all_reduce(owned)
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)            # the bench's max-over-ranks of the time
        if rank == 0:
            q.put((bool((owned == 1).all()), [g.tolist() for g in gathered], float(t)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_partition_without_overlap():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok, gathered, tmax = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok
    assert sum(g[1] for g in gathered) == 1024
    k0, k1 = gathered[0][0], gathered[1][0]
    assert abs(k0 - k1) <= 32768
    assert tmax == 2.0
