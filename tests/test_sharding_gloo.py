"""CPU-only, world_size 2 over gloo: the host logic of the batch-sharded multi-GPU path
(shard ownership, max-over-ranks timing, result gather)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from munet_b200.sharding import gather_shards, max_over_ranks, shard_bounds


def test_shard_bounds_cover_and_balance():
    for n in (0, 1, 7, 64, 65):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _worker(rank, world, port, n_items, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lo, hi = shard_bounds(n_items, rank, world)
        # each rank "runs" its own sequences: result row i is a function of the global index only
        local = torch.arange(lo, hi, dtype=torch.int32).unsqueeze(1) * torch.tensor([[1, 10]], dtype=torch.int32)
        full = gather_shards(local, n_items)
        slow = max_over_ranks(5.0 + rank)  # whole-job time is the slowest rank's
        if rank == 0:
            out.put((full.tolist(), slow))
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    n_items = 7  # ragged: 4 + 3
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_items, q)) for r in range(2)]
    for p in procs:
        p.start()
    full, slow = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert full == [[i, 10 * i] for i in range(n_items)]
    assert slow == 6.0
