"""The multi-GPU host logic (batch sharding, max-over-ranks timing, final gather) on CPU ranks
over gloo, world size 2; the per-rank compute is the oracle standing in for the GPU operator."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gtr_b200.sharding import shard_range


def test_shard_ranges_partition_exactly():
    for total in (0, 1, 7, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, fail_rank, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gtr_b200.sharding import gather_batch, max_over_ranks
        from oracle import c_oracle, gla_ref
        q, k, v, g = gla_ref.make_inputs(total, 96, 2, seed=3, dtype=torch.float32)   # same inputs on every rank
        lo, hi = shard_range(total, rank, world)
        if rank == fail_rank:
            hi = lo                                      # a rank that lost its shard
        o, _ = c_oracle.forward(q[lo:hi], k[lo:hi], v[lo:hi], g[lo:hi])
        slowest = max_over_ranks(10.0 + rank)
        try:
            parts = gather_batch(o, total)
            full = torch.cat(parts)
            ref, _ = c_oracle.forward(q, k, v, g)
            out[rank] = ("ok", slowest, bool(torch.equal(full, ref)))
        except RuntimeError as e:
            out[rank] = ("error", slowest, str(e))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total,fail_rank", [(4, -1), (5, -1), (4, 1)])
def test_two_ranks_shard_and_gather(total, fail_rank):
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), total, fail_rank, out), nprocs=world, join=True)
    assert len(out) == world
    for rank in range(world):
        status, slowest, payload = out[rank]
        assert slowest == 11.0                           # max over ranks of 10 + rank
        if fail_rank < 0:
            assert status == "ok" and payload is True
        else:
            assert status == "error" and f"[{fail_rank}]" in payload
