"""Host logic of the N > 1 paths with two gloo ranks on the CPU: data-parallel batch
sharding and the max-over-ranks timing used by bench.py."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, fn, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def run_ranks(fn, world=2, port=29611):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, fn, out), nprocs=world, join=True)
    return [out[r] for r in range(world)]


def _dp_job(rank, world):
    import bench
    lo, hi = bench.shard_batch(32, world, rank)
    ids = torch.arange(32 * 4).view(32, 4)[lo:hi]            # this rank's sequences
    gathered = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(gathered, ids)
    ms = bench.aggregate_ms(10.0 + 5.0 * rank, dist)         # slowest rank defines the step
    return (lo, hi, torch.cat(gathered).flatten().tolist(), ms)


def test_data_parallel_sharding_and_timing():
    res = run_ranks(_dp_job)
    assert [(r[0], r[1]) for r in res] == [(0, 16), (16, 32)]
    assert res[0][2] == list(range(128))                     # shards tile the batch exactly
    assert res[0][3] == res[1][3] == 15.0


def test_shard_batch_uneven():
    import bench
    parts = [bench.shard_batch(10, 4, r) for r in range(4)]
    assert parts == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [bench.shard_batch(32, 8, r) for r in range(8)] == [(4 * r, 4 * r + 4) for r in range(8)]
