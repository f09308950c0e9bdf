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


# ----------------------------------------------------------------------------- expert parallel
def _ep_exchange_job(rank, world):
    """The exchange arithmetic of the expert-parallel layer, run for real over gloo with CPU
    tensors: every row must reach the rank that owns its expert, arrive grouped by expert
    after `gather_idx`, and come home to its original position."""
    import numpy as np
    from complexity_deep_b200.expert_parallel import exchange_plan
    from oracle import complexity_oracle as oracle
    E, El, V, T = 8, 4, 200, 300 + 50 * rank
    table = oracle.build_token_mapping(V, E, oracle.zipf_probabilities(V, 1.0).float())
    ids = oracle.zipf_token_ids(V, 1.0, T, seed=10 + rank).numpy()
    eid, counts, offsets, perm, inv = oracle.route(ids, table, E)
    all_counts = [torch.empty(E, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(all_counts, torch.from_numpy(counts))
    plan = exchange_plan(torch.stack(all_counts).numpy(), rank, El)
    assert sum(plan.in_splits) == T
    # payload: (home rank, original row, expert id) per row, in expert-sorted order
    rows = torch.tensor([[rank, int(r), int(eid[r])] for r in perm], dtype=torch.int64)
    recv = torch.empty(plan.received, 3, dtype=torch.int64)
    dist.all_to_all_single(recv, rows, plan.out_splits, plan.in_splits)
    grouped = recv[torch.from_numpy(plan.gather_idx).long()]
    # every received row belongs to one of my experts, grouped by expert in segment order
    for e in range(El):
        seg = grouped[plan.seg_offsets[e]:plan.seg_offsets[e + 1]]
        assert bool((seg[:, 2] == rank * El + e).all())
        assert bool((seg[1:, 0] >= seg[:-1, 0]).all())             # source-minor order
    # "expert output" = payload tagged; scatter back to receive order with the same map
    back = torch.empty_like(grouped)
    back[torch.from_numpy(plan.gather_idx).long()] = grouped + torch.tensor([0, 0, 100])
    home = torch.empty(T, 3, dtype=torch.int64)
    dist.all_to_all_single(home, back, plan.in_splits, plan.out_splits)
    assert bool((home[:, 0] == rank).all())
    assert home[:, 1].tolist() == perm.tolist()                    # sorted order preserved
    assert home[:, 2].tolist() == [int(eid[r]) + 100 for r in perm]
    return plan.received


def test_expert_parallel_exchange_plan_two_ranks():
    got = run_ranks(_ep_exchange_job, port=29612)
    assert sum(got) == 300 + 350                                   # nothing lost, nothing padded


def test_exchange_plan_rejects_uneven_split_and_handles_empty():
    import numpy as np
    import pytest
    from complexity_deep_b200.expert_parallel import exchange_plan
    with pytest.raises(ValueError):
        exchange_plan(np.zeros((2, 6)), 0, 4)
    plan = exchange_plan(np.array([[0, 0, 5, 0], [0, 0, 0, 2]]), 0, 2)   # rank 0 receives nothing
    assert plan.received == 0 and plan.out_splits == [0, 0] and plan.in_splits == [0, 5]
    assert plan.seg_offsets.tolist() == [0, 0, 0]
    plan1 = exchange_plan(np.array([[0, 0, 5, 0], [0, 0, 0, 2]]), 1, 2)
    assert plan1.received == 7 and plan1.seg_offsets.tolist() == [0, 5, 7]
    assert plan1.gather_idx.tolist() == [0, 1, 2, 3, 4, 5, 6]


def test_balanced_placement_spreads_heavy_experts():
    from complexity_deep_b200.expert_parallel import balanced_placement
    load = [8.3, 4.1] + [2.9] * 30                       # Zipf(1.0) over 32 experts
    order = balanced_placement(load, 8)
    assert sorted(order) == list(range(32))
    per_rank = [sum(load[e] for e in order[r * 4:(r + 1) * 4]) for r in range(8)]
    assert max(per_rank) <= 8.3 + 3 * 2.9 + 1e-9          # the heaviest expert sits with light ones
    contiguous = [sum(load[r * 4:(r + 1) * 4]) for r in range(8)]
    assert max(per_rank) < max(contiguous)
    owner = {e: i // 4 for i, e in enumerate(order)}
    assert owner[0] != owner[1]                          # the two heaviest are on different ranks
    assert balanced_placement([1.0] * 8, 2) == [0, 2, 4, 6, 1, 3, 5, 7]


def test_push_plan_addresses_cover_every_row_exactly_once():
    """Peer-store exchange arithmetic, all ranks simulated on the host: every (source, sorted
    row) is written to a distinct slot of its expert owner's buffer inside that expert's
    segment, and every received row is sent back to the slot it came from."""
    import numpy as np
    from complexity_deep_b200.expert_parallel import push_plan
    rng = np.random.default_rng(0)
    G, El, H = 4, 2, 16
    E = G * El
    counts = rng.integers(0, 7, size=(G, E))
    counts[2, 3] = 0
    ret_base = [1000000 * (i + 1) for i in range(G)]
    plans = [push_plan(counts, r, El, ret_base, H * 2) for r in range(G)]
    recv = [dict() for _ in range(G)]                    # owner -> {row: (source, expert, k)}
    for src in range(G):
        push_base = plans[src][0]
        for e in range(E):
            owner = e // El
            for k in range(counts[src, e]):
                row = int(push_base[e]) + k
                assert row not in recv[owner]
                recv[owner][row] = (src, e, k)
    for r in range(G):
        _, seg, received, row_ptrs = plans[r]
        assert received == len(recv[r]) == counts[:, r * El:(r + 1) * El].sum()
        assert sorted(recv[r]) == list(range(received))  # dense, no holes
        home_off = np.concatenate([np.zeros((G, 1), np.int64), np.cumsum(counts, 1)[:, :-1]], 1)
        seen = set()
        for row in range(received):
            src, e, k = recv[r][row]
            assert seg[e - r * El] <= row < seg[e - r * El + 1]        # inside its expert's segment
            want = ret_base[src] + (home_off[src, e] + k) * H * 2       # its sorted slot at home
            assert int(row_ptrs[row]) == want
            seen.add(want)
        assert len(seen) == received


def test_device_side_push_plan_equals_host_plan():
    """The tensor-op plan (run on the device in production, no host copy) gives the same
    numbers as the host arithmetic, for every rank."""
    import numpy as np
    from complexity_deep_b200.expert_parallel import push_plan, push_plan_tensors
    rng = np.random.default_rng(1)
    G, El, H = 4, 3, 32
    counts = rng.integers(0, 9, size=(G, G * El))
    counts[1, 4] = 0
    counts[:, 7] = 0                                       # an expert nobody uses
    ret_base = [7000000 * (i + 1) for i in range(G)]
    for r in range(G):
        pb, seg, received, ptrs = push_plan(counts, r, El, ret_base, H * 2)
        tpb, tseg, tptrs = push_plan_tensors(torch.from_numpy(counts).int(), r, El,
                                             torch.tensor(ret_base), H * 2, received + 5)
        assert tpb.dtype == torch.int32 and tseg.dtype == torch.int32 and tptrs.dtype == torch.int64
        assert np.array_equal(tpb.numpy(), pb) and np.array_equal(tseg.numpy(), seg)
        assert np.array_equal(tptrs.numpy()[:received], ptrs)
