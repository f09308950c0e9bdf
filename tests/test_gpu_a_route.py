"""D1 dispatch kernels through the C ABI vs the oracle: bit-exact expert ids, histogram,
offsets, stable permutation and its inverse."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import complexity_oracle as oracle

pytestmark = pytest.mark.gpu


def _run(ids_np, table_np, E):
    from complexity_deep_b200 import ops
    ids = torch.from_numpy(np.asarray(ids_np, dtype=np.int64)).cuda()
    table = torch.from_numpy(np.asarray(table_np, dtype=np.int64)).cuda()
    r = ops.route(ids, table, E)
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in (r.expert_ids, r.counts, r.offsets, r.perm, r.inv_perm)]


def _check(ids_np, table_np, E):
    got = _run(ids_np, table_np, E)
    want = oracle.route(np.asarray(ids_np), np.asarray(table_np, dtype=np.int64), E)
    for name, g, w in zip(["expert_ids", "counts", "offsets", "perm", "inv_perm"], got, want):
        assert g.dtype == np.int32
        assert np.array_equal(g, w), name
    return got


def test_golden_zipf_batch():
    g = np.load(os.path.join(GOLDEN, "routing.npz"))
    eid, counts, offsets, perm, inv = _check(g["ids"], g["table_e8"], 8)
    assert np.array_equal(eid, g["expert_ids"])
    assert np.array_equal(counts, g["counts"])
    assert np.array_equal(perm, g["perm"])


@pytest.mark.parametrize("T", [1, 31, 32, 33, 255, 2047, 2048, 2049, 5000, 65536])
@pytest.mark.parametrize("E", [1, 4, 8, 32])
def test_ragged_sizes_modulo_and_binpacked(T, E):
    V = 1000
    rng = np.random.default_rng(T * 131 + E)
    ids = rng.integers(-50, V + 50, size=T)          # includes ids that must be clamped
    _check(ids, np.arange(V) % E, E)
    table = oracle.build_token_mapping(V, E, oracle.zipf_probabilities(V, 1.1).float())
    _check(ids, table, E)


def test_empty_batch_and_empty_experts():
    got = _run(np.zeros(0, np.int64), np.arange(16) % 4, 4)
    assert got[1].tolist() == [0, 0, 0, 0] and got[2].tolist() == [0, 0, 0, 0, 0]
    # every token on one expert: all other segments are empty
    _check(np.full(3000, 7), np.arange(16) % 8, 8)
    # 256 experts (the library's maximum)
    rng = np.random.default_rng(0)
    _check(rng.integers(0, 4096, size=10000), np.arange(4096) % 256, 256)


def test_full_size_config5_properties():
    """The expert-parallel layer's size (T=65536, V=100000, E=32): compared with the oracle and through
    size-independent properties (permutation validity, sortedness, stability)."""
    V, E, T = 100000, 32, 65536
    ids = oracle.zipf_token_ids(V, 1.0, T).numpy()
    table = oracle.build_token_mapping(V, E, oracle.zipf_probabilities(V, 1.0).float())
    eid, counts, offsets, perm, inv = _check(ids, table, E)
    assert np.array_equal(np.sort(perm), np.arange(T))
    sorted_e = eid[perm]
    assert np.all(np.diff(sorted_e) >= 0)
    same = np.diff(sorted_e) == 0
    assert np.all(np.diff(perm)[same] > 0)            # stable: ascending rows inside a segment
    assert counts.sum() == T and offsets[-1] == T


def test_deterministic_bytes():
    ids = oracle.zipf_token_ids(32000, 1.1, 50000).numpy()
    table = np.arange(32000) % 8
    a = _run(ids, table, 8)
    b = _run(ids, table, 8)
    for x, y in zip(a, b):
        assert x.tobytes() == y.tobytes()


@pytest.mark.parametrize("G,El,seed", [(4, 3, 1), (8, 4, 2), (2, 16, 3), (1, 8, 4), (8, 1, 5)])
def test_ep_plan_kernel_equals_host_plan(G, El, seed):
    """cd_ep_plan (one launch on the device) against the host arithmetic of the same plan, for
    every rank: push bases, segment offsets and the return address of every received row are the
    same integers; entries past the received rows follow the documented rule (last block)."""
    import numpy as np
    from complexity_deep_b200 import ops
    from complexity_deep_b200.expert_parallel import push_plan, push_plan_tensors
    rng = np.random.default_rng(seed)
    E, H = G * El, 64
    counts = rng.integers(0, 300, size=(G, E))
    counts[rng.integers(0, G), rng.integers(0, E)] = 0
    counts[:, rng.integers(0, E)] = 0                      # an expert nobody uses
    ret_base = [1 << 33, *[(1 << 33) + 7000000 * i for i in range(1, G)]]
    dev = torch.device("cuda:0")
    c_dev = torch.from_numpy(counts).int().to(dev)
    ptr_dev = torch.tensor(ret_base, dtype=torch.int64, device=dev)
    for r in range(G):
        pb, seg, received, ptrs = push_plan(counts, r, El, ret_base, H * 2)
        cap = received + 37
        kpb, kseg, kptrs = ops.ep_plan(c_dev, r, El, ptr_dev, H * 2, cap)
        assert kpb.dtype == torch.int32 and kseg.dtype == torch.int32 and kptrs.dtype == torch.int64
        assert np.array_equal(kpb.cpu().numpy(), pb)
        assert np.array_equal(kseg.cpu().numpy(), seg)
        assert np.array_equal(kptrs.cpu().numpy()[:received], ptrs)
        _, _, tptrs = push_plan_tensors(c_dev, r, El, ptr_dev, H * 2, cap)
        assert torch.equal(kptrs, tptrs)                   # the tail too


def test_peer_put_places_a_row_in_every_buffer():
    """cd_peer_put_i32 with the 'peers' being three buffers of this GPU: each gets the row at
    the given element offset and nothing else is touched; used with offset = rank * n it makes
    every rank hold the rows of all ranks (the counts of the expert-parallel plan)."""
    from complexity_deep_b200 import ops
    dev = torch.device("cuda:0")
    world, n = 3, 40
    bufs = [torch.full((2 * world * n,), -7, dtype=torch.int32, device=dev) for _ in range(world)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    rows = [torch.arange(n, dtype=torch.int32, device=dev) * (r + 1) + 1000 * r for r in range(world)]
    for slot in (0, 1):
        for r in range(world):      # what rank r would do
            ops.peer_put_i32(rows[r] + slot, ptrs, world, (slot * world + r) * n)
    torch.cuda.synchronize()
    for b in bufs:
        got = b.view(2, world, n)
        for slot in (0, 1):
            for r in range(world):
                assert torch.equal(got[slot, r], rows[r] + slot)
