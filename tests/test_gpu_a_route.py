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
