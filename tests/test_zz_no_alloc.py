"""cd_route_static — the dispatch entry point for hosts that cannot allocate device memory
where they route a batch (a serving loop under a fixed memory budget; a plugin that only
gets input and output buffers).  Its scratch is a fixed array inside the library, so the
call itself allocates nothing.

Called here directly through the C ABI and compared, bit for bit, with cd_route (the entry
point that takes caller-provided scratch) on two calls in a row: the second call reuses the
shared array with a smaller and differently distributed batch, so leftovers of the first
call would show.  Collected last so a run that stops at the first failure has already run
every other test; it also passes alone in a fresh process."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _outputs(T, E, dev):
    i32 = dict(dtype=torch.int32, device=dev)
    return [torch.full((T,), -1, **i32), torch.full((E,), -1, **i32),
            torch.full((E + 1,), -1, **i32), torch.full((T,), -1, **i32),
            torch.full((T,), -1, **i32)]


def _both(lib, ids, table, E):
    from complexity_deep_b200 import _lib
    dev = ids.device
    T, V = ids.numel(), table.numel()
    stream = torch.cuda.current_stream().cuda_stream
    a = _outputs(T, E, dev)
    ws = torch.empty(max(lib.cd_route_workspace_bytes(T, E), 4), dtype=torch.uint8, device=dev)
    _lib.check(lib.cd_route(ids.data_ptr(), table.data_ptr(), V, E, T, *[t.data_ptr() for t in a],
                            ws.data_ptr(), ws.numel(), stream), "cd_route")
    b = _outputs(T, E, dev)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    _lib.check(lib.cd_route_static(ids.data_ptr(), table.data_ptr(), V, E, T,
                                   *[t.data_ptr() for t in b], stream), "cd_route_static")
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    return a, b, free_before - free_after


def test_static_scratch_dispatch_matches_cd_route_twice():
    from complexity_deep_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    # call 1: many blocks, 32 experts; call 2: fewer tokens, 8 experts, skewed ids
    cases = [(50000, 4096, 32, torch.randint(-10, 4200, (50000,), generator=g)),
             (3001, 1000, 8, (torch.randint(0, 1000, (3001,), generator=g) ** 2) // 1000)]
    from oracle import complexity_oracle as oracle
    for n, (T, V, E, ids) in enumerate(cases):
        table = (torch.arange(V) * 7 + 3) % E
        a, b, grew = _both(lib, ids.to(dev), table.to(dev), E)
        names = ["expert_ids", "counts", "offsets", "perm", "inv_perm"]
        want = oracle.route(ids.numpy(), table.numpy(), E)     # the CPU oracle, directly
        for name, x, y, w in zip(names, a, b, want):
            assert torch.equal(x, y), name        # integer artefacts: bit-exact
            assert np.array_equal(y.cpu().numpy(), w), name
        if n > 0:   # (the first call on a device may load the library's kernels)
            # free device memory as the driver reports it, before and after the call; repeated a
            # few times so that an unrelated process on the same GPU cannot fail the check
            for _ in range(3):
                if grew <= 0:
                    break
                grew = _both(lib, ids.to(dev), table.to(dev), E)[2]
            assert grew <= 0, f"device memory in use grew by {grew} bytes across the call"
        assert int(b[2][-1]) == T and int(b[1].sum()) == T
        assert np.array_equal(np.sort(b[3].cpu().numpy()), np.arange(T))


def test_static_scratch_size_limit_is_rejected():
    from complexity_deep_b200 import _lib
    lib = _lib.load()
    assert lib.cd_route_static_max_tokens(256) == 512 * 2048
    assert lib.cd_route_static_max_tokens(8) == 16384 * 2048
    assert lib.cd_route_static_max_tokens(0) == 0
    dev = torch.device("cuda:0")
    E = 256
    T = lib.cd_route_static_max_tokens(E) + 1
    ids = torch.zeros(8, dtype=torch.int64, device=dev)       # never dereferenced: size check first
    table = torch.zeros(8, dtype=torch.int64, device=dev)
    out = _outputs(8, E, dev)
    st = lib.cd_route_static(ids.data_ptr(), table.data_ptr(), 8, E, T,
                             *[t.data_ptr() for t in out], None)
    assert st == 3                                            # CD_ERR_UNSUPPORTED
    assert b"built-in array" in lib.cd_last_cuda_error()
    with pytest.raises(_lib.CdeepError):
        _lib.check(st, "cd_route_static")
