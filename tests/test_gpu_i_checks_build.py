"""The checking build of the library (libcdeep_checks.so, -DCDEEP_CHECKS): indices that kernels
read from device memory are validated on the device, a bad entry raises the status word to 4
and its access is skipped.

Every bad index used here still points INSIDE a larger allocation that surrounds the buffer the
kernel is given, so nothing can fault even if a check were missing; what the tests observe is the
status word, the untouched sentinel rows, and that every valid row equals the CPU oracle."""
import ctypes

import pytest
import torch

from oracle import complexity_oracle as oracle

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
SENTINEL = 7.0


@pytest.fixture(scope="module")
def libs():
    from complexity_deep_b200 import _lib
    checks = _lib.open_library(_lib.CHECKS_LIB_PATH)
    normal = _lib.load()
    assert checks.cd_checks_enabled() == 1
    assert normal.cd_checks_enabled() == (1 if normal is checks else 0)
    return checks, normal


def _status(lib):
    st = ctypes.c_int(-1)
    assert lib.cd_status_fetch(ctypes.byref(st)) == 0
    return st.value


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _surrounded(T, H, dev):
    """[3T, H] sentinel buffer and the view of its middle T rows that the kernel is given."""
    big = torch.full((3 * T, H), SENTINEL, dtype=BF, device=dev)
    return big, big[T:2 * T]


def test_rmsnorm_scatter_skips_rows_whose_destination_is_out_of_range(libs):
    checks, _ = libs
    dev = torch.device("cuda:0")
    T, H, eps = 64, 256, 1e-6
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, H, generator=g).to(BF)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(BF)
    dst = torch.randperm(T, generator=g).to(torch.int32)
    bad_rows = [5, 40]
    lost = [int(dst[r]) for r in bad_rows]          # destinations that nobody writes now
    dst[5], dst[40] = -1, T + 3
    big, out = _surrounded(T, H, dev)
    xd, wd, dd = x.to(dev), w.to(dev), dst.to(dev)
    assert _status(checks) == 0
    st = checks.cd_rmsnorm(xd.data_ptr(), None, wd.data_ptr(), eps, None, out.data_ptr(),
                           dd.data_ptr(), T, H, _stream())
    assert st == 0
    assert _status(checks) == 4                      # reported ...
    assert _status(checks) == 0                      # ... and cleared
    want = oracle.rmsnorm(x.float(), w.float(), eps)
    got = big.float().cpu()
    for r in range(T):
        if r in bad_rows:
            continue
        assert torch.allclose(got[T + int(dst[r])], want[r], rtol=2e-2, atol=2e-2), r
    untouched = torch.ones(3 * T, dtype=torch.bool)
    untouched[T:2 * T] = False
    for d in lost:
        untouched[T + d] = True
    assert bool((got[untouched] == SENTINEL).all())  # nothing outside, nothing at the skipped rows


def test_gather_rows_skips_rows_whose_source_is_out_of_range(libs):
    checks, _ = libs
    dev = torch.device("cuda:0")
    T, H = 48, 128
    g = torch.Generator().manual_seed(4)
    big_x = torch.randn(3 * T, H, generator=g).to(BF).to(dev)
    x = big_x[T:2 * T]
    src = torch.randperm(T, generator=g).to(torch.int32)
    src[7], src[30] = T + 1, -2
    out = torch.full((T, H), SENTINEL, dtype=BF, device=dev)
    st = checks.cd_gather_rows(x.data_ptr(), src.to(dev).data_ptr(), out.data_ptr(), T, H, _stream())
    assert st == 0 and _status(checks) == 4
    got, xs = out.cpu(), x.cpu()
    for j in range(T):
        if j in (7, 30):
            assert bool((got[j].float() == SENTINEL).all())
        else:
            assert torch.equal(got[j], xs[int(src[j])])


def _down_case(dev, seed=9, T=96, H=64, Ie=64, E=3):
    g = torch.Generator().manual_seed(seed)
    hr = torch.randn(T, Ie, generator=g).to(BF)
    wd = (torch.randn(E, H, Ie, generator=g) * 0.05).to(BF)
    seg = torch.tensor([0, 30, 30, T], dtype=torch.int32)       # the middle expert is empty
    pm = torch.randperm(T, generator=g).to(torch.int32)
    acc = torch.empty(T, H)
    for e in range(E):
        lo, hi = int(seg[e]), int(seg[e + 1])
        acc[lo:hi] = hr[lo:hi].float() @ wd[e].float().t()
    return hr, wd, seg, pm, acc


def _down(lib, hr, wd, seg, pm, out, T, H, Ie, E):
    return lib.cd_moe_down(hr.data_ptr(), Ie, wd.data_ptr(), None, 0, None, seg.data_ptr(), E,
                           pm.data_ptr(), None, None, out.data_ptr(), None, T, H, _stream())


def test_moe_down_row_map_and_segment_table_are_checked(libs):
    checks, normal = libs
    dev = torch.device("cuda:0")
    T, H, Ie, E = 96, 64, 64, 3
    hr, wd, seg, pm, acc = _down_case(dev)
    hrd, wdd = hr.to(dev), wd.to(dev)

    # valid inputs: same bits from both builds, status stays 0
    o_n = torch.empty(T, H, dtype=BF, device=dev)
    o_c = torch.empty(T, H, dtype=BF, device=dev)
    assert _down(normal, hrd, wdd, seg.to(dev), pm.to(dev), o_n, T, H, Ie, E) == 0
    assert _down(checks, hrd, wdd, seg.to(dev), pm.to(dev), o_c, T, H, Ie, E) == 0
    assert _status(checks) == 0 and _status(normal) == 0
    assert torch.equal(o_n, o_c)

    # one destination out of range: that row is not stored, the others equal the oracle
    bad = pm.clone()
    lost = int(bad[11])
    bad[11] = T + 5
    big, out = _surrounded(T, H, dev)
    assert _down(checks, hrd, wdd, seg.to(dev), bad.to(dev), out, T, H, Ie, E) == 0
    assert _status(checks) == 4
    got = big.float().cpu()
    for r in range(T):
        if r == 11:
            continue
        mr, ma = oracle.error_metrics(got[T + int(bad[r])], acc[r])
        assert mr <= 2e-2, (r, mr)
    assert bool((got[T + lost] == SENTINEL).all())
    assert bool((got[:T] == SENTINEL).all()) and bool((got[2 * T:] == SENTINEL).all())

    # a segment table that runs backwards schedules nothing at all
    big, out = _surrounded(T, H, dev)
    seg_bad = torch.tensor([0, 50, 40, T], dtype=torch.int32, device=dev)
    assert _down(checks, hrd, wdd, seg_bad, pm.to(dev), out, T, H, Ie, E) == 0
    assert _status(checks) == 4
    assert bool((big.float() == SENTINEL).all())

    # and the library works normally afterwards
    assert _down(checks, hrd, wdd, seg.to(dev), pm.to(dev), o_c, T, H, Ie, E) == 0
    assert _status(checks) == 0
    assert torch.equal(o_n, o_c)
