"""N1 RMSNorm variants, row gather and the fused Q/K norm + RoPE kernel vs the oracle.

Tolerance: inputs are bf16; the kernels compute in fp32 and round once, so against the
oracle evaluated in fp32 on the same bf16 inputs the error is at most ~1 bf16 ulp of the
result: max_rel <= 2e-2 and mean_abs <= 2e-3 (the path's stated tolerance) with a large
margin (one bf16 rounding of a unit-scale value has mean error ~1.1e-3); the tests assert
max_rel <= 8e-3 and mean_abs <= 2e-3."""
import pytest
import torch

from conftest import load_golden
from oracle import complexity_oracle as oracle

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _close(got, want, max_rel=8e-3, mean_abs=2e-3):
    mr, ma = oracle.error_metrics(got.float().cpu(), want.float().cpu())
    assert mr <= max_rel and ma <= mean_abs, (mr, ma)


@pytest.mark.parametrize("T,H", [(1, 64), (7, 96), (33, 256), (130, 768), (64, 2048), (9, 4096),
                                 (5, 8192), (3, 100)])
def test_rmsnorm_plain(T, H):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(T * H)
    x = torch.randn(T, H, generator=g).to(BF)
    w = (torch.randn(H, generator=g) * 0.1 + 1).to(BF)
    out = ops.rmsnorm(x.cuda(), w.cuda(), 1e-6)
    _close(out, oracle.rmsnorm(x.float(), w.float(), 1e-6))


def test_rmsnorm_golden_fixture():
    from complexity_deep_b200 import ops
    g = load_golden("rmsnorm.pt")
    out = ops.rmsnorm(g["x"].to(BF).cuda(), g["weight"].to(BF).cuda(), 1e-6)
    _close(out, oracle.rmsnorm(g["x"].to(BF).float(), g["weight"].to(BF).float(), 1e-6))
    _close(out, g["out"], max_rel=2e-2, mean_abs=2e-3)


@pytest.mark.parametrize("T,H", [(50, 64), (300, 768), (257, 2048)])
def test_rmsnorm_residual_and_scatter(T, H):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, generator=g).to(BF)
    r = torch.randn(T, H, generator=g).to(BF)
    w = (torch.randn(H, generator=g) * 0.1 + 1).to(BF)
    dst = torch.randperm(T, generator=g).to(torch.int32)
    s, out = ops.rmsnorm(x.cuda(), w.cuda(), 1e-6, residual=r.cuda(), dst_rows=dst.cuda(),
                         want_sum=True)
    want_sum = (x.float() + r.float()).to(BF)
    assert torch.equal(s.cpu(), want_sum)            # one rounding of an exact fp32 sum
    want = oracle.rmsnorm(want_sum.float(), w.float(), 1e-6)
    scattered = torch.empty_like(want)
    scattered[dst.long()] = want
    _close(out, scattered)


def test_gather_rows_bit_exact():
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(2)
    for T, H in [(1, 8), (77, 100), (1000, 768), (4096, 2048)]:
        x = torch.randn(T, H, generator=g).to(BF)
        src = torch.randperm(T, generator=g).to(torch.int32)
        out = ops.gather_rows(x.cuda(), src.cuda())
        assert torch.equal(out.cpu(), x[src.long()])


@pytest.mark.parametrize("hq,hkv,D,S,pos0,norm", [(4, 2, 64, 12, 0, True), (16, 8, 128, 40, 0, True),
                                                  (4, 2, 64, 1, 12, True), (12, 4, 64, 9, 5, False),
                                                  (2, 1, 32, 7, 3, True), (2, 1, 24, 5, 0, True),
                                                  (2, 2, 256, 3, 1, True)])
def test_qk_norm_rope(hq, hkv, D, S, pos0, norm):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(3)
    B = 2
    qkv = torch.randn(B * S, (hq + 2 * hkv) * D, generator=g).to(BF)
    qw = (torch.randn(D, generator=g) * 0.1 + 1).to(BF)
    kw = (torch.randn(D, generator=g) * 0.1 + 1).to(BF)
    cos, sin = oracle.rope_tables(D, pos0 + S, 10000.0)
    got = ops.qk_norm_rope_(qkv.clone().cuda(), qw.cuda() if norm else None,
                            kw.cuda() if norm else None, cos.cuda(), sin.cuda(), 1e-6, S, pos0,
                            hq, hkv, D).cpu()
    f = qkv.float()
    q = f[:, : hq * D].view(B, S, hq, D)
    k = f[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D)
    if norm:
        q = torch.nn.functional.rms_norm(q, (D,), qw.float(), 1e-6)
        k = torch.nn.functional.rms_norm(k, (D,), kw.float(), 1e-6)
    c, s = cos[pos0:, None, :], sin[pos0:, None, :]
    rot = lambda x: torch.cat([-x[..., D // 2:], x[..., : D // 2]], -1)
    q = q * c + rot(q) * s
    k = k * c + rot(k) * s
    _close(got[:, : hq * D], q.reshape(B * S, -1))
    _close(got[:, hq * D:(hq + hkv) * D], k.reshape(B * S, -1))
    assert torch.equal(got[:, (hq + hkv) * D:], qkv[:, (hq + hkv) * D:])   # V untouched


@pytest.mark.parametrize("T,H,scatter", [(50, 64, False), (300, 768, True), (257, 2048, True),
                                         (9, 4096, False), (5, 100, True)])
def test_rmsnorm_split_stream(T, H, scatter):
    """cd_rmsnorm_split: the norm of hi + lo in fp32 (a value carried as a split-bf16 pair) —
    against the oracle on the exact fp32 sum, at a tolerance a bf16-rounded input cannot meet:
    the result may differ from the fp32 answer only by its own final rounding."""
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(T + H)
    v = torch.randn(T, H, generator=g)
    hi = v.to(BF)
    lo = (v - hi.float()).to(BF)
    w = (torch.randn(H, generator=g) * 0.1 + 1).to(BF)
    dst = torch.randperm(T, generator=g).to(torch.int32) if scatter else None
    out = ops.rmsnorm(hi.cuda(), w.cuda(), 1e-6, x_lo=lo.cuda(),
                      dst_rows=dst.cuda() if scatter else None)
    want = oracle.rmsnorm(hi.float() + lo.float(), w.float(), 1e-6)
    if scatter:
        scattered = torch.empty_like(want)
        scattered[dst.long()] = want
        want = scattered
    # equal to the correctly rounded bf16 of the fp32 result up to one ulp on a few elements
    assert (out.cpu() == want.to(BF)).float().mean() > 0.98
    _close(out, want)
    # and measurably closer to the fp32 norm of v than the norm of hi alone
    plain = ops.rmsnorm(hi.cuda(), w.cuda(), 1e-6, dst_rows=dst.cuda() if scatter else None)
    ref = oracle.rmsnorm(v, w.float(), 1e-6)
    if scatter:
        r2 = torch.empty_like(ref)
        r2[dst.long()] = ref
        ref = r2
    e_split = (out.float().cpu() - ref).abs().mean()
    e_plain = (plain.float().cpu() - ref).abs().mean()
    assert e_split < e_plain
