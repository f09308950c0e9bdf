"""tcgen05 GEMM entry points through the C ABI vs fp32 oracle arithmetic on the same
bf16-rounded inputs.

Tolerance (stated by the path's specification): max|y - ref| / max|ref| <= 2e-2 and
mean|y - ref| <= 2e-3 for outputs of unit scale; for outputs of another scale the mean bound
is taken relative to rms(ref).  The kernels accumulate in fp32 and round once (twice where
the SwiGLU intermediate h is stored in bf16), so the observed errors sit well inside."""
import pytest
import torch
import torch.nn.functional as F

from oracle import complexity_oracle as oracle

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _rand(g, *shape, scale=1.0):
    return (torch.randn(*shape, generator=g) * scale).to(BF)


def _close(got, ref, max_rel=2e-2, mean_rel=2e-3):
    got, ref = got.float().cpu(), ref.float().cpu()
    mr, ma = oracle.error_metrics(got, ref)
    rms = float(ref.double().pow(2).mean().sqrt())
    assert torch.isfinite(got).all()
    assert mr <= max_rel and ma <= mean_rel * max(rms, 1e-30), (mr, ma, rms)


def _fetch():
    from complexity_deep_b200 import ops
    ops.status_fetch()


@pytest.mark.parametrize("T,K,N", [(128, 64, 256), (128, 64, 128), (128, 128, 256), (256, 512, 512),
                                   (100, 64, 8), (1, 72, 40), (333, 200, 264), (1000, 768, 1024),
                                   (4096, 2048, 2048), (129, 1032, 520)])
@pytest.mark.parametrize("with_res", [False, True])
def test_linear(T, K, N, with_res):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(T + K + N)
    x, w = _rand(g, T, K), _rand(g, N, K, scale=0.05)
    res = _rand(g, T, N) if with_res else None
    out = ops.linear(x.cuda(), w.cuda(), res.cuda() if with_res else None)
    _fetch()
    ref = x.float() @ w.float().t()
    if with_res:
        ref = ref + res.float()
    _close(out, ref)


def test_linear_many_tiles_persistent_schedule():
    """More tiles than SMs and more k-blocks than pipeline stages: exercises barrier phase
    wrap-around, both TMEM accumulators and the band schedule."""
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(5)
    T, K, N = 128 * 40 + 17, 64 * 13, 256 * 9 + 64
    x, w = _rand(g, T, K), _rand(g, N, K, scale=0.05)
    out = ops.linear(x.cuda(), w.cuda())
    _fetch()
    ref = (x.cuda().float() @ w.cuda().float().t())      # fp32 reference on the device
    _close(out, ref)
    out2 = ops.linear(x.cuda(), w.cuda())
    assert torch.equal(out, out2)                        # deterministic


@pytest.mark.parametrize("T,H,N", [(64, 64, 128), (300, 256, 384), (2048, 768, 1280)])
def test_mu_qkv_k_concat(T, H, N):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(7)
    x, mu = _rand(g, T, H), _rand(g, T, H)
    w, wm = _rand(g, N, H, scale=0.05), _rand(g, N, H, scale=0.05)
    out = ops.mu_qkv(x.cuda(), mu.cuda(), w.cuda(), wm.cuda())
    _fetch()
    # reference arithmetic: cat([x, mu]) @ cat([W, W_mu], dim=1)^T  (attention.py:121-127)
    ref = F.linear(torch.cat([x, mu], -1).float(), torch.cat([w, wm], 1).float())
    _close(out, ref)
    out_nomu = ops.mu_qkv(x.cuda(), None, w.cuda(), None)
    _close(out_nomu, x.float() @ w.float().t())


@pytest.mark.parametrize("T,H", [(40, 64), (513, 768)])
def test_mu_proj_bias_and_clamp(T, H):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(9)
    h, w = _rand(g, T, H), _rand(g, H, H, scale=0.05)
    mu = (torch.randn(H, generator=g) * 1.5 + 1.0).to(BF)
    ref = torch.clamp(mu.float(), 0.0, 2.0) + h.float() @ w.float().t()     # layer.py:61
    out = ops.mu_proj(h.cuda(), w.cuda(), mu.cuda(), 0.0, 2.0)
    _fetch()
    _close(out, ref)
    out_c = ops.mu_proj(h.cuda(), w.cuda(), mu.cuda(), 0.0, 2.0, out_clamp=(-2.0, 2.0))
    _close(out_c, ref.clamp(-2.0, 2.0))                                     # modeling.py:200
    assert out_c.float().abs().max() <= 2.0


def _swiglu_ref(x, gate, up):
    return F.silu(x.float() @ gate.float().t()) * (x.float() @ up.float().t())


def _pack_ref(gate, up, block_n):
    """Layout cd_pack_gate_up must produce, from [G, I, H] sources: per tile of block_n / 2
    output features, the gate rows then the up rows; zero rows pad the last tile."""
    G, I, H = gate.shape
    half = block_n // 2
    chunks = -(-I // half)
    pad = chunks * half - I
    if pad:
        z = gate.new_zeros(G, pad, H)
        gate, up = torch.cat([gate, z], 1), torch.cat([up, z], 1)
    g = gate.reshape(G, chunks, 1, half, H)
    u = up.reshape(G, chunks, 1, half, H)
    return torch.cat([g, u], dim=2).reshape(G, chunks * block_n, H)


@pytest.mark.parametrize("G,I,H,bn", [(2, 40, 8, 128), (1, 200, 8, 256), (3, 72, 136, 64),
                                      (8, 704, 256, 256), (1, 33, 40, 32)])
def test_pack_kernels_match_layout(G, I, H, bn):
    """cd_pack_gate_up (both source layouts) and cd_pack_down, bit-exact."""
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(3)
    gate, up = _rand(g, G, I, H), _rand(g, G, I, H)
    want = _pack_ref(gate, up, bn)
    got = ops.pack_gate_up(gate.cuda(), up.cuda(), bn)
    assert got.shape == want.shape and torch.equal(got.cpu(), want)
    got_t = ops.pack_gate_up(gate.transpose(1, 2).contiguous().cuda(),
                             up.transpose(1, 2).contiguous().cuda(), bn, feature_major=False)
    assert torch.equal(got_t.cpu(), want)
    down = _rand(g, G, I, H)
    assert torch.equal(ops.pack_down(down.cuda()).cpu(), down.transpose(1, 2).contiguous())
    _fetch()


@pytest.mark.parametrize("T,H,I,bn", [(128, 64, 128, 256), (200, 128, 64, 128), (77, 256, 40, 128),
                                      (1000, 768, 512, 256), (512, 2048, 704, 128),
                                      (512, 2048, 704, 256), (300, 512, 200, 256),
                                      (32, 2048, 704, 32), (200, 256, 72, 64), (8, 64, 16, 32)])
def test_moe_up_dense(T, H, I, bn):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(11)
    x = _rand(g, T, H)
    gate, up = _rand(g, I, H, scale=0.05), _rand(g, I, H, scale=0.05)
    packed = ops.pack_gate_up(gate[None].cuda(), up[None].cuda(), bn)
    h = ops.moe_up(x.cuda(), None, 1, packed, I, bn)
    _fetch()
    _close(h, _swiglu_ref(x, gate, up))


def _segments(g, T, E, empty=()):
    w = torch.rand(E, generator=g) + 0.1
    for e in empty:
        w[e] = 0
    counts = torch.floor(w / w.sum() * T).long()
    live = [e for e in range(E) if e not in empty]
    counts[live[0]] += T - counts.sum()
    return torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(torch.int32)


@pytest.mark.parametrize("T,H,I,E,bn,empty", [(300, 64, 64, 4, 128, ()), (1000, 128, 136, 8, 256, (2,)),
                                              (4096, 768, 512, 4, 256, ()), (517, 256, 72, 32, 128, (0, 31)),
                                              (129, 64, 64, 4, 128, (1, 2, 3)),
                                              (256, 256, 88, 8, 32, (3,)), (40, 128, 48, 4, 64, ())])
def test_moe_up_grouped_ragged(T, H, I, E, bn, empty):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(13)
    x = _rand(g, T, H)
    gate, up = _rand(g, E, I, H, scale=0.05), _rand(g, E, I, H, scale=0.05)
    seg = _segments(g, T, E, empty)
    packed = ops.pack_gate_up(gate.cuda(), up.cuda(), bn)
    h = ops.moe_up(x.cuda(), seg.cuda(), E, packed, I, bn)
    _fetch()
    ref = torch.empty(T, I)
    for e in range(E):
        lo, hi = int(seg[e]), int(seg[e + 1])
        ref[lo:hi] = _swiglu_ref(x[lo:hi], gate[e], up[e])
    _close(h, ref)


@pytest.mark.parametrize("T,H,Ie,Is,E,shared,perm,res", [
    (300, 64, 64, 64, 4, True, True, True), (1000, 256, 136, 72, 8, True, True, False),
    (500, 128, 64, 0, 4, False, False, False), (2048, 768, 512, 512, 4, True, True, True),
    (130, 264, 40, 200, 3, True, True, True)])
def test_moe_down_combine_unpermute_residual(T, H, Ie, Is, E, shared, perm, res):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(17)
    hr = _rand(g, T, Ie)
    wd = _rand(g, E, H, Ie, scale=0.05)
    hs = _rand(g, T, Is) if shared else None
    ws = _rand(g, H, Is, scale=0.05) if shared else None
    seg = _segments(g, T, E, (1,) if E > 3 else ())
    pm = torch.randperm(T, generator=g).to(torch.int32) if perm else None
    rs = _rand(g, T, H) if res else None
    out = ops.moe_down(hr.cuda(), wd.cuda(), hs.cuda() if shared else None,
                       ws.cuda() if shared else None, seg.cuda(), E,
                       pm.cuda() if perm else None, rs.cuda() if res else None)
    _fetch()
    acc = torch.empty(T, H)
    for e in range(E):
        lo, hi = int(seg[e]), int(seg[e + 1])
        acc[lo:hi] = hr[lo:hi].float() @ wd[e].float().t()
    if shared:
        acc += hs.float() @ ws.float().t()
    ref = torch.empty(T, H)
    if perm:
        ref[pm.long()] = acc
    else:
        ref = acc
    if res:
        ref = ref + rs.float()
    _close(out, ref)


@pytest.mark.parametrize("T,H,Is,perm,res,routed", [(300, 64, 64, True, True, True),
                                                    (1000, 256, 200, True, False, True),
                                                    (513, 768, 512, False, True, False)])
def test_moe_combine_shared_plus_routed_partial(T, H, Is, perm, res, routed):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(19)
    hs, ws = _rand(g, T, Is), _rand(g, H, Is, scale=0.05)
    yr = _rand(g, T, H) if routed else None
    pm = torch.randperm(T, generator=g).to(torch.int32) if perm else None
    rs = _rand(g, T, H) if res else None
    out = ops.moe_combine(hs.cuda(), ws.cuda(), yr.cuda() if routed else None,
                          pm.cuda() if perm else None, rs.cuda() if res else None)
    _fetch()
    acc = hs.float() @ ws.float().t()
    if routed:
        acc = acc + yr.float()
    ref = torch.empty(T, H)
    if perm:
        ref[pm.long()] = acc
    else:
        ref = acc
    if res:
        ref = ref + rs.float()
    _close(out, ref)


@pytest.mark.parametrize("T,S,pos0,norm,with_mu", [(4096, 512, 3, True, True), (4224, 1056, 0, False, True),
                                                   (8192, 2048, 0, True, False), (96, 32, 5, True, True)])
def test_mu_qkv_with_fused_qk_norm_rope(T, S, pos0, norm, with_mu):
    """QKV projection with per-head RMSNorm + RoPE applied to the fp32 accumulators (the fused
    kernel for many rows, the two-kernel path for few) vs fp32 arithmetic in the reference's
    order: project, norm, rotate (attention.py:120-155)."""
    from complexity_deep_b200 import _lib, ops
    hq, hkv, D, H = 4, 2, 128, 256
    N = (hq + 2 * hkv) * D
    g = torch.Generator().manual_seed(T + pos0)
    x, mu = _rand(g, T, H), _rand(g, T, H)
    w, wm = _rand(g, N, H, scale=0.05), _rand(g, N, H, scale=0.05)
    qw = (torch.randn(D, generator=g) * 0.1 + 1).to(BF)
    kw = (torch.randn(D, generator=g) * 0.1 + 1).to(BF)
    cos, sin = oracle.rope_tables(D, pos0 + S, 10000.0)
    fused = bool(_lib.load().cd_mu_qkv_rope_supported(T, N, hq, hkv, D))
    assert fused == (T >= 4096)
    out = ops.mu_qkv_rope(x.cuda(), mu.cuda() if with_mu else None, w.cuda(),
                          wm.cuda() if with_mu else None, qw.cuda() if norm else None,
                          kw.cuda() if norm else None, cos.cuda(), sin.cuda(), 1e-6, S, pos0,
                          hq, hkv, D)
    _fetch()
    ref = x.float() @ w.float().t()
    if with_mu:
        ref = ref + mu.float() @ wm.float().t()
    B = T // S
    q = ref[:, : hq * D].view(B, S, hq, D)
    k = ref[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D)
    if norm:
        q = F.rms_norm(q, (D,), qw.float(), 1e-6)
        k = F.rms_norm(k, (D,), kw.float(), 1e-6)
    c, s = cos[pos0:, None, :], sin[pos0:, None, :]
    rot = lambda t: torch.cat([-t[..., D // 2:], t[..., : D // 2]], -1)
    q, k = q * c + rot(q) * s, k * c + rot(k) * s
    _close(out[:, : hq * D], q.reshape(T, -1))
    _close(out[:, hq * D:(hq + hkv) * D], k.reshape(T, -1))
    _close(out[:, (hq + hkv) * D:], ref[:, (hq + hkv) * D:])


def test_bounded_waits_report_a_stalled_pipeline_and_leave_the_device_usable():
    """Failure detection without a fault: a tile whose loader is switched off makes the pipeline
    waits run into a 20 ms limit; the kernel returns, the status word is raised once, and the
    next GEMM on the same context is correct."""
    import ctypes
    import time
    from complexity_deep_b200 import _lib, ops
    lib = _lib.load()
    a = torch.zeros(128, 64, dtype=BF, device="cuda")
    b = torch.zeros(128, 64, dtype=BF, device="cuda")
    out = torch.zeros(128, 128, dtype=BF, device="cuda")
    ops.status_fetch()                                            # clean before the test
    t0 = time.perf_counter()
    _lib.check(lib.cd_selftest_wait_timeout(a.data_ptr(), b.data_ptr(), out.data_ptr(), 20,
                                            torch.cuda.current_stream().cuda_stream), "selftest")
    st = ctypes.c_int(0)
    _lib.check(lib.cd_status_fetch(ctypes.byref(st)), "cd_status_fetch")
    elapsed = time.perf_counter() - t0
    assert st.value == 1                                          # the wait ran out and said so
    assert elapsed < 1.0                                          # bounded: ~20 ms, not seconds
    _lib.check(lib.cd_status_fetch(ctypes.byref(st)), "cd_status_fetch")
    assert st.value == 0                                          # cleared by the first read
    with pytest.raises(_lib.CdeepError):                          # the Python layer raises on it
        _lib.check(lib.cd_selftest_wait_timeout(a.data_ptr(), b.data_ptr(), out.data_ptr(), 20,
                                                torch.cuda.current_stream().cuda_stream), "st")
        ops.status_fetch()
    g = torch.Generator().manual_seed(3)                          # the context still works
    x, w = _rand(g, 300, 256), _rand(g, 512, 256, scale=0.05)
    y = ops.linear(x.cuda(), w.cuda())
    _fetch()
    _close(y, x.float() @ w.float().t())


# ------------------------------------------------------------------ per-row destinations
@pytest.mark.parametrize("T,E,I_e,H", [(300, 4, 64, 256), (4500, 8, 704, 2048), (64, 8, 96, 512)])
def test_moe_down_push_stores_rows_at_their_addresses(T, E, I_e, H):
    """cd_moe_down_push: row j of the routed down projection lands at out_row_ptrs[j] — here
    addresses inside two local buffers in a shuffled order (on several GPUs they point into
    the peers' return buffers).  Covers the wide-tile epilogue (eight warps) and the narrow one."""
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    counts = torch.multinomial(torch.ones(E), T, replacement=True, generator=g).bincount(minlength=E)
    counts[1] = 0 if E > 2 else counts[1]                      # an expert without rows
    counts[0] += T - int(counts.sum())
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0)
    h = _rand(g, T, I_e)
    wd = _rand(g, E, H, I_e, scale=0.05)
    dest = torch.randperm(T, generator=g)                      # row j -> slot dest[j]
    bufs = [torch.zeros(T, H, dtype=BF, device="cuda") for _ in range(2)]
    ptrs = torch.tensor([bufs[int(d) % 2].data_ptr() + (int(d) // 2) * H * 2 for d in dest],
                        dtype=torch.int64)
    ops.moe_down_push(h.cuda(), wd.cuda(), offsets.cuda(), E, ptrs.cuda())
    _fetch()
    ref = torch.zeros(T, H)
    for e in range(E):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        ref[lo:hi] = h[lo:hi].float() @ wd[e].float().t()
    got = torch.stack([bufs[int(d) % 2][int(d) // 2] for d in dest]).cpu()
    _close(got, ref)


def test_push_rows_places_sorted_rows_in_owner_buffers():
    """cd_push_rows with two 'ranks' whose receive buffers are local: every expert-sorted row
    is copied, bit for bit, to row push_base[e] + (j - offsets[e]) of the buffer of the rank
    that owns expert e."""
    from complexity_deep_b200 import ops
    T, E, H, per_rank = 1000, 8, 512, 4
    g = torch.Generator().manual_seed(3)
    eid = torch.sort(torch.randint(0, E, (T,), generator=g)).values
    counts = eid.bincount(minlength=E)
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0)
    x = _rand(g, T, H)
    base = torch.zeros(E, dtype=torch.int32)                   # position inside the owner's buffer
    for r in range(E // per_rank):
        acc = 7 * r                                            # some rows already taken by other sources
        for e in range(r * per_rank, (r + 1) * per_rank):
            base[e] = acc
            acc += int(counts[e])
    bufs = [torch.full((T + 16, H), -1.0, dtype=BF, device="cuda") for _ in range(E // per_rank)]
    peer = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    ops.push_rows(x.cuda(), offsets.cuda(), base.cuda(), E, per_rank, peer.data_ptr())
    torch.cuda.synchronize()
    for e in range(E):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        got = bufs[e // per_rank][int(base[e]):int(base[e]) + hi - lo].cpu()
        assert torch.equal(got, x[lo:hi]), e


def _split(v):
    """fp32 -> (hi, lo) bf16 pair with hi = bf16(v), lo = bf16(v - hi)."""
    hi = v.to(BF)
    return hi, (v - hi.float()).to(BF)


@pytest.mark.parametrize("T,K,N", [(128, 64, 256), (300, 128, 264), (1000, 768, 1024),
                                   (4096, 2048, 2048), (40, 256, 96), (129, 1032, 520)])
@pytest.mark.parametrize("res_lo", [False, True])
def test_linear_split_residual_stream(T, K, N, res_lo):
    """cd_linear with the residual as a split-bf16 pair and the result stored as one: hi must be
    the correctly rounded fp32 result (up to accumulation-order noise) and hi + lo must be
    closer to it by two orders of magnitude than a bf16 tensor can be."""
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(T + K + N)
    x, w = _rand(g, T, K), _rand(g, N, K, scale=0.05)
    r_hi, r_lo = _split(torch.randn(T, N, generator=g))
    out, out_lo = ops.linear(x.cuda(), w.cuda(), r_hi.cuda(), residual_lo=r_lo.cuda() if res_lo else None,
                             want_lo=True)
    _fetch()
    ref = x.float() @ w.float().t() + r_hi.float() + (r_lo.float() if res_lo else 0)
    _close(out, ref)
    both = out.float().cpu() + out_lo.float().cpu()
    rms = float(ref.pow(2).mean().sqrt())
    err_pair = float((both - ref).abs().mean())
    err_hi = float((out.float().cpu() - ref).abs().mean())
    assert err_pair <= 2e-5 * max(1.0, rms), (err_pair, rms)      # fp32 accumulation-order noise
    assert err_pair * 20 < err_hi


@pytest.mark.parametrize("T,H,Ie,Is,E", [(300, 64, 64, 64, 4), (2048, 768, 512, 512, 4),
                                         (130, 264, 40, 200, 3), (5000, 256, 136, 72, 8)])
def test_moe_down_split_residual_stream(T, H, Ie, Is, E):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(23)
    hr, wd = _rand(g, T, Ie), _rand(g, E, H, Ie, scale=0.05)
    hs, ws = _rand(g, T, Is), _rand(g, H, Is, scale=0.05)
    seg = _segments(g, T, E, (1,) if E > 3 else ())
    pm = torch.randperm(T, generator=g).to(torch.int32)
    r_hi, r_lo = _split(torch.randn(T, H, generator=g))
    out, out_lo = ops.moe_down(hr.cuda(), wd.cuda(), hs.cuda(), ws.cuda(), seg.cuda(), E, pm.cuda(),
                               r_hi.cuda(), r_lo.cuda(), True)
    _fetch()
    acc = torch.empty(T, H)
    for e in range(E):
        lo, hi = int(seg[e]), int(seg[e + 1])
        acc[lo:hi] = hr[lo:hi].float() @ wd[e].float().t()
    acc += hs.float() @ ws.float().t()
    ref = torch.empty(T, H)
    ref[pm.long()] = acc
    ref = ref + r_hi.float() + r_lo.float()
    _close(out, ref)
    rms = float(ref.pow(2).mean().sqrt())
    err_pair = float((out.float().cpu() + out_lo.float().cpu() - ref).abs().mean())
    assert err_pair <= 2e-5 * max(1.0, rms), (err_pair, rms)


def test_moe_combine_split_residual_stream():
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(29)
    T, H, Is = 777, 512, 264
    hs, ws, yr = _rand(g, T, Is), _rand(g, H, Is, scale=0.05), _rand(g, T, H)
    pm = torch.randperm(T, generator=g).to(torch.int32)
    r_hi, r_lo = _split(torch.randn(T, H, generator=g))
    out, out_lo = ops.moe_combine(hs.cuda(), ws.cuda(), yr.cuda(), pm.cuda(), r_hi.cuda(), r_lo.cuda(),
                                  True)
    _fetch()
    ref = torch.empty(T, H)
    ref[pm.long()] = hs.float() @ ws.float().t() + yr.float()
    ref = ref + r_hi.float() + r_lo.float()
    _close(out, ref)
    err_pair = float((out.float().cpu() + out_lo.float().cpu() - ref).abs().mean())
    assert err_pair <= 2e-5 * max(1.0, float(ref.pow(2).mean().sqrt()))


@pytest.mark.parametrize("T,H,I,Is,E,bn,empty", [
    (300, 64, 64, 64, 4, 128, ()), (1000, 128, 136, 200, 8, 256, (2,)),
    (4096, 768, 512, 512, 4, 256, ()), (517, 256, 72, 40, 32, 128, (0, 31)),
    (8192, 2048, 704, 704, 8, 256, ()), (256, 256, 88, 88, 8, 32, (3,)), (40, 128, 48, 112, 4, 64, ())])
def test_moe_up_pair_routed_and_shared_one_launch(T, H, I, Is, E, bn, empty):
    """cd_moe_up_pair = cd_moe_up over the groups + cd_moe_up of the shared expert, same bits."""
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(31)
    x = _rand(g, T, H)
    gate, up = _rand(g, E, I, H, scale=0.05), _rand(g, E, I, H, scale=0.05)
    sg, su = _rand(g, 1, Is, H, scale=0.05), _rand(g, 1, Is, H, scale=0.05)
    seg = _segments(g, T, E, empty).cuda()
    packed = ops.pack_gate_up(gate.cuda(), up.cuda(), bn)
    packed_s = ops.pack_gate_up(sg.cuda(), su.cuda(), bn)
    xc = x.cuda()
    h, hs = ops.moe_up_pair(xc, seg, E, packed, I, packed_s, Is, bn)
    h1 = ops.moe_up(xc, seg, E, packed, I, bn)
    hs1 = ops.moe_up(xc, None, 1, packed_s, Is, bn)
    _fetch()
    assert torch.equal(h, h1) and torch.equal(hs, hs1)
    _close(hs, _swiglu_ref(x, sg[0], su[0]))


# ---- split-K of the few-row projections ---------------------------------------------------

@pytest.fixture
def split_k_modes():
    """Hands the test a switch over the forms of split-K (0 none, 1 cluster, 2 workspace) and
    puts the default back afterwards."""
    from complexity_deep_b200 import ops
    ops.split_k(True)                  # registers the workspace (used only under mode 2)
    before = ops.split_k_config(-1)
    yield ops
    ops.split_k_config(before)


def _noise_bound(ref):
    # one bf16 step at the value's size, plus the fp32 accumulation-order noise of the sum itself
    return ref.abs() * 2.0 ** -7 + 1e-5 * float(ref.pow(2).mean().sqrt())


@pytest.mark.parametrize("T,K,N,with_res", [(32, 4096, 2048, False), (128, 5632, 2048, True),
                                            (8, 3072, 1024, True), (100, 8192, 512, False),
                                            (256, 4096, 1024, True), (17, 4096 + 64, 264, False),
                                            (200, 6144, 1024, True), (32, 2048, 2048, True),
                                            (32, 8192, 6144, True)])   # the last: two ranges per cluster
def test_linear_split_k_forms_match_unsplit_and_fp32(split_k_modes, T, K, N, with_res):
    """The same call unsplit, with the cluster form and with the workspace form of split-K: all
    within the projection tolerance of the fp32 product and within fp32 accumulation-order noise
    (one bf16 rounding step of the output at most) of each other; each form twice in a row, so
    state left behind by a launch (a counter, a barrier phase) would show."""
    ops = split_k_modes
    from complexity_deep_b200 import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(T + K + N)
    x, w = _rand(g, T, K).cuda(), _rand(g, N, K, scale=0.05).cuda()
    res = _rand(g, T, N).cuda() if with_res else None
    ref = x.float() @ w.float().t() + (res.float() if with_res else 0)
    ops.split_k_config(0)
    assert lib.cd_splitk_ranges(T, K, N) == 1
    plain = ops.linear(x, w, res)
    _close(plain, ref)
    used = 0
    for mode in (1, 2):
        ops.split_k_config(mode)
        ranges = lib.cd_splitk_ranges(T, K, N)
        a = ops.linear(x, w, res)
        b = ops.linear(x, w, res)
        _fetch()
        _close(a, ref)
        assert torch.equal(a, b)                              # fixed order of the partial sums
        assert bool(((a.float() - plain.float()).abs() <= _noise_bound(ref)).all()), mode
        used += ranges > 1
    assert used >= 1 or K < 3072, "this shape is meant to split in at least one form"


def test_split_k_through_the_fused_epilogues(split_k_modes):
    """Split-K in front of every fused epilogue a few-row call can take: the mu K-concatenation,
    mu_proj's clamped bias and output clamp, the split-bf16 residual stream (both forms), and the
    dense SwiGLU (workspace form)."""
    ops = split_k_modes
    from complexity_deep_b200 import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(99)
    T, H = 48, 3072
    x, mu = _rand(g, T, H).cuda(), _rand(g, T, H).cuda()
    w, wm = _rand(g, 768, H, scale=0.05).cuda(), _rand(g, 768, H, scale=0.05).cuda()
    wp, mu_param = _rand(g, H, H, scale=0.05).cuda(), (_rand(g, H) * 3).cuda()
    r_hi, r_lo = _split(torch.randn(T, H, generator=g))
    ref_lin = x.float().cpu() @ wp.float().cpu().t() + r_hi.float() + r_lo.float()
    for mode in (1, 2):
        ops.split_k_config(mode)
        assert lib.cd_splitk_ranges(T, 2 * H, 768) > 1
        assert mode == 2 or lib.cd_splitk_ranges(T, H, H) > 1
        out = ops.mu_qkv(x, mu, w, wm)
        _close(out, F.linear(torch.cat([x, mu], -1).float(), torch.cat([w, wm], 1).float()))
        got = ops.mu_proj(x, wp, mu_param, -2.0, 2.0, out_clamp=(-1.5, 1.5))
        want = (x.float() @ wp.float().t() + mu_param.float().clamp(-2.0, 2.0)).clamp(-1.5, 1.5)
        _close(got, want)
        hi, lo = ops.linear(x, wp, r_hi.cuda(), residual_lo=r_lo.cuda(), want_lo=True)
        _close(hi, ref_lin)
        pair_err = float((hi.float().cpu() + lo.float().cpu() - ref_lin).abs().mean())
        assert pair_err <= 2e-5 * max(1.0, float(ref_lin.pow(2).mean().sqrt())), mode
    ops.split_k_config(2)
    for bn, I in ((64, 512), (128, 1024)):
        gate, up = _rand(g, I, H, scale=0.05), _rand(g, I, H, scale=0.05)
        packed = ops.pack_gate_up(gate[None].cuda(), up[None].cuda(), bn)
        h = ops.moe_up(x, None, 1, packed, I, bn)
        _close(h, _swiglu_ref(x.float().cpu(), gate, up))
    _fetch()
