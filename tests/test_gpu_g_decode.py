"""Decode-side kernels: single-query attention over a KV cache (cd_decode_attention) and the
narrow-tile GEMM path used when there are few rows, against fp32 references on the same
bf16-rounded inputs.  Tolerance: max|y - ref| / max|ref| <= 2e-2 and mean|y - ref| <= 2e-3 *
max(1, rms(ref)) (outputs are rounded to bf16 once)."""
import pytest
import torch

from conftest import assert_close

from oracle import complexity_oracle as oracle

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _close(got, ref, max_rel=2e-2, mean_abs=2e-3):
    assert_close(got, ref, max_rel, mean_abs)


@pytest.mark.parametrize("B,hq,hkv,D,L", [(3, 4, 2, 64, 1), (2, 4, 2, 128, 7), (3, 16, 8, 128, 300),
                                          (2, 12, 4, 64, 1000), (1, 8, 8, 128, 4100),
                                          (5, 4, 1, 128, 513)])
@pytest.mark.parametrize("masked", [False, True])
def test_decode_attention_vs_fp32_softmax(B, hq, hkv, D, L, masked):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(B * L + hq)
    qkv = torch.randn(B, (hq + 2 * hkv) * D, generator=g).to(BF)
    cap = L + 37                                      # the cache is a view of a larger buffer
    kbuf = torch.randn(B, hkv, cap, D, generator=g).to(BF)
    vbuf = torch.randn(B, hkv, cap, D, generator=g).to(BF)
    mask = None
    if masked:
        mask = torch.randn(B, 1, 1, L, generator=g)
        mask[:, :, :, ::5] = float("-inf")            # padding-style entries
        mask[:, :, :, 0] = 0.0                        # keep at least one key
        mask = mask.to(BF)
    k, v = kbuf.cuda()[:, :, :L], vbuf.cuda()[:, :, :L]
    out = ops.decode_attention(qkv.cuda(), k, v, mask.cuda() if masked else None, hq, hkv, D)
    q = qkv[:, : hq * D].float().view(B, hq, 1, D)
    kr = kbuf[:, :, :L].float().repeat_interleave(hq // hkv, dim=1)
    vr = vbuf[:, :, :L].float().repeat_interleave(hq // hkv, dim=1)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q, kr, vr, attn_mask=mask.float() if masked else None)
    _close(out, ref.view(B, hq * D))


def test_attention_module_decode_step_uses_cache_in_place():
    """ComplexityAttention with head_dim 128: prefill, then two decode steps with a zero
    additive mask (whole cache visible) and one with no mask (the reference's is_causal=True
    with q_len 1 sees only key 0), vs the oracle."""
    import complexity_deep_b200 as cd
    torch.manual_seed(0)
    att = cd.ComplexityAttention(512, 4, 2)
    sd = {k: v.clone() for k, v in att.state_dict().items()}
    sd_f = {k: (v.to(BF).float() if v.is_floating_point() else v) for k, v in sd.items()}
    att = att.to(device="cuda", dtype=BF).eval()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 9, 512, generator=g).to(BF)
    mu = torch.randn(2, 9, 512, generator=g).to(BF)
    _, kv = att(x.cuda(), mu_prev=mu.cuda(), use_cache=True)
    _, ref_kv = oracle.attention(sd_f, "", x.float(), 4, 2, mu_prev=mu.float(), use_cache=True)
    for step in range(3):
        xs = torch.randn(2, 1, 512, generator=g).to(BF)
        ms = torch.randn(2, 1, 512, generator=g).to(BF)
        L = 9 + step + 1
        mask = None if step == 2 else torch.zeros(2, 1, 1, L, dtype=BF)
        out, kv = att(xs.cuda(), attention_mask=None if mask is None else mask.cuda(),
                      past_key_value=kv, use_cache=True, mu_prev=ms.cuda())
        ref, ref_kv = oracle.attention(sd_f, "", xs.float(), 4, 2,
                                       attention_mask=None if mask is None else mask.float(),
                                       past_key_value=ref_kv, use_cache=True, mu_prev=ms.float())
        _close(out, ref)
        _close(kv[0], ref_kv[0])
        assert kv[0].shape == (2, 2, L, 128)
        if step > 0:
            assert kv[0]._cd_kv.buf.data_ptr() == buf_ptr      # appended in place, no copy
        buf_ptr = kv[0]._cd_kv.buf.data_ptr()


@pytest.mark.parametrize("T,K,N", [(32, 2048, 4096), (8, 256, 2048), (256, 2048, 2048),
                                   (64, 768, 40), (200, 512, 1000), (1, 64, 32)])
def test_few_rows_use_narrow_tiles(T, K, N):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, K, generator=g).to(BF)
    w = (torch.randn(N, K, generator=g) * 0.05).to(BF)
    res = torch.randn(T, N, generator=g).to(BF)
    out = ops.linear(x.cuda(), w.cuda(), res.cuda())
    ops.status_fetch()
    _close(out, x.float() @ w.float().t() + res.float())
    mu = torch.randn(T, K, generator=g).to(BF)
    wm = (torch.randn(N, K, generator=g) * 0.05).to(BF)
    out2 = ops.mu_qkv(x.cuda(), mu.cuda(), w.cuda(), wm.cuda())
    _close(out2, x.float() @ w.float().t() + mu.float() @ wm.float().t())


# ------------------------------------------------------------------ device-side positions
@pytest.mark.parametrize("B,hq,hkv,D,L", [(3, 16, 8, 128, 300), (2, 12, 4, 64, 1000),
                                          (5, 4, 1, 128, 513), (2, 4, 2, 128, 1)])
def test_decode_attention_device_length_is_bit_exact(B, hq, hkv, D, L):
    """The launch sized for the cache capacity with the length in device memory returns the
    same bits as the launch sized for that length."""
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(L)
    cap = 4 * L + 123
    qkv = torch.randn(B, (hq + 2 * hkv) * D, generator=g).to(BF).cuda()
    kbuf = torch.randn(B, hkv, cap, D, generator=g).to(BF).cuda()
    vbuf = torch.randn(B, hkv, cap, D, generator=g).to(BF).cuda()
    ref = ops.decode_attention(qkv, kbuf[:, :, :L], vbuf[:, :, :L], None, hq, hkv, D)
    n = torch.tensor([L], dtype=torch.int32, device="cuda")
    got = ops.decode_attention(qkv, kbuf, vbuf, None, hq, hkv, D, kv_len_dev=n)
    assert torch.equal(got, ref)
    n.fill_(cap + 50)                      # clamped to the capacity
    full = ops.decode_attention(qkv, kbuf, vbuf, None, hq, hkv, D)
    assert torch.equal(ops.decode_attention(qkv, kbuf, vbuf, None, hq, hkv, D, kv_len_dev=n), full)


@pytest.mark.parametrize("hq,hkv,D,norm", [(16, 8, 128, True), (4, 2, 64, True),
                                           (4, 2, 96, True), (6, 3, 128, False)])
def test_decode_rope_append_matches_in_place_kernel(hq, hkv, D, norm):
    """cd_decode_rope_append = cd_qk_norm_rope at the device-side position + the new k / v rows
    stored at that position of the caches; the rest of the caches is untouched."""
    from complexity_deep_b200 import ops
    B, cap, pos = 5, 40, 17
    g = torch.Generator().manual_seed(hq * D)
    qkv = torch.randn(B, (hq + 2 * hkv) * D, generator=g).to(BF).cuda()
    qw = (torch.randn(D, generator=g) * 0.1 + 1).to(BF).cuda() if norm else None
    kw = (torch.randn(D, generator=g) * 0.1 + 1).to(BF).cuda() if norm else None
    ang = torch.outer(torch.arange(cap).float(), 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D)))
    cos, sin = torch.cat([ang, ang], -1).cos().cuda(), torch.cat([ang, ang], -1).sin().cuda()
    ref = ops.qk_norm_rope_(qkv.clone(), qw, kw, cos, sin, 1e-6, 1, pos, hq, hkv, D)
    big_k = torch.full((B, hkv, cap + 8, D), 7.0, dtype=BF, device="cuda")   # strided views
    big_v = torch.full((B, hkv, cap + 8, D), 7.0, dtype=BF, device="cuda")
    kc, vc = big_k[:, :, :cap], big_v[:, :, :cap]
    p = torch.tensor([pos], dtype=torch.int32, device="cuda")
    got = ops.decode_rope_append(qkv.clone(), qw, kw, cos, sin, 1e-6, hq, hkv, D, kc, vc, p)
    assert torch.equal(got, ref)
    assert torch.equal(kc[:, :, pos], ref[:, hq * D:(hq + hkv) * D].view(B, hkv, D))
    assert torch.equal(vc[:, :, pos], ref[:, (hq + hkv) * D:].view(B, hkv, D))
    untouched = torch.ones(cap + 8, dtype=torch.bool)
    untouched[pos] = False
    assert bool((big_k[:, :, untouched] == 7.0).all()) and bool((big_v[:, :, untouched] == 7.0).all())
    p.fill_(cap)                           # outside the cache: nothing is written anywhere
    before = (big_k.clone(), big_v.clone())
    ops.decode_rope_append(qkv.clone(), qw, kw, cos, sin, 1e-6, hq, hkv, D, kc, vc, p)
    assert torch.equal(big_k, before[0]) and torch.equal(big_v, before[1])


def _decode_model():
    import complexity_deep_b200 as cd
    torch.manual_seed(0)
    cfg = cd.ComplexityConfig(vocab_size=512, hidden_size=256, intermediate_size=512,
                              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                              num_experts=4)
    model = cd.ComplexityModel(cfg)
    with torch.no_grad():
        model.mu_init.normal_(0, 0.5)
    return cfg, model.to(device="cuda", dtype=BF).eval()


def test_static_cache_steps_equal_growing_cache_steps():
    """Five decode steps on a StaticKVCache (device-side position, fixed launches) give the
    same logits, bit for bit, as the same steps on the growing cache with an all-zero mask;
    the eager static path and its CUDA-graph replay (DecodeGraph) agree too, and the last
    step agrees with the oracle run over the whole sequence."""
    from complexity_deep_b200.core.attention import StaticKVCache
    from complexity_deep_b200.models import DecodeGraph
    cfg, model = _decode_model()
    B, P, steps = 3, 10, 5
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (B, P + steps), generator=g).cuda()
    with torch.no_grad():
        pre = model(ids[:, :P], use_cache=True)
        # growing cache, zero additive mask
        past, dyn = pre.past_key_values, []
        for s in range(steps):
            mask = torch.zeros(B, 1, 1, P + s + 1, dtype=BF, device="cuda")
            out = model(ids[:, P + s:P + s + 1], attention_mask=mask, past_key_values=past,
                        use_cache=True)
            past = out.past_key_values
            dyn.append(out.logits.clone())
        # static cache, eager
        cache = StaticKVCache(cfg.num_hidden_layers, B, 2, 64, P + steps + 3, "cuda")
        cache.load(pre.past_key_values)
        for s in range(steps):
            out = model(ids[:, P + s:P + s + 1], past_key_values=cache.layers, use_cache=True)
            cache.advance()
            assert torch.equal(out.logits, dyn[s]), s
        assert cache.length == P + steps
        assert torch.equal(cache.k[1][:, :, :P + steps], past[1][0])
        assert torch.equal(cache.v[0][:, :, :P + steps], past[0][1])
    # static cache, graph replay
    dec = DecodeGraph(model, batch=B, capacity=P + steps)
    assert torch.equal(dec.prefill(ids[:, :P]), pre.logits)
    for s in range(steps):
        assert torch.equal(dec.step(ids[:, P + s:P + s + 1]), dyn[s]), s
    with pytest.raises(RuntimeError):
        dec.step(ids[:, :1])               # cache full
    # oracle over the whole sequence (fp32 on the bf16-rounded weights)
    state = {k: (v.float().cpu() if v.is_floating_point() else v.cpu())
             for k, v in model.state_dict().items()}
    ref, _ = oracle.model_forward(state, cfg.to_dict(), ids.cpu())
    _close(dyn[-1][:, 0], ref[:, -1])
