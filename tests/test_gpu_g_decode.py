"""Decode-side kernels: single-query attention over a KV cache (cd_decode_attention) and the
narrow-tile GEMM path used when there are few rows, against fp32 references on the same
bf16-rounded inputs.  Tolerance: max|y - ref| / max|ref| <= 2e-2 and mean|y - ref| <= 2e-3 *
max(1, rms(ref)) (outputs are rounded to bf16 once)."""
import pytest
import torch

from oracle import complexity_oracle as oracle

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _close(got, ref, max_rel=2e-2, mean_abs=2e-3):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all()
    mr, ma = oracle.error_metrics(got, ref)
    rms = float(ref.double().pow(2).mean().sqrt())
    assert mr <= max_rel and ma <= mean_abs * max(1.0, rms), (mr, ma, rms)


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
