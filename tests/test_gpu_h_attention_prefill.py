"""cd_attention_prefill (causal prompt attention on tcgen05, S / P / O in tensor memory) through
the C ABI against fp32 softmax attention in the reference's order of operations
(complexity_deep/core/attention.py:163-177: repeat_interleave of the KV heads, then
scaled_dot_product_attention(is_causal=True)) on the same bf16-rounded q, k, v.

Tolerance: max|y - ref| / max|ref| <= 2e-2 and mean|y - ref| <= 2e-3 (outputs are averages of
unit-scale values, rms <= 1, so the bound applies as written)."""
import pytest
import torch
import torch.nn.functional as F

from conftest import assert_close

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _reference(qkv, B, S, hq, hkv, D):
    x = qkv.float().view(B, S, hq + 2 * hkv, D)
    q = x[:, :, :hq].transpose(1, 2)
    k = x[:, :, hq:hq + hkv].transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    v = x[:, :, hq + hkv:].transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    out = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    return out.transpose(1, 2).reshape(B * S, hq * D)


@pytest.mark.parametrize("B,S,hq,hkv,D", [
    (2, 128, 4, 2, 128),      # one full tile per sequence
    (1, 256, 2, 1, 128),      # one pair of tiles
    (2, 300, 4, 2, 128),      # ragged: last tile partly filled, odd number of tiles
    (3, 77, 12, 4, 64),       # shorter than a tile, three query heads per KV head, D 64
    (1, 513, 4, 4, 128),      # no grouping, one row in the last tile
    (2, 1000, 6, 2, 64),
    (1, 2048, 16, 8, 128),    # the 1B configuration's sequence
    (4, 1, 2, 1, 128),        # single token
    (1, 4096, 2, 1, 128),     # 32 KV tiles: both ring stages wrap many times
])
def test_attention_prefill_vs_fp32_softmax(B, S, hq, hkv, D):
    from complexity_deep_b200 import ops
    g = torch.Generator().manual_seed(B * S + hq + D)
    qkv = torch.randn(B * S, (hq + 2 * hkv) * D, generator=g).to(BF)
    out = ops.attention_prefill(qkv.cuda(), B, S, hq, hkv, D)
    ops.status_fetch()
    assert_close(out, _reference(qkv, B, S, hq, hkv, D), what=f"prefill attention {B}x{S} hq{hq} hkv{hkv} D{D}")


def test_attention_prefill_large_scores_rescale_path():
    """Scores that grow along the sequence (keys scaled up with position) force the running
    maximum to move by more than the rescale threshold many times: exercises the in-TMEM
    rescale of O and of the row sum."""
    from complexity_deep_b200 import ops
    B, S, hq, hkv, D = 1, 1024, 2, 1, 128
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B * S, hq + 2 * hkv, D, generator=g)
    ramp = torch.linspace(0.2, 6.0, S).view(S, 1)
    x[:, hq:hq + hkv] *= ramp.view(S, 1, 1)        # keys: later positions score higher
    qkv = x.view(B * S, -1).to(BF)
    out = ops.attention_prefill(qkv.cuda(), B, S, hq, hkv, D)
    ops.status_fetch()
    assert_close(out, _reference(qkv, B, S, hq, hkv, D), what="prefill attention, growing scores")


def test_attention_module_uses_kernel_and_matches_sdpa_path(monkeypatch):
    """ComplexityAttention on a prompt: the kernel path against the same module routed through
    scaled_dot_product_attention (same projections, same rounding points before attention)."""
    import complexity_deep_b200 as cd
    from complexity_deep_b200 import ops
    from complexity_deep_b200.core import attention as attn_mod
    torch.manual_seed(0)
    m = cd.ComplexityAttention(512, 4, 2).to(device="cuda", dtype=BF).eval()
    x = torch.randn(2, 200, 512, device="cuda").to(BF)
    mu = torch.randn(2, 200, 512, device="cuda").to(BF)
    with torch.no_grad():
        monkeypatch.setattr(attn_mod, "_PREFILL_KERNEL", True)
        ops.PROFILE.reset(True)
        y, kv = m(x, mu_prev=mu, use_cache=True)
        names = {e[0] for e in ops.PROFILE.events}
        ops.PROFILE.reset(False)
        assert "attention_prefill" in names and "sdpa" not in names
        monkeypatch.setattr(attn_mod, "_PREFILL_KERNEL", False)
        y2, _ = m(x, mu_prev=mu)
    ops.status_fetch()
    assert kv[0].shape == (2, 2, 200, 128)
    assert_close(y, y2.float(), what="attention module: kernel vs SDPA route")
