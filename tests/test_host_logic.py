"""Host-side mirror of the reference interface: names, constructor signatures, state_dict
layout, table construction, weight packing, caches, and the no-fallback rule."""
import inspect
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, load_golden
import complexity_deep_b200 as cd
from complexity_deep_b200 import ops
from complexity_deep_b200.core._cache import DerivedCache
from complexity_deep_b200.core.token_routed_mlp import ROUTING_CACHE
from complexity_deep_b200.models import (CausalLMOutput, ComplexityConfig, ComplexityModel,
                                         ModelOutput, count_parameters, create_complexity_model)
from oracle import complexity_oracle as oracle


def _shapes(sd):
    return {k: (tuple(v.shape), v.dtype) for k, v in sd.items()}


def test_public_names():
    for name in ["RMSNorm", "RotaryEmbedding", "ComplexityAttention", "SwiGLU", "TokenRoutedMLP",
                 "TransformerBlock", "MuGuidance", "ComplexityConfig", "ComplexityModel",
                 "create_complexity_model", "count_parameters"]:
        assert hasattr(cd, name)
    assert CausalLMOutput().logits is None and ModelOutput().last_hidden_state is None


def test_constructor_signatures():
    sig = lambda c: list(inspect.signature(c.__init__).parameters)[1:]
    assert sig(cd.TokenRoutedMLP) == ["hidden_size", "intermediate_size", "num_experts",
                                      "vocab_size", "shared_expert", "token_frequencies"]
    assert sig(cd.ComplexityAttention) == ["hidden_size", "num_attention_heads",
                                           "num_key_value_heads", "max_position_embeddings",
                                           "rope_theta", "attention_dropout", "use_qk_norm"]
    assert sig(cd.TransformerBlock) == [
        "hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads",
        "max_position_embeddings", "rms_norm_eps", "rope_theta", "attention_dropout",
        "use_token_routed_mlp", "num_experts", "vocab_size", "shared_expert", "token_frequencies",
        "use_qk_norm", "use_mu_guidance"]
    assert sig(cd.MuGuidance) == ["hidden_size", "mu_min", "mu_max"]
    assert sig(cd.RMSNorm) == ["hidden_size", "eps"]
    fwd = list(inspect.signature(cd.TransformerBlock.forward).parameters)[1:]
    assert fwd == ["hidden_states", "attention_mask", "past_key_value", "use_cache", "token_ids",
                   "mu_prev"]
    fwd = list(inspect.signature(ComplexityModel.forward).parameters)[1:]
    assert fwd == ["input_ids", "attention_mask", "labels", "past_key_values", "use_cache"]


def test_state_dict_layout_matches_reference_checkpoints():
    g = load_golden("model_tiny.pt")
    model = ComplexityModel(ComplexityConfig.from_dict(g["config"]))
    assert _shapes(model.state_dict()) == _shapes(g["state"])
    missing, unexpected = model.load_state_dict(g["state"], strict=True)
    assert not missing and not unexpected
    assert model.lm_head.weight is model.embed_tokens.weight

    g = load_golden("moe_layer.pt")
    mlp = cd.TokenRoutedMLP(**g["config"], shared_expert=True)
    assert _shapes(mlp.state_dict()) == _shapes(g["state"])
    g = load_golden("attention.pt")
    assert _shapes(cd.ComplexityAttention(64, 4, 2).state_dict()) == _shapes(g["state"])
    g = load_golden("block.pt")
    blk = cd.TransformerBlock(64, 128, 4, 2, num_experts=4, vocab_size=256)
    assert _shapes(blk.state_dict()) == _shapes(g["state"])


def test_init_statistics_follow_reference_rules():
    torch.manual_seed(0)
    cfg = ComplexityConfig(vocab_size=512, hidden_size=128, intermediate_size=256,
                           num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2)
    m = ComplexityModel(cfg)
    rstd = 0.02 / (2 * 4) ** 0.5
    l0 = m.layers[0]
    assert abs(l0.self_attn.q_proj.weight.std().item() - 0.02) < 2e-3
    assert abs(l0.mu_guidance.mu_proj.weight.std().item() - 0.02) < 2e-3   # re-drawn, not zero
    assert abs(l0.self_attn.o_proj.weight.std().item() - rstd) < 1e-3
    assert abs(l0.mlp.down_proj_w.std().item() - rstd) < 1e-3
    assert abs(l0.mlp.shared_down.weight.std().item() - rstd) < 1e-3
    assert abs(l0.mlp.gate_proj_w.std().item() - 0.02) < 2e-3
    assert torch.all(m.mu_init == 0) and torch.all(l0.mu_guidance.mu == 1.0)
    assert torch.equal(l0.mlp.token_to_expert, torch.arange(512) % 4)


def test_token_mapping_bit_exact_with_reference_tables():
    g = np.load(os.path.join(GOLDEN, "routing.npz"))
    p = oracle.zipf_probabilities(32000, 1.1).float()
    t8 = cd.TokenRoutedMLP._build_token_mapping(32000, 8, p)
    assert t8.dtype == torch.int64
    assert np.array_equal(t8.numpy(), g["table_e8"].astype(np.int64))
    t4 = cd.TokenRoutedMLP._build_token_mapping(32000, 4, p)
    assert np.array_equal(t4.numpy(), g["table_e4"].astype(np.int64))
    # ties (equal frequencies) follow the reference's argsort + first-minimum rule
    f = torch.tensor([0.25, 0.25, 0.25, 0.25, 0.1, 0.1, 0.0, 0.0])
    assert np.array_equal(cd.TokenRoutedMLP._build_token_mapping(8, 3, f).numpy(),
                          oracle.build_token_mapping(8, 3, f))
    with pytest.raises(ValueError):
        cd.TokenRoutedMLP._build_token_mapping(8, 3, torch.ones(7))


def test_config_presets_and_serialisation():
    c = ComplexityConfig.complexity_1b()
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.num_attention_heads,
            c.num_key_value_heads, c.num_experts, c.vocab_size) == (2048, 5632, 24, 16, 8, 8, 100000)
    d = c.to_dict()
    d["unknown_key"] = 1
    assert ComplexityConfig.from_dict(d) == c
    assert ComplexityConfig().num_hidden_layers == 12 and ComplexityConfig().eos_token_id == 0
    n = count_parameters(ComplexityConfig(vocab_size=32000, hidden_size=768, num_hidden_layers=18))
    assert n["total"] == n["embedding"] + 18 * n["per_layer"] + 768
    with pytest.raises(ValueError):
        create_complexity_model("nope")
    m = create_complexity_model("tiny", vocab_size=128, num_hidden_layers=1, bogus=3)
    assert len(m.layers) == 1 and m.config.vocab_size == 128


def test_choose_block_n():
    assert ops.choose_block_n(5632) == 256 and ops.choose_block_n(704) == 256
    assert ops.choose_block_n(64) == 128 and ops.choose_block_n(48) == 128
    assert ops.choose_block_n(704, rows=4096) == 256
    # few rows: narrowest tile with at most one tile per SM (148), experts count as row tiles
    assert ops.choose_block_n(704, rows=256, sm_count=148) == 32            # shared expert: 2 x 44 tiles
    assert ops.choose_block_n(704, rows=256, groups=8, sm_count=148) == 128  # 8 x 11 tiles
    assert ops.choose_block_n(5632, rows=32, sm_count=148) == 128           # 88 tiles
    assert ops.choose_block_n(5632, rows=32, groups=8, sm_count=148) == 256  # nothing fits
    assert ops.choose_block_n(2816) == 256 and ops.choose_block_n(512) == 256


def test_derived_cache_tracks_in_place_mutation():
    cache = DerivedCache()
    w = torch.ones(4)
    calls = []
    make = lambda: (calls.append(1), w * 2)[1]
    a = cache.get("x", (w,), make)
    b = cache.get("x", (w,), make)
    assert a is b and len(calls) == 1
    w.mul_(3)                                  # what the reference's ablation scripts do
    c = cache.get("x", (w,), make)
    assert len(calls) == 2 and torch.equal(c, torch.full((4,), 6.0))
    w2 = w.clone()
    cache.get("x", (w2,), make)
    assert len(calls) == 3


def test_no_cpu_fallback():
    mlp = cd.TokenRoutedMLP(64, 128, 4, 256)
    x = torch.randn(1, 4, 64)
    ids = torch.randint(0, 256, (1, 4))
    with pytest.raises(RuntimeError, match="no CPU path|CUDA"):
        mlp(x, ids)
    with pytest.raises(RuntimeError):
        cd.RMSNorm(64)(x)
    with pytest.raises(RuntimeError):
        cd.MuGuidance(64)(x)
    ROUTING_CACHE.clear()


def test_table_validation():
    mlp = cd.TokenRoutedMLP(64, 128, 4, 256)
    mlp.token_to_expert[3] = 7
    with pytest.raises(ValueError, match="outside"):
        mlp._table_signature()
    mlp.token_to_expert[3] = 1
    sig = mlp._table_signature()
    assert sig == mlp._table_signature()
    mlp.token_to_expert.zero_()               # ablation: in-place edit must change the signature
    assert mlp._table_signature() != sig


def test_kv_cache_append_in_place_semantics():
    """The growing KV view equals torch.cat, reuses its buffer on a linear decode, and falls
    back to a copy when the same past is extended twice (branching)."""
    from complexity_deep_b200.core.attention import _kv_append
    g = torch.Generator().manual_seed(0)
    past = torch.randn(2, 2, 5, 4, generator=g)
    n1, n2, n3 = (torch.randn(2, 2, 1, 4, generator=g) for _ in range(3))
    a = _kv_append(past, n1)
    assert torch.equal(a, torch.cat([past, n1], 2))
    b = _kv_append(a, n2)
    assert torch.equal(b, torch.cat([past, n1, n2], 2))
    assert b._cd_kv.buf.data_ptr() == a._cd_kv.buf.data_ptr()      # no copy on the second step
    assert torch.equal(a, torch.cat([past, n1], 2))                # the shorter view is intact
    c = _kv_append(a, n3)                                          # branch from the older view
    assert torch.equal(c, torch.cat([past, n1, n3], 2))
    assert torch.equal(b, torch.cat([past, n1, n2], 2))            # first branch not clobbered
    assert c._cd_kv.buf.data_ptr() != b._cd_kv.buf.data_ptr()


def test_forward_only_is_loud():
    """An activation with autograd history is refused (no silent loss of gradients)."""
    x = torch.randn(1, 4, 64, requires_grad=True)
    with pytest.raises(RuntimeError, match="forward pass only"):
        cd.RMSNorm(64)(x)
    with pytest.raises(RuntimeError, match="forward pass only"):
        cd.TokenRoutedMLP(64, 128, 4, 256)(x, torch.zeros(1, 4, dtype=torch.long))
    model = create_complexity_model("tiny", vocab_size=64, num_hidden_layers=1)
    with pytest.raises(RuntimeError, match="forward pass only"):
        model(torch.zeros(1, 4, dtype=torch.long))          # grad mode: embedding output requires grad


def test_static_kv_cache_bookkeeping():
    """Host side of the fixed-capacity decode cache: load from a prefill cache, position
    scalars (cached tokens, keys visible to the next step), capacity checks."""
    from complexity_deep_b200.core.attention import StaticKVCache
    cache = StaticKVCache(num_layers=2, batch=3, kv_heads=2, head_dim=8, capacity=6, device="cpu",
                          dtype=torch.float32)
    assert cache.state.tolist() == [0, 1] and cache.length == 0 and len(cache.layers) == 2
    past = [(torch.randn(3, 2, 4, 8), torch.randn(3, 2, 4, 8)) for _ in range(2)]
    cache.load(past)
    assert cache.state.tolist() == [4, 5] and cache.length == 4
    assert torch.equal(cache.layers[1].k[:, :, :4], past[1][0])
    assert torch.equal(cache.layers[0].v[:, :, :4], past[0][1])
    assert float(cache.k[0][:, :, 4:].abs().sum()) == 0.0
    cache.advance()
    assert cache.state.tolist() == [5, 6] and cache.length == 5
    with pytest.raises(ValueError):
        cache.load([(torch.zeros(3, 2, 7, 8), torch.zeros(3, 2, 7, 8))] * 2)
    with pytest.raises(ValueError):
        cache.set_length(7)


def test_rotary_tables_grow_geometrically():
    """Positions past the configured maximum rebuild the tables once per doubling, not on
    every decode step; values do not depend on the table length."""
    from complexity_deep_b200.core.rotary import RotaryEmbedding
    rot = RotaryEmbedding(16, max_seq_len=8)
    cos_a, _ = rot.tables_fp32(9)
    assert rot.max_seq_len == 16 and cos_a.shape[0] == 16
    ptr = cos_a.data_ptr()
    for n in range(10, 17):
        assert rot.tables_fp32(n)[0].data_ptr() == ptr
    cos_b, sin_b = rot.tables_fp32(17)
    assert rot.max_seq_len == 32
    assert torch.equal(cos_b[:16], cos_a)
    ref = RotaryEmbedding(16, max_seq_len=32)
    assert torch.equal(ref.cos_cached, cos_b) and torch.equal(ref.sin_cached, sin_b)


def test_expert_parallel_rejects_oversized_batch_before_any_collective(monkeypatch):
    """A rank whose batch does not fit the exchange buffers must raise before it enters any
    collective or launches anything: it then has nothing in flight, and since no rank ever
    sends more than max_tokens_per_rank rows no receive buffer can be overrun."""
    from types import SimpleNamespace
    from complexity_deep_b200 import expert_parallel as epm
    ep = epm.ExpertParallelMoE.__new__(epm.ExpertParallelMoE)
    ep.exchange, ep.max_tokens = "peer", 8
    ep.mlp = SimpleNamespace(num_experts=4)

    def reached(*a, **k):
        raise AssertionError("a collective / launch was reached before the size check")
    monkeypatch.setattr(ep, "peer_plan_for", reached, raising=False)
    monkeypatch.setattr(ep, "_peer_buffers", reached, raising=False)
    monkeypatch.setattr(epm.dist, "all_gather_into_tensor", reached)
    routing = SimpleNamespace(perm=torch.zeros(9, dtype=torch.int32), num_experts=4)
    with pytest.raises(ValueError, match="max_tokens_per_rank"):
        ep.forward_sorted(torch.zeros(9, 4), routing, None)
    short = SimpleNamespace(perm=torch.zeros(5, dtype=torch.int32), num_experts=4)
    with pytest.raises(ValueError, match="token_ids"):
        ep.forward_sorted(torch.zeros(8, 4), short, None)
    ep.max_tokens = 0
    ok = SimpleNamespace(perm=torch.zeros(8, dtype=torch.int32), num_experts=4)
    with pytest.raises(ValueError, match="needs max_tokens_per_rank"):
        ep.forward_sorted(torch.zeros(8, 4), ok, None)


def test_reference_import_lines_resolve_to_this_package():
    """The reference's own import lines, verbatim, in a fresh interpreter with only this
    repository on the path: they must resolve to the classes of complexity_deep_b200."""
    import subprocess
    import sys
    from conftest import ROOT
    code = """
from complexity_deep import (RMSNorm, RotaryEmbedding, ComplexityAttention, SwiGLU,
                             TokenRoutedMLP, TransformerBlock, MuGuidance)
from complexity_deep import ComplexityConfig, ComplexityModel, create_complexity_model, count_parameters
from complexity_deep.models import (ComplexityConfig, ComplexityModel, CausalLMOutput, ModelOutput,
                                    create_complexity_model, count_parameters)
from complexity_deep.core import (RMSNorm, RotaryEmbedding, apply_rotary_pos_emb, ComplexityAttention,
                                  SwiGLU, TokenRoutedMLP, TransformerBlock, MuGuidance)
from complexity_deep.core.token_routed_mlp import TokenRoutedMLP as T2
from complexity_deep.core.layer import TransformerBlock as B2, MuGuidance as M2
from complexity_deep.core.attention import ComplexityAttention as A2
from complexity_deep.core.normalization import RMSNorm as N2
from complexity_deep.models.modeling import ComplexityModel as CM2
from complexity_deep.models.config import ComplexityConfig as CC2
import complexity_deep, complexity_deep_b200 as impl
assert TokenRoutedMLP is impl.TokenRoutedMLP is T2 and ComplexityModel is impl.ComplexityModel is CM2
assert TransformerBlock is B2 and MuGuidance is M2 and ComplexityAttention is A2 and RMSNorm is N2
assert ComplexityConfig is CC2 and complexity_deep.__version__ == "1.0.0"
m = create_complexity_model("tiny", vocab_size=64, num_hidden_layers=1)
assert type(m).__module__ == "complexity_deep_b200.models.modeling"
print("ok")
"""
    proc = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True,
                          env={**__import__("os").environ, "PYTHONPATH": ROOT})
    assert proc.returncode == 0 and proc.stdout.strip() == "ok", proc.stderr
