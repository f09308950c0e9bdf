"""Pins the CPU oracle against outputs of the reference implementation itself
(fixtures made by tests/golden/make_golden.py).  Integer artefacts must be bit-exact;
fp32 outputs agree to rounding (same torch operators in the same order)."""
import hashlib
import os

import numpy as np
import torch

from conftest import GOLDEN, load_golden
from oracle import complexity_oracle as oracle

TOL = dict(rtol=1e-5, atol=1e-6)


def _routing():
    return np.load(os.path.join(GOLDEN, "routing.npz"))


def test_token_mapping_matches_reference_tables():
    g = _routing()
    p = oracle.zipf_probabilities(32000, 1.1).float()
    assert np.array_equal(oracle.build_token_mapping(32000, 8, p), g["table_e8"].astype(np.int64))
    assert np.array_equal(oracle.build_token_mapping(32000, 4, p), g["table_e4"].astype(np.int64))
    assert np.array_equal(oracle.build_token_mapping(64, 4, None),
                          g["table_mod_e4_head"].astype(np.int64))


def test_token_mapping_large_vocab_digest():
    g = _routing()
    p = oracle.zipf_probabilities(100000, 1.0).float()
    t = oracle.build_token_mapping(100000, 32, p)
    digest = np.frombuffer(hashlib.sha256(t.astype(np.int64).tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(digest, g["table_e32_sha256"])


def test_zipf_ids_match_reference_draw():
    g = _routing()
    assert np.array_equal(oracle.zipf_token_ids(32000, 1.1, 4096).numpy(), g["ids"].astype(np.int64))


def test_route_artefacts():
    g = _routing()
    eid, counts, offsets, perm, inv = oracle.route(g["ids"], g["table_e8"].astype(np.int64), 8)
    assert np.array_equal(eid, g["expert_ids"])
    assert np.array_equal(counts, g["counts"])
    assert np.array_equal(perm, g["perm"])
    assert np.array_equal(offsets, np.concatenate([[0], np.cumsum(g["counts"])]))
    assert np.array_equal(inv[perm], np.arange(perm.size))


def test_route_edge_cases():
    table = np.arange(16, dtype=np.int64) % 4
    eid, counts, offsets, perm, inv = oracle.route(np.zeros(0, np.int64), table, 4)
    assert eid.size == 0 and perm.size == 0 and counts.tolist() == [0, 0, 0, 0]
    assert offsets.tolist() == [0, 0, 0, 0, 0]
    # out-of-range ids clamp; expert 3 unused -> empty segment
    ids = np.array([-5, 0, 1, 2, 99, 4, 5, 6], dtype=np.int64)
    table2 = np.array([0, 1, 2, 0, 1, 2, 0, 1, 2, 0, 1, 2, 0, 1, 2, 2], dtype=np.int64)
    eid, counts, offsets, perm, inv = oracle.route(ids, table2, 4)
    assert eid.tolist() == [0, 0, 1, 2, 2, 1, 2, 0]
    assert counts.tolist() == [3, 2, 3, 0]
    assert perm.tolist() == [0, 1, 7, 2, 5, 3, 4, 6]


def test_rmsnorm():
    g = load_golden("rmsnorm.pt")
    torch.testing.assert_close(oracle.rmsnorm(g["x"], g["weight"], 1e-6), g["out"], **TOL)


def test_moe_layer():
    g = load_golden("moe_layer.pt")
    out = oracle.token_routed_mlp(g["state"], "", g["x"], g["token_ids"])
    torch.testing.assert_close(out, g["out"], **TOL)
    out_all = oracle.token_routed_mlp(g["state"], "", g["x"], None)
    torch.testing.assert_close(out_all, g["out_no_ids"], **TOL)


def test_moe_layer_modulo_no_shared_empty_expert():
    g = load_golden("moe_layer_modulo.pt")
    out = oracle.token_routed_mlp(g["state"], "", g["x"], g["token_ids"])
    torch.testing.assert_close(out, g["out"], **TOL)


def test_attention_prefill_and_decode():
    g = load_golden("attention.pt")
    out, kv = oracle.attention(g["state"], "", g["x"], 4, 2, mu_prev=g["mu_prev"], use_cache=True)
    torch.testing.assert_close(out, g["out"], **TOL)
    torch.testing.assert_close(kv[0], g["k"], **TOL)
    torch.testing.assert_close(kv[1], g["v"], **TOL)
    out_nomu, _ = oracle.attention(g["state"], "", g["x"], 4, 2)
    torch.testing.assert_close(out_nomu, g["out_no_mu"], **TOL)
    # decode step: with mask=None the reference passes is_causal=True (top-left aligned)
    step, kv2 = oracle.attention(g["state"], "", g["x_step"], 4, 2, past_key_value=(g["k"], g["v"]),
                                 use_cache=True, mu_prev=g["mu_step"])
    torch.testing.assert_close(step, g["out_step_causal_flag"], **TOL)
    torch.testing.assert_close(kv2[0], g["k_step"], **TOL)
    full, _ = oracle.attention(g["state"], "", g["x_step"], 4, 2,
                               attention_mask=torch.zeros(2, 1, 1, 13),
                               past_key_value=(g["k"], g["v"]), use_cache=True,
                               mu_prev=g["mu_step"])
    torch.testing.assert_close(full, g["out_step_zero_mask"], **TOL)


def test_mu_guidance():
    g = load_golden("mu_guidance.pt")
    torch.testing.assert_close(oracle.mu_guidance(g["state"], "", g["x"]), g["out"], **TOL)


def test_transformer_block():
    g = load_golden("block.pt")
    h, _, mu = oracle.transformer_block(g["state"], "", g["x"], 4, 2, token_ids=g["token_ids"],
                                        mu_prev=g["mu_prev"])
    torch.testing.assert_close(h, g["hidden"], **TOL)
    torch.testing.assert_close(mu, g["mu"], **TOL)


def test_model_forward_and_decode_step():
    g = load_golden("model_tiny.pt")
    logits, kvs = oracle.model_forward(g["state"], g["config"], g["input_ids"], use_cache=True)
    torch.testing.assert_close(logits, g["logits"], **TOL)
    step, _ = oracle.model_forward(g["state"], g["config"], g["next_ids"],
                                   attention_mask=torch.zeros(2, 1, 1, 17), past_key_values=kvs,
                                   use_cache=True)
    torch.testing.assert_close(step, g["step_logits"], **TOL)
    # loss as the reference computes it (modeling.py:209-217)
    loss = torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, 256),
                                             g["input_ids"][:, 1:].reshape(-1))
    torch.testing.assert_close(loss, g["loss"], **TOL)


def test_model_config_switches():
    """mu guidance off, QK-norm off, no shared expert, dense SwiGLU, untied lm_head, one expert."""
    for g in load_golden("model_variants.pt"):
        logits, _ = oracle.model_forward(g["state"], g["config"], g["input_ids"])
        torch.testing.assert_close(logits, g["logits"], **TOL)
