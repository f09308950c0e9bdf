"""Generates the golden fixtures in this directory by running the REFERENCE implementation
(Complexity-ML/complexity-deep) on the CPU.

    python tests/golden/make_golden.py [/path/to/reference]

The reference checkout is only needed to (re)generate the fixtures; the tests read the
committed files.  Everything is seeded; fp32 throughout.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("COMPLEXITY_DEEP_REFERENCE")
if not REF:
    raise SystemExit("usage: make_golden.py <reference checkout> (or set COMPLEXITY_DEEP_REFERENCE)")
sys.path.insert(0, REF)
from complexity_deep.core.attention import ComplexityAttention  # noqa: E402
from complexity_deep.core.layer import MuGuidance, TransformerBlock  # noqa: E402
from complexity_deep.core.normalization import RMSNorm  # noqa: E402
from complexity_deep.core.token_routed_mlp import TokenRoutedMLP  # noqa: E402
from complexity_deep.models import ComplexityConfig, ComplexityModel  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def zipf_p(V, s):
    r = torch.arange(1, V + 1, dtype=torch.float64)
    p = r.pow(-s)
    return p / p.sum()


def zipf_ids(V, s, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.multinomial(zipf_p(V, s).float(), n, replacement=True, generator=g)


def save(name, obj):
    torch.save(obj, os.path.join(OUT, name))
    print(name, os.path.getsize(os.path.join(OUT, name)), "bytes")


@torch.no_grad()
def main():
    # ---------------------------------------------------------------- routing tables
    p32k = zipf_p(32000, 1.1).float()
    table_e8 = TokenRoutedMLP._build_token_mapping(32000, 8, p32k)
    table_e4 = TokenRoutedMLP._build_token_mapping(32000, 4, p32k)
    p100k = zipf_p(100000, 1.0).float()
    table_e32 = TokenRoutedMLP._build_token_mapping(100000, 32, p100k)
    ids = zipf_ids(32000, 1.1, 4096)
    eid = table_e8[ids.clamp(0, 31999)]
    order = torch.sort(eid, stable=True).indices
    np.savez_compressed(
        os.path.join(OUT, "routing.npz"),
        table_e8=table_e8.numpy().astype(np.uint8),
        table_e4=table_e4.numpy().astype(np.uint8),
        table_e32_sha256=np.frombuffer(
            hashlib.sha256(table_e32.numpy().astype(np.int64).tobytes()).digest(), dtype=np.uint8),
        table_mod_e4_head=(TokenRoutedMLP._build_token_mapping(64, 4, None)).numpy().astype(np.uint8),
        ids=ids.numpy().astype(np.int32),
        expert_ids=eid.numpy().astype(np.int32),
        counts=torch.bincount(eid, minlength=8).numpy().astype(np.int32),
        perm=order.numpy().astype(np.int32),
    )
    print("routing.npz", os.path.getsize(os.path.join(OUT, "routing.npz")), "bytes")

    # ---------------------------------------------------------------- rmsnorm
    torch.manual_seed(0)
    norm = RMSNorm(96, eps=1e-6)
    norm.weight.copy_(torch.randn(96) * 0.1 + 1.0)
    xn = torch.randn(3, 7, 96)
    save("rmsnorm.pt", {"weight": norm.weight.clone(), "x": xn, "out": norm(xn)})

    # ---------------------------------------------------------------- MoE layer
    torch.manual_seed(0)
    V, E, H, I_e = 512, 4, 64, 48
    freqs = zipf_p(V, 1.1).float()
    mlp = TokenRoutedMLP(H, I_e * E, E, V, True, freqs).eval()
    for lin in (mlp.shared_gate, mlp.shared_up, mlp.shared_down):
        lin.weight.normal_(0, 0.02)
    x = torch.randn(2, 40, H)
    tid = zipf_ids(V, 1.1, 80, seed=1).view(2, 40)
    tid[0, 0], tid[0, 1], tid[1, 5] = -3, 600, 511          # out of range -> clamp
    save("moe_layer.pt", {
        "config": dict(hidden_size=H, intermediate_size=I_e * E, num_experts=E, vocab_size=V),
        "state": {k: v.clone() for k, v in mlp.state_dict().items()},
        "x": x, "token_ids": tid, "out": mlp(x, tid), "out_no_ids": mlp(x, None),
    })
    # modulo table, no shared expert, one expert never hit
    torch.manual_seed(1)
    mlp2 = TokenRoutedMLP(H, I_e * E, E, V, False, None).eval()
    tid2 = (torch.randint(0, V // 4, (2, 24)) * 4 + torch.randint(0, 2, (2, 24)))  # experts 0, 1
    x2 = torch.randn(2, 24, H)
    save("moe_layer_modulo.pt", {
        "config": dict(hidden_size=H, intermediate_size=I_e * E, num_experts=E, vocab_size=V),
        "state": {k: v.clone() for k, v in mlp2.state_dict().items()},
        "x": x2, "token_ids": tid2, "out": mlp2(x2, tid2),
    })

    # ---------------------------------------------------------------- attention
    torch.manual_seed(0)
    att = ComplexityAttention(64, 4, 2).eval()
    xa, mu = torch.randn(2, 12, 64), torch.randn(2, 12, 64)
    out_a, kv = att(xa, mu_prev=mu, use_cache=True)
    out_nomu, _ = att(xa)
    x1, mu1 = torch.randn(2, 1, 64), torch.randn(2, 1, 64)
    step_quirk, kv2 = att(x1, past_key_value=kv, use_cache=True, mu_prev=mu1)
    zero_mask = torch.zeros(2, 1, 1, 13)
    step_full, _ = att(x1, attention_mask=zero_mask, past_key_value=kv, use_cache=True, mu_prev=mu1)
    save("attention.pt", {
        "state": {k: v.clone() for k, v in att.state_dict().items()},
        "x": xa, "mu_prev": mu, "out": out_a, "k": kv[0].clone(), "v": kv[1].clone(),
        "out_no_mu": out_nomu, "x_step": x1, "mu_step": mu1, "out_step_causal_flag": step_quirk,
        "out_step_zero_mask": step_full, "k_step": kv2[0].clone(),
    })

    # ---------------------------------------------------------------- mu guidance + block
    torch.manual_seed(0)
    mg = MuGuidance(64).eval()
    mg.mu_proj.weight.normal_(0, 0.02)
    mg.mu.copy_(torch.randn(64) * 1.5 + 1.0)   # values on both sides of the clamp range
    xm = torch.randn(2, 9, 64)
    save("mu_guidance.pt", {"state": {k: v.clone() for k, v in mg.state_dict().items()},
                            "x": xm, "out": mg(xm)})

    torch.manual_seed(0)
    blk = TransformerBlock(64, 128, 4, 2, num_experts=4, vocab_size=256,
                           token_frequencies=zipf_p(256, 1.1).float()).eval()
    blk.mu_guidance.mu_proj.weight.normal_(0, 0.02)
    xb, mub = torch.randn(2, 16, 64), torch.randn(2, 16, 64)
    tb = zipf_ids(256, 1.1, 32, seed=2).view(2, 16)
    hb, _, mu_out = blk(xb, token_ids=tb, mu_prev=mub)
    save("block.pt", {"state": {k: v.clone() for k, v in blk.state_dict().items()},
                      "x": xb, "mu_prev": mub, "token_ids": tb, "hidden": hb, "mu": mu_out})

    # ---------------------------------------------------------------- tiny model
    torch.manual_seed(0)
    cfg = ComplexityConfig(vocab_size=256, hidden_size=64, intermediate_size=128,
                           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                           num_experts=4)
    model = ComplexityModel(cfg).eval()
    table = TokenRoutedMLP._build_token_mapping(256, 4, zipf_p(256, 1.1).float())
    for layer in model.layers:
        layer.mlp.token_to_expert.copy_(table)
    model.mu_init.normal_(0, 0.5)
    mids = zipf_ids(256, 1.1, 32, seed=3).view(2, 16)
    full = model(mids, labels=mids, use_cache=True)
    nxt = zipf_ids(256, 1.1, 2, seed=4).view(2, 1)
    step = model(nxt, attention_mask=torch.zeros(2, 1, 1, 17), past_key_values=full.past_key_values,
                 use_cache=True)
    save("model_tiny.pt", {
        "config": cfg.to_dict(),
        "state": {k: v.clone() for k, v in model.state_dict().items()},
        "input_ids": mids, "logits": full.logits, "loss": full.loss,
        "next_ids": nxt, "step_logits": step.logits,
    })

    # ---------------------------------------------------------------- config switches
    variants = []
    for flags in (dict(use_mu_guidance=False), dict(use_qk_norm=False), dict(shared_expert=False),
                  dict(use_token_routed_mlp=False), dict(tie_word_embeddings=False),
                  dict(num_experts=1)):
        torch.manual_seed(7)
        base = dict(vocab_size=48, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                    num_attention_heads=2, num_key_value_heads=1, num_experts=2)
        base.update(flags)
        vcfg = ComplexityConfig(**base)
        vm = ComplexityModel(vcfg).eval()
        vids = zipf_ids(48, 1.1, 12, seed=9).view(2, 6)
        variants.append({"config": vcfg.to_dict(),
                         "state": {k: v.clone() for k, v in vm.state_dict().items()},
                         "input_ids": vids, "logits": vm(vids).logits})
    save("model_variants.pt", variants)


if __name__ == "__main__":
    main()
