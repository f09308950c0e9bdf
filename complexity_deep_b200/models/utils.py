"""Model factory and parameter accounting (complexity_deep/models/utils.py:9-98)."""
from __future__ import annotations

from .config import ComplexityConfig
from .modeling import ComplexityModel

SIZE_PRESETS = {
    "tiny": ComplexityConfig.complexity_tiny,
    "20m": ComplexityConfig.complexity_20m,
    "small": ComplexityConfig.complexity_small,
    "150m": ComplexityConfig.complexity_150m,
    "350m": ComplexityConfig.complexity_350m,
    "1b": ComplexityConfig.complexity_1b,
}


def create_complexity_model(size: str = "150m", vocab_size: int = 100_000, **overrides
                            ) -> ComplexityModel:
    """Builds a model from a preset name; unknown override keys are ignored."""
    if size not in SIZE_PRESETS:
        raise ValueError(f"Unknown size '{size}'. Choose from {list(SIZE_PRESETS.keys())}")
    config = SIZE_PRESETS[size]()
    config.vocab_size = vocab_size
    for key, value in overrides.items():
        if hasattr(config, key):
            setattr(config, key, value)
    return ComplexityModel(config)


def count_parameters(config: ComplexityConfig) -> dict:
    """Analytic parameter counts per component (shared expert as wide as one routed expert)."""
    H, I, V, L = (config.hidden_size, config.intermediate_size, config.vocab_size,
                  config.num_hidden_layers)
    hq, hkv = config.num_attention_heads, config.num_key_value_heads
    D = H // hq
    q_dim, kv_dim = hq * D, hkv * D

    qkv = q_dim * H + 2 * kv_dim * H
    attention = qkv + H * H                      # + o_proj
    if config.use_mu_guidance:
        attention += qkv                         # mu_to_q / k / v
    if config.use_qk_norm:
        attention += 2 * D

    if config.use_token_routed_mlp:
        E = config.num_experts
        per_expert = 3 * H * (I // E)
        mlp = E * per_expert + (per_expert if config.shared_expert else 0)
    else:
        mlp = 3 * H * I

    mu = H + H * H if config.use_mu_guidance else 0
    per_layer = attention + mlp + 2 * H + mu
    embedding = V * H
    total = embedding + L * per_layer + H
    return {
        "total": total,
        "embedding": embedding,
        "per_layer": per_layer,
        "attention_per_layer": attention,
        "mlp_per_layer": mlp,
        "mu_per_layer": mu,
        "num_layers": L,
        "memory_bf16_gb": total * 2 / (1024 ** 3),
    }
