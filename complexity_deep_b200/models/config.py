"""Hyper-parameters of a Complexity model: same fields, defaults, presets and
(de)serialisation behaviour as the reference's ``ComplexityConfig``
(complexity_deep/models/config.py:14-109), so configs and checkpoints are interchangeable."""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass


@dataclass
class ComplexityConfig:
    vocab_size: int = 100_000
    hidden_size: int = 768
    intermediate_size: int = 2048      # total routed width; each expert gets 1/num_experts
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    num_key_value_heads: int = 4
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    attention_dropout: float = 0.0
    hidden_act: str = "silu"
    tie_word_embeddings: bool = True
    initializer_range: float = 0.02
    pad_token_id: int = 1
    bos_token_id: int = 2
    eos_token_id: int = 0
    use_token_routed_mlp: bool = True
    num_experts: int = 4
    shared_expert: bool = True
    use_mu_guidance: bool = True
    use_qk_norm: bool = True

    # ---- presets: (hidden, intermediate, layers, q heads, kv heads[, experts]) ----
    @classmethod
    def _preset(cls, h, i, l, q, kv, **kw) -> "ComplexityConfig":
        return cls(hidden_size=h, intermediate_size=i, num_hidden_layers=l,
                   num_attention_heads=q, num_key_value_heads=kv, **kw)

    @classmethod
    def complexity_tiny(cls) -> "ComplexityConfig":
        return cls._preset(256, 704, 6, 4, 2)

    @classmethod
    def complexity_20m(cls) -> "ComplexityConfig":
        return cls._preset(320, 896, 8, 8, 4)

    @classmethod
    def complexity_small(cls) -> "ComplexityConfig":
        return cls._preset(512, 1408, 8, 8, 4)

    @classmethod
    def complexity_150m(cls) -> "ComplexityConfig":
        return cls._preset(768, 2048, 12, 12, 4)

    @classmethod
    def complexity_350m(cls) -> "ComplexityConfig":
        return cls._preset(1280, 3456, 20, 16, 4)

    @classmethod
    def complexity_1b(cls) -> "ComplexityConfig":
        return cls._preset(2048, 5632, 24, 16, 8, num_experts=8)

    # ---- serialisation ----
    def to_dict(self) -> dict:
        return {k: v for k, v in vars(self).items() if not k.startswith("_")}

    @classmethod
    def from_dict(cls, d: dict) -> "ComplexityConfig":
        known = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})
