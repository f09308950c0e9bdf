"""Building blocks with the reference's names (complexity_deep/core/__init__.py:13-29)."""
from .normalization import RMSNorm
from .rotary import RotaryEmbedding, apply_rotary_pos_emb
from .attention import ComplexityAttention
from .mlp import SwiGLU
from .token_routed_mlp import TokenRoutedMLP
from .layer import TransformerBlock, MuGuidance

__all__ = [
    "RMSNorm", "RotaryEmbedding", "apply_rotary_pos_emb", "ComplexityAttention", "SwiGLU",
    "TokenRoutedMLP", "TransformerBlock", "MuGuidance",
]
