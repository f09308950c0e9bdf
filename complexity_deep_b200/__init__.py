"""B200-native drop-in for the hot path of Complexity-ML/complexity-deep.

Exports the same names as the reference package (complexity_deep/__init__.py:21-54); the
token-routed MoE layer, the mu-guided QKV projection, RMSNorm and mu_proj run on
hand-written sm_100a CUDA kernels behind a C ABI (include/cdeep.h, libcdeep.so).
"""
from .core import (RMSNorm, RotaryEmbedding, ComplexityAttention, SwiGLU, TokenRoutedMLP,
                   TransformerBlock, MuGuidance)
from .models import (ComplexityConfig, ComplexityModel, create_complexity_model,
                     count_parameters)

__version__ = "1.0.0"

__all__ = [
    "RMSNorm", "RotaryEmbedding", "ComplexityAttention", "SwiGLU", "TokenRoutedMLP",
    "TransformerBlock", "MuGuidance", "ComplexityConfig", "ComplexityModel",
    "create_complexity_model", "count_parameters",
]
