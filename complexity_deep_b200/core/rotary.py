"""Rotary position embedding tables (complexity_deep/core/rotary.py:17-86).

Same buffers as the reference: persistent ``inv_freq`` [D/2], non-persistent fp32
``cos_cached`` / ``sin_cached`` [positions, D].  The rotation itself is applied by the
cd_qk_norm_rope kernel; ``apply_rotary_pos_emb`` is kept for callers that use it directly.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn as nn


class RotaryEmbedding(nn.Module):
    def __init__(self, dim: int, max_seq_len: int = 2048, theta: float = 10000.0):
        super().__init__()
        self.dim, self.max_seq_len, self.theta = dim, max_seq_len, theta
        exponents = torch.arange(0, dim, 2).float() / dim
        self.register_buffer("inv_freq", 1.0 / (theta ** exponents))
        self._build_cache(max_seq_len)

    def _build_cache(self, seq_len: int) -> None:
        pos = torch.arange(seq_len, device=self.inv_freq.device).float()
        angles = torch.outer(pos, self.inv_freq)
        table = torch.cat([angles, angles], dim=-1)
        self.register_buffer("cos_cached", table.cos(), persistent=False)
        self.register_buffer("sin_cached", table.sin(), persistent=False)

    def forward(self, seq_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
        if seq_len > self.max_seq_len:
            self._build_cache(seq_len)
            self.max_seq_len = seq_len
        return self.cos_cached[:seq_len], self.sin_cached[:seq_len]

    def tables_fp32(self, seq_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Full fp32 tables covering at least `seq_len` positions, for the CUDA kernel.

        ``module.to(bfloat16)`` also casts the cached tables; they are then rebuilt in fp32
        from ``inv_freq`` so the kernel always reads full-precision angles.
        """
        if seq_len > self.max_seq_len or self.cos_cached.dtype != torch.float32:
            if self.inv_freq.dtype != torch.float32:
                exponents = torch.arange(0, self.dim, 2, device=self.inv_freq.device).float()
                self.inv_freq = 1.0 / (self.theta ** (exponents / self.dim))
            if seq_len > self.max_seq_len:
                # grow geometrically: decode steps past the configured maximum must not
                # rebuild the tables on every step
                self.max_seq_len = 1 << (seq_len - 1).bit_length()
            self._build_cache(self.max_seq_len)
        return self.cos_cached, self.sin_cached


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat([-x[..., half:], x[..., :half]], dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin):
    """q, k: [B, heads, S, D]; cos, sin: [S, D]."""
    cos, sin = cos[None, None], sin[None, None]
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin
