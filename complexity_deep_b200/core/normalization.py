"""RMSNorm with the reference's constructor, parameters and forward signature
(complexity_deep/core/normalization.py:17-35), computed by the N1 CUDA kernel."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class RMSNorm(nn.Module):
    """y = weight * x * rsqrt(mean(x^2, -1) + eps); state_dict key: ``weight`` [hidden_size]."""

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops.forward_only(x, "RMSNorm")
        return ops.rmsnorm(x.contiguous(), self.weight, self.eps)

    def extra_repr(self) -> str:
        return f"{self.weight.numel()}, eps={self.eps}"
