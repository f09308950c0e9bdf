"""Dense SwiGLU MLP with the reference's parameters (complexity_deep/core/mlp.py:19-40),
run as the one-group case of the fused up-projection and down-projection kernels."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ._cache import DerivedCache


class SwiGLU(nn.Module):
    """out = down_proj(silu(gate_proj(x)) * up_proj(x)); three bias-free nn.Linear."""

    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)
        self._derived = DerivedCache()

    def _packed(self):
        g, u = self.gate_proj.weight, self.up_proj.weight
        bn = ops.choose_block_n(g.shape[0])
        packed = self._derived.get(
            "gate_up", (g, u),
            lambda: ops.pack_gate_up(g.detach()[None].contiguous(), u.detach()[None].contiguous(), bn))
        return packed, bn

    def _run(self, x2: torch.Tensor, residual=None, residual_lo=None, want_lo: bool = False):
        packed, bn = self._packed()
        width = self.gate_proj.weight.shape[0]
        h = ops.moe_up(x2, None, 1, packed, width, bn)
        wd = self.down_proj.weight.detach()[None]  # [1, H, I]
        return ops.moe_down(h, wd, None, None, None, 1, None, residual, residual_lo, want_lo)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops.forward_only(x, "SwiGLU")
        shape = x.shape
        return self._run(x.reshape(-1, shape[-1]).contiguous()).view(shape)
