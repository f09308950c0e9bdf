"""Decoder block and mu guidance — drop-ins for the reference's ``TransformerBlock`` and
``MuGuidance`` (complexity_deep/core/layer.py:27-190): same constructors, same sub-module
names (input_layernorm, self_attn, post_attention_layernorm, mlp, mu_guidance), same
forward signature and return triple.

``TransformerBlock.forward`` has two routes that produce the same values:
  * the fused route (default): the attention residual add runs in o_proj's epilogue, the
    post-attention RMSNorm writes its rows straight into expert-sorted order, and the MoE
    down-projection's epilogue un-permutes, combines shared + routed and adds the residual;
  * the module route, taken when a caller has registered hooks on a sub-module (analysis
    scripts hook ``layer.mlp``): each sub-module is then invoked through ``__call__`` with
    the reference's inputs and outputs, and the residual adds are separate.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from .attention import ComplexityAttention
from .mlp import SwiGLU
from .normalization import RMSNorm
from .token_routed_mlp import TokenRoutedMLP


class MuClampRequest:
    """Set by ComplexityModel.forward around its layer loop: asks each block to apply the
    model's clamp of mu (complexity_deep/models/modeling.py:199-200) in the mu_proj GEMM's
    epilogue instead of a separate elementwise pass.  A block honours it only when nobody
    hooks the block or its mu_guidance (their hooks must see the unclamped value), and
    reports back through `applied`."""
    current = None

    def __init__(self, lo: float, hi: float) -> None:
        self.range = (lo, hi)
        self.applied = False

    def __enter__(self):
        self.previous, MuClampRequest.current = MuClampRequest.current, self
        return self

    def __exit__(self, *exc):
        MuClampRequest.current = self.previous
        return False


class SplitStream:
    """Set by ComplexityModel.forward around its layer loop: lets consecutive blocks hand the
    residual stream to each other as a split-bf16 pair.  The tensor a block returns is
    hi = bf16(v); the part the rounding dropped, lo = bf16(v - hi), travels here.  The next
    block adds both to what it computes (its RMSNorms and residual epilogues read hi + lo), so
    the 2 * num_layers additions into the stream (complexity_deep/core/layer.py:174, :183) are
    not each rounded to 8 significant bits.  Measured on the README model (18 layers, 4 x 512
    tokens): mean |logit error| against the fp32 reference 1.4e-3 instead of 3.5e-3.

    `take` hands out the low part only for the very tensor object that `put` registered, so a
    caller (or hook) that replaces the hidden states between blocks silently drops it."""
    current = None

    def __init__(self) -> None:
        self.hi = None
        self.lo = None

    def __enter__(self):
        self.previous, SplitStream.current = SplitStream.current, self
        return self

    def __exit__(self, *exc):
        SplitStream.current = self.previous
        self.hi = self.lo = None
        return False

    def put(self, hi: torch.Tensor, lo: Optional[torch.Tensor]) -> None:
        self.hi, self.lo = hi, lo

    def take(self, hidden_states: torch.Tensor) -> Optional[torch.Tensor]:
        lo = self.lo if hidden_states is self.hi else None
        self.hi = self.lo = None
        return lo


def _has_hooks(m: nn.Module) -> bool:
    return bool(m._forward_hooks or m._forward_pre_hooks or m._backward_hooks
                or getattr(m, "_forward_hooks_with_kwargs", None)
                or getattr(m, "_forward_pre_hooks_with_kwargs", None))


class MuGuidance(nn.Module):
    """mu_contextual = clamp(mu, mu_min, mu_max) + mu_proj(hidden_states)  (layer.py:54-61)."""

    def __init__(self, hidden_size: int, mu_min: float = 0.0, mu_max: float = 2.0):
        super().__init__()
        self.mu_min, self.mu_max = mu_min, mu_max
        self.mu = nn.Parameter(torch.full((hidden_size,), (mu_min + mu_max) / 2))
        self.mu_proj = nn.Linear(hidden_size, hidden_size, bias=False)
        nn.init.zeros_(self.mu_proj.weight)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        ops.forward_only(hidden_states, "MuGuidance")
        shape = hidden_states.shape
        h2 = hidden_states.reshape(-1, shape[-1]).contiguous()
        return ops.mu_proj(h2, self.mu_proj.weight, self.mu, self.mu_min, self.mu_max).view(shape)


class TransformerBlock(nn.Module):
    def __init__(
        self,
        hidden_size: int,
        intermediate_size: int,
        num_attention_heads: int,
        num_key_value_heads: int,
        max_position_embeddings: int = 2048,
        rms_norm_eps: float = 1e-6,
        rope_theta: float = 10000.0,
        attention_dropout: float = 0.0,
        use_token_routed_mlp: bool = True,
        num_experts: int = 4,
        vocab_size: int = 100_000,
        shared_expert: bool = True,
        token_frequencies: Optional[torch.Tensor] = None,
        use_qk_norm: bool = True,
        use_mu_guidance: bool = True,
    ):
        super().__init__()
        self.hidden_size = hidden_size
        self.use_token_routed_mlp = use_token_routed_mlp
        self.input_layernorm = RMSNorm(hidden_size, eps=rms_norm_eps)
        self.self_attn = ComplexityAttention(
            hidden_size=hidden_size,
            num_attention_heads=num_attention_heads,
            num_key_value_heads=num_key_value_heads,
            max_position_embeddings=max_position_embeddings,
            rope_theta=rope_theta,
            attention_dropout=attention_dropout,
            use_qk_norm=use_qk_norm,
        )
        self.post_attention_layernorm = RMSNorm(hidden_size, eps=rms_norm_eps)
        if use_token_routed_mlp:
            self.mlp = TokenRoutedMLP(
                hidden_size=hidden_size,
                intermediate_size=intermediate_size,
                num_experts=num_experts,
                vocab_size=vocab_size,
                shared_expert=shared_expert,
                token_frequencies=token_frequencies,
            )
        else:
            self.mlp = SwiGLU(hidden_size=hidden_size, intermediate_size=intermediate_size)
        self.use_mu_guidance = use_mu_guidance
        self.mu_guidance = MuGuidance(hidden_size=hidden_size) if use_mu_guidance else None
        # set by ComplexityModel.enable_expert_parallel: runs the routed experts sharded over
        # the GPUs of a process group (the parameters stay where they are)
        self.expert_parallel = None

    def _fusable(self, token_ids) -> bool:
        subs = [self.input_layernorm, self.self_attn, self.post_attention_layernorm, self.mlp]
        if any(_has_hooks(m) for m in subs):
            return False
        return not (self.use_token_routed_mlp and token_ids is None)

    def forward(
        self,
        hidden_states: torch.Tensor,
        attention_mask: Optional[torch.Tensor] = None,
        past_key_value: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
        use_cache: bool = False,
        token_ids: Optional[torch.Tensor] = None,
        mu_prev: Optional[torch.Tensor] = None,
    ) -> Tuple[torch.Tensor, Optional[Tuple[torch.Tensor, torch.Tensor]], Optional[torch.Tensor]]:
        ops.forward_only(hidden_states, "TransformerBlock")
        if self._fusable(token_ids):
            hidden_states, new_kv = self._forward_fused(
                hidden_states, attention_mask, past_key_value, use_cache, token_ids, mu_prev)
        else:
            residual = hidden_states
            hidden_states = self.input_layernorm(hidden_states)
            hidden_states, new_kv = self.self_attn(
                hidden_states, attention_mask=attention_mask, past_key_value=past_key_value,
                use_cache=use_cache, mu_prev=mu_prev)
            hidden_states = residual + hidden_states
            residual = hidden_states
            hidden_states = self.post_attention_layernorm(hidden_states)
            if self.use_token_routed_mlp:
                hidden_states = self.mlp(hidden_states, token_ids=token_ids)
            else:
                hidden_states = self.mlp(hidden_states)
            hidden_states = residual + hidden_states

        mu_contextual = None
        if self.mu_guidance is not None:
            req = MuClampRequest.current
            if req is not None and not _has_hooks(self) and not _has_hooks(self.mu_guidance):
                mg = self.mu_guidance
                shape = hidden_states.shape
                mu_contextual = ops.mu_proj(
                    hidden_states.reshape(-1, shape[-1]).contiguous(), mg.mu_proj.weight, mg.mu,
                    mg.mu_min, mg.mu_max, out_clamp=req.range).view(shape)
                req.applied = True
            else:
                mu_contextual = self.mu_guidance(hidden_states)
        return hidden_states, new_kv, mu_contextual

    def _forward_fused(self, hidden_states, attention_mask, past_key_value, use_cache, token_ids,
                       mu_prev):
        B, S, H = hidden_states.shape
        if (self.use_token_routed_mlp and token_ids is not None
                and token_ids.numel() != B * S):
            raise ValueError(f"token_ids has {token_ids.numel()} entries for {B * S} tokens")
        stream = SplitStream.current
        split = stream is not None
        lo0 = stream.take(hidden_states) if split else None
        h0 = hidden_states.reshape(B * S, H).contiguous()
        ln1 = self.input_layernorm
        normed = ops.rmsnorm(h0, ln1.weight, ln1.eps, x_lo=lo0).view(B, S, H)
        # h1 = h0 + o_proj(attention(...)): residual added in the GEMM epilogue
        h1, h1_lo, new_kv = self.self_attn.forward_with_residual(
            normed, h0, attention_mask=attention_mask, past_key_value=past_key_value,
            use_cache=use_cache, mu_prev=mu_prev, residual_lo=lo0, want_lo=split)
        h1 = h1.view(B * S, H)
        ln2 = self.post_attention_layernorm
        if self.use_token_routed_mlp:
            runner = self.expert_parallel if self.expert_parallel is not None else self.mlp
            routing = runner.routing(token_ids)
            # normalised rows land directly in expert-sorted order
            x_sorted = ops.rmsnorm(h1, ln2.weight, ln2.eps, dst_rows=routing.inv_perm, x_lo=h1_lo)
            h2 = runner.forward_sorted(x_sorted, routing, residual=h1, residual_lo=h1_lo,
                                       want_lo=split)
        else:
            x = ops.rmsnorm(h1, ln2.weight, ln2.eps, x_lo=h1_lo)
            h2 = self.mlp._run(x, residual=h1, residual_lo=h1_lo, want_lo=split)
        if split:
            h2, h2_lo = h2
            out = h2.view(B, S, H)
            stream.put(out, h2_lo)
            return out, new_kv
        return h2.view(B, S, H), new_kv
