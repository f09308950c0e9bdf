"""Decoder-only Complexity model — drop-in for the reference's ``ComplexityModel``
(complexity_deep/models/modeling.py:58-318): same constructor, sub-module names
(embed_tokens, layers, norm, lm_head, mu_init), initialisation, forward / generate /
save_pretrained / from_pretrained signatures and output containers, so a reference
state_dict loads here unchanged and vice versa.

The forward pass keeps mu in bf16 and the residual stream as a split-bf16 pair (bf16 tensor
plus its rounding remainder, see core.layer.SplitStream) on the GPU and runs the final
RMSNorm and lm_head on the library's kernels; embedding lookup, attention (SDPA), sampling
and the optional cross-entropy stay PyTorch operators.
"""
from __future__ import annotations

import contextlib
import json
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..core.layer import MuClampRequest, SplitStream, TransformerBlock
from ..core.normalization import RMSNorm
from .config import ComplexityConfig

KVCache = List[Tuple[torch.Tensor, torch.Tensor]]


@dataclass
class ModelOutput:
    logits: Optional[torch.Tensor] = None
    last_hidden_state: Optional[torch.Tensor] = None
    past_key_values: Optional[KVCache] = None


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    past_key_values: Optional[KVCache] = None


class ComplexityModel(nn.Module):
    # The residual stream travels between the fused kernels of consecutive blocks as a
    # split-bf16 pair (see core.layer.SplitStream); False keeps it as one bf16 tensor, as the
    # reference's bf16 path does (two fewer tensor reads / writes per block, ~2.5x the error
    # at the logits of an 18-layer model).
    split_residual_stream = True

    def __init__(self, config: ComplexityConfig):
        super().__init__()
        self.config = config
        c = config
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(
            TransformerBlock(
                hidden_size=c.hidden_size,
                intermediate_size=c.intermediate_size,
                num_attention_heads=c.num_attention_heads,
                num_key_value_heads=c.num_key_value_heads,
                max_position_embeddings=c.max_position_embeddings,
                rms_norm_eps=c.rms_norm_eps,
                rope_theta=c.rope_theta,
                attention_dropout=c.attention_dropout,
                use_token_routed_mlp=c.use_token_routed_mlp,
                num_experts=c.num_experts,
                vocab_size=c.vocab_size,
                shared_expert=c.shared_expert,
                use_qk_norm=c.use_qk_norm,
                use_mu_guidance=c.use_mu_guidance,
            )
            for _ in range(c.num_hidden_layers)
        )
        self.norm = RMSNorm(c.hidden_size, eps=c.rms_norm_eps)
        self.lm_head = nn.Linear(c.hidden_size, c.vocab_size, bias=False)
        if c.tie_word_embeddings:
            self.lm_head.weight = self.embed_tokens.weight
        if c.use_mu_guidance:
            self.mu_init = nn.Parameter(torch.zeros(1, 1, c.hidden_size))

        # Same order of random draws as the reference (modeling.py:110-149): every Linear and
        # Embedding ~ N(0, initializer_range), then the residual output projections are
        # re-drawn with std / sqrt(2 * num_layers).
        self.apply(self._init_weights)
        self._init_residual_scaling()

    def _init_weights(self, module: nn.Module) -> None:
        std = self.config.initializer_range
        if isinstance(module, nn.Linear):
            nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=std)

    def _init_residual_scaling(self) -> None:
        std = self.config.initializer_range / (2 * self.config.num_hidden_layers) ** 0.5
        for layer in self.layers:
            nn.init.normal_(layer.self_attn.o_proj.weight, mean=0.0, std=std)
            mlp = layer.mlp
            if isinstance(getattr(mlp, "down_proj_w", None), nn.Parameter):
                nn.init.normal_(mlp.down_proj_w, mean=0.0, std=std)
            elif isinstance(getattr(mlp, "down_proj", None), nn.Linear):
                nn.init.normal_(mlp.down_proj.weight, mean=0.0, std=std)
            if isinstance(getattr(mlp, "shared_down", None), nn.Linear):
                nn.init.normal_(mlp.shared_down.weight, mean=0.0, std=std)

    # ------------------------------------------------------------------ expert parallelism
    def enable_expert_parallel(self, group=None, exchange: str = "peer",
                               max_tokens_per_rank: int = 0, expert_load=None) -> None:
        """Shards the routed experts of every layer over the ranks of `group` (needs
        num_experts % world_size == 0); tokens stay data-parallel, each rank calls forward on
        its own sequences and gets the same logits as without sharding.  Not part of the
        reference's API (it has no distributed code).  `max_tokens_per_rank`: upper bound of
        batch x sequence length per rank (sizes the exchange buffers, which all layers share)."""
        from ..expert_parallel import ExpertParallelMoE
        for layer in self.layers:
            if layer.use_token_routed_mlp:
                layer.expert_parallel = ExpertParallelMoE(
                    layer.mlp, group, expert_load=expert_load, exchange=exchange,
                    max_tokens_per_rank=max_tokens_per_rank)

    def disable_expert_parallel(self) -> None:
        for layer in self.layers:
            layer.expert_parallel = None

    # ------------------------------------------------------------------ forward
    def forward(
        self,
        input_ids: torch.Tensor,
        attention_mask: Optional[torch.Tensor] = None,
        labels: Optional[torch.Tensor] = None,
        past_key_values: Optional[KVCache] = None,
        use_cache: bool = False,
    ) -> CausalLMOutput:
        B, S = input_ids.shape
        H = self.config.hidden_size
        hidden = self.embed_tokens(input_ids)
        mu_prev = self.mu_init.expand(B, S, -1) if self.config.use_mu_guidance else None
        new_kvs: Optional[KVCache] = [] if use_cache else None

        stream_ctx = SplitStream() if self.split_residual_stream else contextlib.nullcontext()
        with MuClampRequest(-2.0, 2.0) as clamp, stream_ctx as stream:
            for i, layer in enumerate(self.layers):
                past = past_key_values[i] if past_key_values is not None else None
                clamp.applied = False
                hidden, new_kv, mu = layer(hidden, attention_mask=attention_mask,
                                           past_key_value=past, use_cache=use_cache,
                                           token_ids=input_ids, mu_prev=mu_prev)
                if mu is not None:  # clamp fused into the block's mu_proj epilogue when allowed
                    mu_prev = mu if clamp.applied else torch.clamp(mu, -2.0, 2.0)
                if use_cache:
                    new_kvs.append(new_kv)
            hidden_lo = stream.take(hidden) if stream is not None else None

        normed = ops.rmsnorm(hidden.reshape(B * S, H).contiguous(), self.norm.weight, self.norm.eps,
                             x_lo=hidden_lo)
        logits = ops.linear(normed, self.lm_head.weight, tag="linear_lm_head").view(B, S, -1)

        loss = None
        if labels is not None:
            loss = F.cross_entropy(
                logits[..., :-1, :].reshape(-1, self.config.vocab_size).float(),
                labels[..., 1:].reshape(-1), ignore_index=-100)
        return CausalLMOutput(loss=loss, logits=logits, past_key_values=new_kvs)

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(
        self,
        input_ids: torch.Tensor,
        max_new_tokens: int = 100,
        temperature: float = 1.0,
        top_k: int = 50,
        top_p: float = 0.9,
        do_sample: bool = True,
        eos_token_id: Optional[int] = None,
    ) -> torch.Tensor:
        """Autoregressive sampling with a KV cache; same filtering rules as the reference
        (temperature, then top-k, then nucleus top-p that always keeps the best token)."""
        eos = self.config.eos_token_id if eos_token_id is None else eos_token_id
        cache: Optional[KVCache] = None
        for _ in range(max_new_tokens):
            step_ids = input_ids if cache is None else input_ids[:, -1:]
            out = self.forward(step_ids, past_key_values=cache, use_cache=True)
            cache = out.past_key_values
            scores = out.logits[:, -1, :].float() / temperature
            if top_k > 0:
                kth = torch.topk(scores, top_k).values[..., -1:]
                scores = scores.masked_fill(scores < kth, float("-inf"))
            if top_p < 1.0:
                ordered, order = torch.sort(scores, descending=True)
                mass = torch.cumsum(F.softmax(ordered, dim=-1), dim=-1)
                drop = mass > top_p
                drop = torch.cat([torch.zeros_like(drop[..., :1]), drop[..., :-1]], dim=-1)
                scores = scores.masked_fill(drop.scatter(1, order, drop), float("-inf"))
            if do_sample:
                nxt = torch.multinomial(F.softmax(scores, dim=-1), num_samples=1)
            else:
                nxt = scores.argmax(dim=-1, keepdim=True)
            input_ids = torch.cat([input_ids, nxt], dim=-1)
            if bool((nxt == eos).all()):
                break
        return input_ids

    # ------------------------------------------------------------------ utilities
    def num_parameters(self, trainable_only: bool = True) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not trainable_only)

    def save_pretrained(self, path: str) -> None:
        """Writes ``config.json`` and ``model.pt`` (a plain state_dict), as the reference does."""
        target = Path(path)
        target.mkdir(parents=True, exist_ok=True)
        (target / "config.json").write_text(json.dumps(self.config.to_dict(), indent=2))
        torch.save(self.state_dict(), target / "model.pt")

    @classmethod
    def from_pretrained(cls, path: str, device: str = "cpu") -> "ComplexityModel":
        source = Path(path)
        config = ComplexityConfig.from_dict(json.loads((source / "config.json").read_text()))
        model = cls(config)
        model.load_state_dict(torch.load(source / "model.pt", map_location=device), strict=False)
        return model.to(device)
