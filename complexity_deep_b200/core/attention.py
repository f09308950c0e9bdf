"""Grouped-query attention with mu-guided projections — drop-in for the reference's
``ComplexityAttention`` (complexity_deep/core/attention.py:34-199): same constructor, same
parameters (q/k/v/o_proj, mu_to_q/k/v, q_norm/k_norm, rotary_emb), same forward signature
and the same scaled_dot_product_attention call (including its ``is_causal`` rule).

What changes is how q, k, v are produced:
  * one K-concatenated GEMM ``[x | mu_prev] @ [W ; W_mu]^T`` (cd_mu_qkv) reading x and
    mu_prev in place and the stacked weights from a cache, instead of a ``torch.cat`` of the
    activations, three ``torch.cat`` of the weights and three GEMMs per call (:120-127);
  * Q/K RMSNorm and RoPE applied in that GEMM's epilogue (cd_mu_qkv_rope, head size 128) or
    in place by one kernel (cd_qk_norm_rope) instead of ~10 elementwise passes (:138-155);
  * grouped KV heads are handed to SDPA with ``enable_gqa`` instead of being copied by
    ``repeat_interleave`` (:164-165) — the same arithmetic without the copies; with one
    query per sequence the cache is streamed once by cd_decode_attention;
  * the KV cache grows in place instead of by ``torch.cat`` (:158-161), or lives in a
    fixed-capacity ``StaticKVCache`` whose decode steps can be replayed from a CUDA graph;
  * ``o_proj`` runs on the tcgen05 GEMM, optionally with the residual add fused.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ._cache import DerivedCache
from .rotary import RotaryEmbedding


# CDEEP_PREFILL_ATTENTION=sdpa sends prompts through torch's scaled_dot_product_attention instead
# of cd_attention_prefill (comparison / debugging aid)
_PREFILL_KERNEL = os.environ.get("CDEEP_PREFILL_ATTENTION", "kernel") != "sdpa"


class _KVBuffer:
    """Backing store of a KV cache that grows in place.

    The reference appends with ``torch.cat([past, new], dim=2)`` (attention.py:158-161), which
    copies the whole cache on every decode step.  Here the tensor handed back to the caller is
    a view ``buf[:, :, :used]`` of a larger buffer; when that same tensor comes back as
    ``past_key_value`` and nobody has appended to it since (``used`` still equals its length),
    the new rows are written behind it and a longer view is returned — same values as the
    concatenation, without the copy.  Any other tensor (a user-built cache, a cache that was
    already extended by another branch) is copied once into a fresh buffer.
    """

    def __init__(self, buf: torch.Tensor, used: int) -> None:
        self.buf, self.used = buf, used


def _kv_append(past: torch.Tensor, new: torch.Tensor) -> torch.Tensor:
    P, S = past.shape[2], new.shape[2]
    holder = getattr(past, "_cd_kv", None)
    if (holder is None or holder.used != P or holder.buf.shape[2] < P + S
            or holder.buf.dtype != new.dtype or holder.buf.device != new.device):
        B, Hk, _, D = past.shape
        cap = P + S + max(256, (P + S) // 8)
        buf = torch.empty(B, Hk, cap, D, dtype=new.dtype, device=new.device)
        buf[:, :, :P].copy_(past)
        holder = _KVBuffer(buf, P)
    holder.buf[:, :, P:P + S].copy_(new)
    holder.used = P + S
    out = holder.buf[:, :, :P + S]
    out._cd_kv = holder
    return out


class StaticKVCache:
    """Fixed-capacity KV cache of a whole model for decode steps whose launches never change.

    The reference's cache is a list of ``(k, v)`` tensors that grow by ``torch.cat``
    (attention.py:158-161), so every step has new shapes and addresses.  Here each layer owns
    ``k`` / ``v`` buffers ``[batch, kv_heads, capacity, head_dim]`` and the number of cached
    tokens lives in DEVICE memory (``state[0]``; ``state[1]`` = that + 1, the keys a step sees
    after appending its own).  A decode step through ``model(ids, past_key_values=cache.layers,
    use_cache=True)`` then issues exactly the same launches at every length, which is what a
    CUDA graph needs (see ``DecodeGraph``).  Steps attend to the whole cache — what the
    reference computes when it is given an all-zero additive mask.  Not part of the
    reference's API.
    """

    def __init__(self, num_layers: int, batch: int, kv_heads: int, head_dim: int, capacity: int,
                 device, dtype=torch.bfloat16) -> None:
        self.capacity = capacity
        self.k = [torch.zeros(batch, kv_heads, capacity, head_dim, dtype=dtype, device=device)
                  for _ in range(num_layers)]
        self.v = [torch.zeros_like(t) for t in self.k]
        self.state = torch.zeros(2, dtype=torch.int32, device=device)
        self.state[1] = 1
        self.length = 0                       # host mirror of state[0]
        self.layers = [StaticKVLayer(self, i) for i in range(num_layers)]

    def load(self, past_key_values) -> None:
        """Copies a cache produced by a prefill (list of (k, v) [B, kv_heads, P, D])."""
        P = past_key_values[0][0].shape[2]
        if P > self.capacity:
            raise ValueError(f"{P} cached tokens do not fit a capacity of {self.capacity}")
        for i, (k, v) in enumerate(past_key_values):
            self.k[i][:, :, :P].copy_(k)
            self.v[i][:, :, :P].copy_(v)
        self.set_length(P)

    def set_length(self, length: int) -> None:
        if not 0 <= length <= self.capacity:
            raise ValueError("length outside the cache")
        self.length = length
        self.state.copy_(torch.tensor([length, length + 1], dtype=torch.int32), non_blocking=False)

    def advance(self) -> None:
        """One token was appended to every layer: move the device-side position (stream
        ordered, capturable) and its host mirror."""
        self.state.add_(1)
        self.length += 1


class StaticKVLayer:
    """One layer's slice of a StaticKVCache, passed as that layer's ``past_key_value``."""

    def __init__(self, cache: StaticKVCache, index: int) -> None:
        self.cache, self.index = cache, index

    @property
    def k(self) -> torch.Tensor:
        return self.cache.k[self.index]

    @property
    def v(self) -> torch.Tensor:
        return self.cache.v[self.index]


class ComplexityAttention(nn.Module):
    def __init__(
        self,
        hidden_size: int,
        num_attention_heads: int,
        num_key_value_heads: int,
        max_position_embeddings: int = 2048,
        rope_theta: float = 10000.0,
        attention_dropout: float = 0.0,
        use_qk_norm: bool = True,
    ):
        super().__init__()
        if hidden_size % num_attention_heads or num_attention_heads % num_key_value_heads:
            raise AssertionError("hidden_size / heads / kv heads are not divisible")
        self.hidden_size = hidden_size
        self.num_heads = num_attention_heads
        self.num_kv_heads = num_key_value_heads
        self.head_dim = hidden_size // num_attention_heads
        self.num_kv_groups = num_attention_heads // num_key_value_heads
        q_dim = self.num_heads * self.head_dim
        kv_dim = self.num_kv_heads * self.head_dim

        self.q_proj = nn.Linear(hidden_size, q_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, kv_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, kv_dim, bias=False)
        self.o_proj = nn.Linear(q_dim, hidden_size, bias=False)
        self.mu_to_q = nn.Linear(hidden_size, q_dim, bias=False)
        self.mu_to_k = nn.Linear(hidden_size, kv_dim, bias=False)
        self.mu_to_v = nn.Linear(hidden_size, kv_dim, bias=False)

        self.use_qk_norm = use_qk_norm
        if use_qk_norm:
            self.q_norm = nn.RMSNorm(self.head_dim, eps=1e-6)
            self.k_norm = nn.RMSNorm(self.head_dim, eps=1e-6)
        self.rotary_emb = RotaryEmbedding(self.head_dim, max_seq_len=max_position_embeddings,
                                          theta=rope_theta)
        self.attention_dropout = attention_dropout
        self._derived = DerivedCache()

    # ------------------------------------------------------------------ stacked weights
    def _w_qkv(self) -> torch.Tensor:
        src = (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight)
        return self._derived.get("w_qkv", src, lambda: torch.cat([w.detach() for w in src], 0))

    def _w_mu(self) -> torch.Tensor:
        src = (self.mu_to_q.weight, self.mu_to_k.weight, self.mu_to_v.weight)
        return self._derived.get("w_mu", src, lambda: torch.cat([w.detach() for w in src], 0))

    # ------------------------------------------------------------------ forward
    def _attend(self, hidden_states, attention_mask, past_key_value, use_cache, mu_prev):
        """Everything up to (not including) o_proj; returns ([T, q_dim], new_kv)."""
        ops.forward_only(hidden_states, "ComplexityAttention")
        B, S, H = hidden_states.shape
        hq, hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        x2 = hidden_states.reshape(B * S, H).contiguous()
        mu2 = None
        if mu_prev is not None:
            mu2 = mu_prev.reshape(B * S, H).contiguous()  # materialises a broadcast mu_init
        if isinstance(past_key_value, StaticKVLayer):
            return (self._attend_static(x2, mu2, past_key_value, S, attention_mask),
                    past_key_value if use_cache else None)
        past_len = past_key_value[0].shape[2] if past_key_value is not None else 0
        cos, sin = self.rotary_emb.tables_fp32(past_len + S)
        qkv = ops.mu_qkv_rope(x2, mu2, self._w_qkv(), self._w_mu() if mu2 is not None else None,
                              self.q_norm.weight if self.use_qk_norm else None,
                              self.k_norm.weight if self.use_qk_norm else None, cos, sin, 1e-6, S,
                              past_len, hq, hkv, D)

        q = qkv[:, : hq * D].view(B, S, hq, D).transpose(1, 2)
        k = qkv[:, hq * D: (hq + hkv) * D].view(B, S, hkv, D).transpose(1, 2)
        v = qkv[:, (hq + hkv) * D:].view(B, S, hkv, D).transpose(1, 2)
        if past_key_value is not None:
            k = _kv_append(past_key_value[0], k)
            v = _kv_append(past_key_value[1], v)
        new_kv = (k, v) if use_cache else None

        if self._decode_kernel_applies(S, attention_mask, k, v):
            # one query per sequence: stream the cache once with the library's kernel.  With no
            # mask the reference's is_causal=True is top-left aligned, i.e. only key 0 is seen.
            if attention_mask is None:
                kk, vv, mask = k[:, :, :1], v[:, :, :1], None
            else:
                kk, vv, mask = k, v, attention_mask
            return ops.decode_attention(qkv, kk, vv, mask, hq, hkv, D), new_kv

        if self._prefill_kernel_applies(B, S, attention_mask, past_key_value):
            # a prompt with nothing cached and no mask: causal attention on the library's
            # tcgen05 kernel, reading q / k / v in place from the projection buffer
            return ops.attention_prefill(qkv, B, S, hq, hkv, D), new_kv

        with ops._Span("sdpa", kernels=0):  # PyTorch operator, timed for the breakdown only
            attn = F.scaled_dot_product_attention(
                q, k, v,
                attn_mask=attention_mask,
                dropout_p=self.attention_dropout if self.training else 0.0,
                is_causal=(attention_mask is None),
                enable_gqa=self.num_kv_groups > 1,
            )
            attn = attn.transpose(1, 2).reshape(B * S, hq * D).contiguous()
        return attn, new_kv

    def _attend_static(self, x2, mu2, past: StaticKVLayer, S, attention_mask) -> torch.Tensor:
        """Decode step on a StaticKVCache: projection, then one kernel that normalises and
        rotates q / k at the device-side position and appends k / v to the cache, then the
        split-KV attention over the device-side length."""
        hq, hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        if S != 1 or attention_mask is not None:
            raise RuntimeError("a StaticKVCache takes one new token per sequence and no mask "
                               "(steps attend to the whole cache)")
        if D not in (64, 128) or self.num_kv_groups > 4:
            raise RuntimeError("StaticKVCache decode needs head size 64 or 128 and at most 4 "
                               "query heads per KV head")
        cache = past.cache
        cos, sin = self.rotary_emb.tables_fp32(cache.capacity)
        qkv = ops.mu_qkv(x2, mu2, self._w_qkv(), self._w_mu() if mu2 is not None else None)
        ops.decode_rope_append(qkv, self.q_norm.weight if self.use_qk_norm else None,
                               self.k_norm.weight if self.use_qk_norm else None, cos, sin, 1e-6,
                               hq, hkv, D, past.k, past.v, cache.state[0:1])
        return ops.decode_attention(qkv, past.k, past.v, None, hq, hkv, D,
                                    kv_len_dev=cache.state[1:2])

    def _prefill_kernel_applies(self, B, S, attention_mask, past_key_value) -> bool:
        if attention_mask is not None or past_key_value is not None or not _PREFILL_KERNEL:
            return False
        if self.training and self.attention_dropout > 0:
            return False
        return ops.attention_prefill_supported(B, S, self.num_heads, self.num_kv_heads,
                                               self.head_dim)

    def _decode_kernel_applies(self, S, attention_mask, k, v) -> bool:
        if S != 1 or self.head_dim not in (64, 128) or self.num_kv_groups > 4:
            return False
        if k.stride() != v.stride() or k.stride(3) != 1 or any(st % 8 for st in k.stride()[:3]):
            return False
        if self.training and self.attention_dropout > 0:
            return False
        if attention_mask is None:
            return True
        m = attention_mask
        return (m.dtype == torch.bfloat16 and m.dim() == 4 and m.shape[1] == 1 and m.shape[2] == 1
                and m.shape[3] == k.shape[2] and m.shape[0] in (1, k.shape[0]) and m.stride(3) == 1)

    def forward(
        self,
        hidden_states: torch.Tensor,
        attention_mask: Optional[torch.Tensor] = None,
        past_key_value: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
        use_cache: bool = False,
        mu_prev: Optional[torch.Tensor] = None,
    ) -> Tuple[torch.Tensor, Optional[Tuple[torch.Tensor, torch.Tensor]]]:
        B, S, H = hidden_states.shape
        attn, new_kv = self._attend(hidden_states, attention_mask, past_key_value, use_cache,
                                    mu_prev)
        return ops.linear(attn, self.o_proj.weight, tag="linear_o_proj").view(B, S, H), new_kv

    def forward_with_residual(self, hidden_states, residual, attention_mask=None,
                              past_key_value=None, use_cache=False, mu_prev=None,
                              residual_lo=None, want_lo=False):
        """Same as forward, with ``residual (+ residual_lo) + o_proj(attn)`` computed in the GEMM
        epilogue; returns (out, out_lo or None, new_kv) — out_lo is the low part of the
        split-bf16 result when `want_lo`."""
        B, S, H = hidden_states.shape
        attn, new_kv = self._attend(hidden_states, attention_mask, past_key_value, use_cache,
                                    mu_prev)
        out = ops.linear(attn, self.o_proj.weight, residual.reshape(B * S, H), tag="linear_o_proj",
                         residual_lo=residual_lo, want_lo=want_lo)
        out, out_lo = out if want_lo else (out, None)
        return out.view(B, S, H), out_lo, new_kv
