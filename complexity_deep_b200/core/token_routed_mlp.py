"""Token-routed MoE layer with a shared SwiGLU expert — drop-in for the reference's
``TokenRoutedMLP`` (complexity_deep/core/token_routed_mlp.py:28-194): same constructor,
same parameters/buffers (``gate_proj_w``, ``up_proj_w`` [E, H, I_e], ``down_proj_w``
[E, I_e, H], ``shared_gate/up/down`` Linear, ``token_to_expert`` int64 [V]), same forward
signature.  The per-expert Python loop of boolean masks is replaced by

    cd_route      ids -> expert ids, histogram, offsets, stable permutation (cached per batch)
    cd_moe_up     grouped gate|up GEMM with silu(gate)*up in the epilogue (routed, then shared)
    cd_moe_down   routed + shared down GEMMs as one fp32 accumulation, rows scattered back

on the GPU, with no host synchronisation inside the layer.
"""
from __future__ import annotations

import hashlib
import heapq
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ._cache import DerivedCache


class _RoutingCache:
    """Routing artefacts of recent id batches.

    The ids never change between the layers of a forward pass and every layer of a model
    normally carries the same table, so the dispatch kernels run once per batch.  An entry
    keeps a reference to its ids tensor: while the entry lives that memory cannot be
    re-used by another tensor, so (data_ptr, shape, strides, _version) identifies the
    content.  Tables are identified by a digest of their content, taken once per version.
    """

    def __init__(self, capacity: int = 8) -> None:
        self.capacity = capacity
        self.entries: List[Tuple[Tuple, torch.Tensor, ops.Routing]] = []

    @staticmethod
    def _key(ids: torch.Tensor, table_sig: Tuple) -> Tuple:
        return (ids.data_ptr(), tuple(ids.shape), tuple(ids.stride()), ids._version, ids.device,
                table_sig)

    def lookup(self, ids: torch.Tensor, table: torch.Tensor, table_sig: Tuple, num_experts: int
               ) -> ops.Routing:
        key = self._key(ids, table_sig)
        for k, _, routing in self.entries:
            if k == key:
                return routing
        routing = ops.route(ids.contiguous(), table, num_experts)
        self.entries.append((key, ids, routing))
        if len(self.entries) > self.capacity:
            self.entries.pop(0)
        return routing

    def clear(self) -> None:
        self.entries.clear()


ROUTING_CACHE = _RoutingCache()


class TokenRoutedMLP(nn.Module):
    def __init__(
        self,
        hidden_size: int,
        intermediate_size: int,
        num_experts: int = 4,
        vocab_size: int = 100_000,
        shared_expert: bool = True,
        token_frequencies: Optional[torch.Tensor] = None,
    ):
        super().__init__()
        self.hidden_size = hidden_size
        self.num_experts = num_experts
        self.vocab_size = vocab_size
        self.expert_intermediate_size = intermediate_size // num_experts
        E, H, I_e = num_experts, hidden_size, self.expert_intermediate_size

        self.gate_proj_w = nn.Parameter(torch.randn(E, H, I_e) * 0.02)
        self.up_proj_w = nn.Parameter(torch.randn(E, H, I_e) * 0.02)
        self.down_proj_w = nn.Parameter(torch.randn(E, I_e, H) * 0.02)

        self.use_shared_expert = shared_expert
        if shared_expert:
            self.shared_gate = nn.Linear(H, I_e, bias=False)
            self.shared_up = nn.Linear(H, I_e, bias=False)
            self.shared_down = nn.Linear(I_e, H, bias=False)

        self.register_buffer(
            "token_to_expert", self._build_token_mapping(vocab_size, num_experts, token_frequencies))
        self._derived = DerivedCache()
        self._table_sig_key = None
        self._table_sig = None

    # ------------------------------------------------------------------ routing table
    @staticmethod
    def _build_token_mapping(vocab_size: int, num_experts: int,
                             token_frequencies: Optional[torch.Tensor]) -> torch.Tensor:
        """vocab -> expert table (reference: token_routed_mlp.py:87-119).

        With frequencies: tokens in ``argsort(descending=True)`` order each go to the expert
        with the smallest accumulated load (ties: lowest expert index); loads accumulate in
        double precision exactly as the reference's Python floats do.  A heap of
        (load, expert) pairs picks the same expert as the reference's linear ``min``.
        Without frequencies: ``token_id % num_experts``.
        """
        if token_frequencies is None:
            return torch.arange(vocab_size, dtype=torch.long) % num_experts
        if token_frequencies.shape[0] != vocab_size:
            raise ValueError("token_frequencies must have one entry per vocabulary item")
        order = token_frequencies.argsort(descending=True).tolist()
        freq = token_frequencies.tolist()
        table = [0] * vocab_size
        heap = [(0.0, e) for e in range(num_experts)]
        for tid in order:
            load, e = heapq.heappop(heap)
            table[tid] = e
            heapq.heappush(heap, (load + freq[tid], e))
        return torch.tensor(table, dtype=torch.long)

    def _table_signature(self) -> Tuple:
        t = self.token_to_expert
        key = (t.data_ptr(), t._version, t.device, tuple(t.shape))
        if key != self._table_sig_key:
            host = t.detach().cpu()
            if host.numel() != self.vocab_size:
                raise ValueError("token_to_expert must have vocab_size entries")
            if host.numel() and (int(host.min()) < 0 or int(host.max()) >= self.num_experts):
                raise ValueError("token_to_expert holds expert ids outside [0, num_experts)")
            digest = hashlib.sha1(host.numpy().tobytes()).hexdigest()
            self._table_sig = (digest, self.num_experts, self.vocab_size)
            self._table_sig_key = key
        return self._table_sig

    def routing(self, token_ids: torch.Tensor) -> ops.Routing:
        """Dispatch artefacts for `token_ids` (cached across the layers of a forward)."""
        if token_ids.dtype != torch.int64:
            token_ids = token_ids.long()
        return ROUTING_CACHE.lookup(token_ids, self.token_to_expert, self._table_signature(),
                                    self.num_experts)

    # ------------------------------------------------------------------ packed weights
    def _packed_routed(self, rows: Optional[int] = None):
        g, u = self.gate_proj_w, self.up_proj_w
        bn = ops.choose_block_n(self.expert_intermediate_size, rows, self.num_experts)
        packed = self._derived.get(
            f"routed_gate_up_{bn}", (g, u),
            lambda: ops.pack_gate_up(g.detach().contiguous(), u.detach().contiguous(), bn,
                                     feature_major=False))
        return packed, bn

    def _packed_shared(self, rows: Optional[int] = None):
        g, u = self.shared_gate.weight, self.shared_up.weight
        bn = ops.choose_block_n(g.shape[0], rows)
        packed = self._derived.get(
            f"shared_gate_up_{bn}", (g, u),
            lambda: ops.pack_gate_up(g.detach()[None].contiguous(), u.detach()[None].contiguous(), bn))
        return packed, bn

    def _down_routed(self) -> torch.Tensor:
        d = self.down_proj_w
        return self._derived.get("routed_down", (d,),
                                 lambda: ops.pack_down(d.detach().contiguous()))  # [E, H, I_e]

    # ------------------------------------------------------------------ compute
    def forward_sorted(self, x_sorted: torch.Tensor, routing: ops.Routing,
                       residual: Optional[torch.Tensor],
                       residual_lo: Optional[torch.Tensor] = None, want_lo: bool = False):
        """MoE on rows already grouped by expert; returns rows in ORIGINAL order,
        ``out[perm[j]] = shared(x_j) + expert(x_j) (+ residual[perm[j]])``.  `residual_lo` /
        `want_lo`: the residual stream as a split-bf16 pair (returns (out, out_lo))."""
        rows = x_sorted.shape[0]
        if routing.perm.numel() != rows:
            raise ValueError(f"token_ids has {routing.perm.numel()} entries for {rows} tokens")
        packed_r, bn_r = self._packed_routed(rows)
        h_s = wd_s = None
        if self.use_shared_expert:
            packed_s, bn_s = self._packed_shared(rows)
            wd_s = self.shared_down.weight.detach()
            I_s = self.shared_gate.weight.shape[0]
        if self.use_shared_expert and bn_s == bn_r:
            # routed and shared up-projections share one launch (one tail instead of two)
            h_r, h_s = ops.moe_up_pair(x_sorted, routing.offsets, self.num_experts, packed_r,
                                       self.expert_intermediate_size, packed_s, I_s, bn_r)
        else:
            h_r = ops.moe_up(x_sorted, routing.offsets, self.num_experts, packed_r,
                             self.expert_intermediate_size, bn_r)
            if self.use_shared_expert:
                h_s = ops.moe_up(x_sorted, None, 1, packed_s, I_s, bn_s)
        return ops.moe_down(h_r, self._down_routed(), h_s, wd_s, routing.offsets,
                            self.num_experts, routing.perm, residual, residual_lo, want_lo)

    def forward(self, hidden_states: torch.Tensor, token_ids: Optional[torch.Tensor] = None
                ) -> torch.Tensor:
        ops.forward_only(hidden_states, "TokenRoutedMLP")
        B, S, H = hidden_states.shape
        if token_ids is None:
            return self._forward_all_experts(hidden_states)
        if token_ids.numel() != B * S:
            raise ValueError(f"token_ids has {token_ids.numel()} entries for {B * S} tokens")
        routing = self.routing(token_ids)
        x2 = hidden_states.reshape(-1, H).contiguous()
        x_sorted = ops.gather_rows(x2, routing.perm)
        return self.forward_sorted(x_sorted, routing, None).view(B, S, H)

    def _forward_all_experts(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """No token ids: mean over all routed experts (+ shared), reference :180-194."""
        shape = hidden_states.shape
        x2 = hidden_states.reshape(-1, shape[-1]).contiguous()
        packed_r, bn_r = self._packed_routed()
        wd_r = self._down_routed()
        acc = torch.zeros(x2.shape, dtype=torch.float32, device=x2.device)
        for e in range(self.num_experts):
            h = ops.moe_up(x2, None, 1, packed_r[e:e + 1], self.expert_intermediate_size, bn_r)
            acc += ops.moe_down(h, wd_r[e:e + 1], None, None, None, 1, None, None).float()
        acc /= self.num_experts
        if self.use_shared_expert:
            packed_s, bn_s = self._packed_shared()
            h = ops.moe_up(x2, None, 1, packed_s, self.shared_gate.weight.shape[0], bn_s)
            acc += ops.moe_down(h, self.shared_down.weight.detach()[None], None, None, None, 1,
                                None, None).float()
        return acc.to(hidden_states.dtype).view(shape)
