"""Expert-parallel execution of the token-routed MoE layer over the GPUs of one node.

The reference has no distributed code; this is the sharded form of
``TokenRoutedMLP.forward`` (complexity_deep/core/token_routed_mlp.py:125-178) for expert
counts >= GPU count: tokens stay data-parallel, the routed experts are split
``experts_per_rank`` per GPU (expert e lives on rank ``e // experts_per_rank``), the shared
expert is replicated and runs on the token's home GPU.

Per layer: local dispatch (cd_route) -> rows sorted by expert are also sorted by destination
rank, so ONE ``all_to_all_single`` with exact split sizes (routing is known from the token
ids, nothing is padded) sends them to their experts -> grouped SwiGLU experts on the received
rows -> a second all-to-all returns the down-projected rows -> the home GPU adds
shared + routed + residual in fp32 in its GEMM epilogue (cd_moe_combine).  The shared
expert's up-projection is enqueued while the dispatch is in flight.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from . import ops
from .core.token_routed_mlp import TokenRoutedMLP


@dataclass
class ExchangePlan:
    """Split sizes and index maps of one id batch on one rank (host integers + device maps)."""
    in_splits: List[int]        # rows this rank sends to rank j (its rows of rank j's experts)
    out_splits: List[int]       # rows this rank receives from rank i
    received: int               # sum(out_splits)
    seg_offsets: np.ndarray     # [experts_per_rank + 1] segments of the expert-grouped order
    gather_idx: np.ndarray      # [received] expert-grouped position -> position in receive order


def exchange_plan(counts: np.ndarray, rank: int, experts_per_rank: int) -> ExchangePlan:
    """Exact exchange arithmetic from the [ranks, experts] count matrix.

    Rank i's send buffer is sorted by expert, hence by destination rank; the rows rank `rank`
    receives are ordered source-major, expert-minor.  The experts want them expert-major
    (one contiguous segment per local expert), source-minor — `gather_idx` is that
    permutation, and it is also the row map that puts results back in receive order.
    """
    counts = np.asarray(counts, dtype=np.int64)
    G, E = counts.shape
    El = experts_per_rank
    if G * El != E:
        raise ValueError(f"{E} experts do not split {El} per rank over {G} ranks")
    mine = counts[:, rank * El:(rank + 1) * El]                 # [source, local expert]
    in_splits = counts[rank].reshape(G, El).sum(axis=1)
    out_splits = mine.sum(axis=1)
    received = int(out_splits.sum())
    # start of block (source i, expert e) in receive order
    recv_start = np.concatenate([[0], np.cumsum(mine.reshape(-1))])[:-1].reshape(G, El)
    per_expert = mine.sum(axis=0)
    seg_offsets = np.concatenate([[0], np.cumsum(per_expert)])
    gather_idx = np.empty(received, dtype=np.int64)
    pos = 0
    for e in range(El):
        for i in range(G):
            n = int(mine[i, e])
            gather_idx[pos:pos + n] = recv_start[i, e] + np.arange(n)
            pos += n
    return ExchangePlan([int(v) for v in in_splits], [int(v) for v in out_splits], received,
                        seg_offsets.astype(np.int32), gather_idx.astype(np.int32))


def balanced_placement(expert_load, world: int) -> List[int]:
    """Longest-processing-time placement: experts in order of decreasing load each go to the
    rank with the smallest load so far that still has a free slot (E / world slots per rank).

    Returns `order`, a permutation of the expert ids: rank r owns ``order[r*El:(r+1)*El]``.
    The Zipf head token makes one expert much heavier than the mean and bin-packing cannot
    split a token, so with contiguous placement one GPU gets the two heaviest experts; this
    spreads them.
    """
    load = [float(v) for v in expert_load]
    E = len(load)
    if E % world:
        raise ValueError(f"{E} experts cannot be split evenly over {world} ranks")
    El = E // world
    slots: List[List[int]] = [[] for _ in range(world)]
    totals = [0.0] * world
    for e in sorted(range(E), key=lambda i: (-load[i], i)):
        r = min((r for r in range(world) if len(slots[r]) < El), key=lambda r: (totals[r], r))
        slots[r].append(e)
        totals[r] += load[e]
    return [e for r in range(world) for e in sorted(slots[r])]


class ExpertParallelMoE:
    """Sharded runner for one ``TokenRoutedMLP``.

    `mlp` is a full module (every rank builds or loads the same one); this object keeps only
    the packed weights of the rank's own experts plus the replicated shared expert, so the
    full routed weights can be freed by the caller afterwards.
    """

    def __init__(self, mlp: TokenRoutedMLP, group: Optional[dist.ProcessGroup] = None,
                 expert_load=None):
        """`expert_load` (one number per expert, e.g. the summed token frequencies of its
        tokens, identical on every rank) switches from contiguous placement (expert e on rank
        e // El) to `balanced_placement`."""
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.mlp = mlp
        E = mlp.num_experts
        if E % self.world:
            raise ValueError(f"{E} experts cannot be split evenly over {self.world} ranks")
        self.experts_per_rank = El = E // self.world
        # order[new id] = original expert id; rank r owns new ids r*El .. (r+1)*El - 1
        order = list(range(E)) if expert_load is None else balanced_placement(expert_load, self.world)
        self.order = order
        mine = torch.tensor(order[self.rank * El:(self.rank + 1) * El],
                            device=mlp.gate_proj_w.device)
        I_e = mlp.expert_intermediate_size
        self.block_n = ops.choose_block_n(I_e)
        with torch.no_grad():
            self.packed_local = ops.pack_gate_up(
                mlp.gate_proj_w.detach().index_select(0, mine).transpose(1, 2),
                mlp.up_proj_w.detach().index_select(0, mine).transpose(1, 2), self.block_n)
            self.down_local = mlp.down_proj_w.detach().index_select(0, mine).transpose(1, 2).contiguous()
        self._relabel = None
        if expert_load is not None:
            new_of_old = [0] * E
            for new, old in enumerate(order):
                new_of_old[old] = new
            self._relabel = torch.tensor(new_of_old, dtype=torch.long)
        self._table = None
        self._table_key = None
        self._plans = {}

    def routing(self, token_ids: torch.Tensor) -> ops.Routing:
        """Dispatch with expert ids renumbered so that every rank's experts are contiguous."""
        if self._relabel is None:
            return self.mlp.routing(token_ids)
        from .core.token_routed_mlp import ROUTING_CACHE
        sig = self.mlp._table_signature()
        if self._table_key != sig:
            t = self.mlp.token_to_expert
            self._table = self._relabel.to(t.device)[t]
            self._table_key = sig
        if token_ids.dtype != torch.int64:
            token_ids = token_ids.long()
        return ROUTING_CACHE.lookup(token_ids, self._table, ("ep", tuple(self.order)) + sig,
                                    self.mlp.num_experts)

    # ------------------------------------------------------------------ plan
    def plan_for(self, routing: ops.Routing):
        """Exchange plan of a routed batch (one small all-gather and one device->host copy per
        NEW id batch; cached for the other layers of the forward)."""
        key = id(routing)
        hit = self._plans.get(key)
        if hit is not None and hit[0] is routing:
            return hit[1], hit[2], hit[3]
        E = self.mlp.num_experts
        all_counts = torch.empty(self.world, E, dtype=torch.int32, device=routing.counts.device)
        dist.all_gather_into_tensor(all_counts, routing.counts, group=self.group)
        plan = exchange_plan(all_counts.cpu().numpy(), self.rank, self.experts_per_rank)
        dev = routing.counts.device
        seg = torch.from_numpy(plan.seg_offsets).to(dev)
        gidx = torch.from_numpy(plan.gather_idx).to(dev)
        if len(self._plans) > 8:
            self._plans.clear()
        self._plans[key] = (routing, plan, seg, gidx)
        return plan, seg, gidx

    # ------------------------------------------------------------------ forward
    def forward_sorted(self, x_sorted: torch.Tensor, routing: ops.Routing,
                       residual: Optional[torch.Tensor]) -> torch.Tensor:
        """x_sorted: this rank's rows in expert-sorted order [T_local, H]; returns rows in
        ORIGINAL order with shared + routed (+ residual) combined in fp32."""
        mlp = self.mlp
        H = x_sorted.shape[1]
        plan, seg, gidx = self.plan_for(routing)
        recv = torch.empty(plan.received, H, dtype=x_sorted.dtype, device=x_sorted.device)
        work = dist.all_to_all_single(recv, x_sorted, plan.out_splits, plan.in_splits,
                                      group=self.group, async_op=True)
        # shared expert of the local tokens while the dispatch is in flight
        h_s = wd_s = None
        if mlp.use_shared_expert:
            packed_s, bn_s = mlp._packed_shared()
            h_s = ops.moe_up(x_sorted, None, 1, packed_s, mlp.shared_gate.weight.shape[0], bn_s)
            wd_s = mlp.shared_down.weight.detach()
        work.wait()
        # local experts on the received rows
        if plan.received > 0:
            xe = ops.gather_rows(recv, gidx)
            h_r = ops.moe_up(xe, seg, self.experts_per_rank, self.packed_local,
                             mlp.expert_intermediate_size, self.block_n)
            y_recv = ops.moe_down(h_r, self.down_local, None, None, seg, self.experts_per_rank,
                                  gidx, None)                       # back in receive order
        else:
            y_recv = recv
        y_sorted = torch.empty_like(x_sorted)
        dist.all_to_all_single(y_sorted, y_recv, plan.in_splits, plan.out_splits,
                               group=self.group)
        if h_s is not None:
            return ops.moe_combine(h_s, wd_s, y_sorted, routing.perm, residual)
        # no shared expert: un-permute (+ residual) only
        out = ops.gather_rows(y_sorted, routing.inv_perm)
        return out if residual is None else out + residual.reshape(out.shape)

    def forward(self, hidden_states: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        """Drop-in for ``TokenRoutedMLP.forward`` on this rank's tokens."""
        shape = hidden_states.shape
        H = shape[-1]
        routing = self.routing(token_ids)
        x_sorted = ops.gather_rows(hidden_states.reshape(-1, H).contiguous(), routing.perm)
        return self.forward_sorted(x_sorted, routing, None).view(shape)

    __call__ = forward
