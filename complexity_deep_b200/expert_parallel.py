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


def push_plan(counts: np.ndarray, rank: int, experts_per_rank: int, ret_ptrs: List[int],
              row_bytes: int):
    """Index arithmetic of the exchange by peer stores (no NCCL call on the data path).

    Receive buffers are laid out expert-major, source-minor — the order the grouped GEMM wants —
    so nothing is regrouped on arrival.  Returns
      push_base  [E] int32: row in the owner's receive buffer where THIS rank's rows of expert
                 e start (the owner's segment start of e plus the rows of lower-ranked sources);
      seg_offsets [El + 1] int32: segments of this rank's own receive buffer;
      received   rows this rank receives;
      row_ptrs   [received] int64: for every received row, the address of its slot in its home
                 rank's return buffer (home base + (home's sorted offset of e + k) * row_bytes).
    """
    counts = np.asarray(counts, dtype=np.int64)
    G, E = counts.shape
    El = experts_per_rank
    if G * El != E:
        raise ValueError(f"{E} experts do not split {El} per rank over {G} ranks")
    per_expert = counts.sum(axis=0)                              # rows of expert e over all sources
    seg_start = np.zeros(E, dtype=np.int64)                      # start of e in ITS OWNER's buffer
    for r in range(G):
        block = per_expert[r * El:(r + 1) * El]
        seg_start[r * El:(r + 1) * El] = np.concatenate([[0], np.cumsum(block)[:-1]])
    before = np.concatenate([np.zeros((1, E), np.int64), np.cumsum(counts, axis=0)[:-1]])  # [G, E]
    push_base = seg_start + before[rank]
    mine = counts[:, rank * El:(rank + 1) * El]                  # [source, local expert]
    seg_offsets = np.concatenate([[0], np.cumsum(mine.sum(axis=0))])
    received = int(seg_offsets[-1])
    home_off = np.concatenate([np.zeros((G, 1), np.int64), np.cumsum(counts, axis=1)[:, :-1]], 1)
    row_ptrs = np.empty(received, dtype=np.int64)
    pos = 0
    for e in range(El):
        ge = rank * El + e
        for i in range(G):
            n = int(mine[i, e])
            row_ptrs[pos:pos + n] = ret_ptrs[i] + (home_off[i, ge] + np.arange(n)) * row_bytes
            pos += n
    return push_base.astype(np.int32), seg_offsets.astype(np.int32), received, row_ptrs


def push_plan_tensors(counts: torch.Tensor, rank: int, experts_per_rank: int,
                      ret_ptrs: torch.Tensor, row_bytes: int, capacity: int):
    """`push_plan` with tensor operations on the device that holds `counts` ([ranks, E]), so the
    layer needs no device->host copy: nothing here depends on a host-side value of the counts.
    `ret_ptrs`: int64 [ranks] base addresses of the ranks' return buffers.  `row_ptrs` has
    `capacity` entries; entries past the received rows are never used (the grouped GEMM's tile
    schedule comes from `seg_offsets` on the device)."""
    G, E = counts.shape
    El = experts_per_rank
    c = counts.to(torch.int64)
    per_expert = c.sum(dim=0).view(G, El)
    seg_start = (per_expert.cumsum(dim=1) - per_expert).reshape(E)
    before = c.cumsum(dim=0) - c
    push_base = (seg_start + before[rank]).to(torch.int32)
    mine = c[:, rank * El:(rank + 1) * El]                                   # [source, local e]
    zero = torch.zeros(1, dtype=torch.int64, device=c.device)
    seg_offsets = torch.cat([zero, mine.sum(dim=0).cumsum(dim=0)]).to(torch.int32)
    blocks = mine.t().reshape(-1)                                            # (local e, source)
    block_end = blocks.cumsum(dim=0)
    block_start = block_end - blocks
    rows = torch.arange(capacity, dtype=torch.int64, device=c.device)
    bid = torch.searchsorted(block_end, rows, right=True).clamp_(max=El * G - 1)
    k = rows - block_start[bid]
    e_loc, src = bid // G, bid % G
    home_off = c.cumsum(dim=1) - c                                           # [rank, expert]
    slot = home_off[src, rank * El + e_loc] + k
    row_ptrs = ret_ptrs[src] + slot * row_bytes
    return push_base, seg_offsets, row_ptrs


def plan_kernel_fits(world: int, num_experts: int) -> bool:
    """Whether cd_ep_plan takes the count matrix of `world` ranks x `num_experts` experts."""
    return world * num_experts <= 8192 and num_experts <= 2048


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


class _PeerContext:
    """Symmetric buffers, their handles and the per-batch plans, shared by every layer that
    uses the same process group, row width, capacity and expert placement: the layers of a
    model run one after the other, and the barriers of the exchange order the re-use."""
    pool = {}

    def __init__(self):
        self.buffers = None      # (recv, ret, recv_handle, ret_handle)
        self.ret_ptrs = None
        self.flags = None        # this rank's barrier signal pad, int32 [1 + world] (symmetric)
        self.flag_ptrs = None    # int64 [world]: every rank's pad as seen from this GPU
        self.plans = {}
        self.counts = None       # int32 [2, world, E] (symmetric): count matrices of the last two batches
        self.count_ptrs = None   # int64 [world]: every rank's counts buffer as seen from this GPU
        self.count_seq = 0       # batches planned so far (selects the slot; the same on every rank)

    @classmethod
    def get(cls, key):
        ctx = cls.pool.get(key)
        if ctx is None:
            ctx = cls.pool[key] = cls()
        return ctx


class ExpertParallelMoE:
    """Sharded runner for one ``TokenRoutedMLP``.

    `mlp` is a full module (every rank builds or loads the same one); this object keeps only
    the packed weights of the rank's own experts plus the replicated shared expert, so the
    full routed weights can be freed by the caller afterwards.
    """

    def __init__(self, mlp: TokenRoutedMLP, group: Optional[dist.ProcessGroup] = None,
                 expert_load=None, exchange: str = "nccl", max_tokens_per_rank: int = 0):
        """`expert_load` (one number per expert, e.g. the summed token frequencies of its
        tokens, identical on every rank) switches from contiguous placement (expert e on rank
        e // El) to `balanced_placement`.

        `exchange`: "nccl" — two all_to_all_single per call; "peer" — the rows are stored
        straight into the other GPUs' buffers (symmetric memory over NVLink) by the kernels
        that produce them: a push kernel for the dispatch, the down-projection's epilogue for
        the way back, with a cross-GPU barrier kernel of this library (bounded wait)
        between the phases and no NCCL call on the data path.  "peer" needs `max_tokens_per_rank` (same on every rank) to size the
        buffers once."""
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.exchange = exchange
        self.max_tokens = int(max_tokens_per_rank)
        self.barrier_limit_ms = 2000
        self._peer = None
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
                mlp.gate_proj_w.detach().index_select(0, mine),
                mlp.up_proj_w.detach().index_select(0, mine), self.block_n, feature_major=False)
            self.down_local = ops.pack_down(mlp.down_proj_w.detach().index_select(0, mine))
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

    # ------------------------------------------------------------------ peer exchange
    def _peer_context(self, H: int) -> _PeerContext:
        if self._peer is None:
            group = self.group if self.group is not None else dist.group.WORLD
            self._peer = _PeerContext.get((group.group_name, H, self.max_tokens,
                                           self.mlp.num_experts, tuple(self.order)))
        return self._peer

    def _peer_buffers(self, H: int, device):
        """Symmetric (peer-mapped) receive and return buffers, allocated once per context."""
        ctx = self._peer_context(H)
        if ctx.buffers is None:
            import os
            # plain peer loads/stores only: no NVLink multicast object is bound to these buffers
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem
            if self.max_tokens <= 0:
                raise ValueError("exchange='peer' needs max_tokens_per_rank")
            group = self.group if self.group is not None else dist.group.WORLD
            recv = symm_mem.empty(self.world * self.max_tokens, H, dtype=torch.bfloat16,
                                  device=device)
            ret = symm_mem.empty(self.max_tokens, H, dtype=torch.bfloat16, device=device)
            recv_h = symm_mem.rendezvous(recv, group=group)
            ret_h = symm_mem.rendezvous(ret, group=group)
            flags = symm_mem.empty(64, dtype=torch.int32, device=device)
            flags.zero_()
            flags_h = symm_mem.rendezvous(flags, group=group)
            ctx.buffers = (recv, ret, recv_h, ret_h)
            ctx.ret_ptrs = torch.tensor([int(p) for p in ret_h.buffer_ptrs], dtype=torch.int64,
                                        device=device)
            # two slots of [world, E] counts: the all-gather of a batch's counts by peer stores
            E = self.mlp.num_experts
            counts = symm_mem.empty(2 * self.world * E, dtype=torch.int32, device=device)
            counts.zero_()
            counts_h = symm_mem.rendezvous(counts, group=group)
            ctx.counts, ctx.counts_handle = counts, counts_h
            ctx.count_ptrs = torch.tensor([int(p) for p in counts_h.buffer_ptrs], dtype=torch.int64,
                                          device=device)
            ctx.flags, ctx.flags_handle = flags, flags_h
            ctx.flag_ptrs = torch.tensor([int(p) for p in flags_h.buffer_ptrs], dtype=torch.int64,
                                         device=device)
            # every pad is zeroed before any rank's first barrier kernel can write into it
            torch.cuda.synchronize(device)
            dist.barrier(group=group)
        return ctx.buffers

    def _barrier(self, H: int, tag: str = "peer_barrier") -> None:
        """Cross-GPU barrier between two phases of the peer exchange (cd_peer_barrier): a
        bounded device-side wait that raises the library's status word instead of spinning
        forever when a rank never arrives."""
        ctx = self._peer_context(H)
        ops.peer_barrier(ctx.flag_ptrs, ctx.flags, self.rank, self.world, self.barrier_limit_ms, tag)

    def peer_plan_for(self, routing: ops.Routing, H: int):
        """Exchange plan of a routed batch for the peer-store exchange, computed on the device
        from the count rows of all ranks (gathered by peer stores: no collective library call,
        no device->host copy); cached per batch and shared by all layers of the context."""
        recv, ret, recv_h, ret_h = self._peer_buffers(H, routing.counts.device)
        ctx = self._peer_context(H)
        key = id(routing)
        hit = ctx.plans.get(key)
        if hit is not None and hit[0] is routing:
            return hit[1:]
        E = self.mlp.num_experts
        dev = routing.counts.device
        # all-gather of the counts by peer stores: every rank writes its row into every rank's
        # buffer, the barrier makes the rows visible.  Slots alternate; a rank can only be one
        # batch ahead of another (the later barriers of the layer hold it), so a row is never
        # overwritten while a peer's plan kernel may still read it.
        slot = ctx.count_seq & 1
        ctx.count_seq += 1
        ops.peer_put_i32(routing.counts, ctx.count_ptrs, self.world, (slot * self.world + self.rank) * E)
        self._barrier(H, "peer_barrier_counts")
        all_counts = ctx.counts[slot * self.world * E:(slot + 1) * self.world * E].view(self.world, E)
        if plan_kernel_fits(self.world, E):
            out = ops.ep_plan(all_counts, self.rank, self.experts_per_rank, ctx.ret_ptrs, H * 2,
                              recv.shape[0])
        else:   # more ranks x experts than one plan launch holds: the same arithmetic as tensor operations
            out = push_plan_tensors(all_counts, self.rank, self.experts_per_rank, ctx.ret_ptrs,
                                    H * 2, recv.shape[0])
        if len(ctx.plans) > 8:
            ctx.plans.clear()
        ctx.plans[key] = (routing,) + out
        return out

    def _check_batch(self, x_sorted: torch.Tensor, routing: ops.Routing) -> None:
        """Host-side checks of one call, made BEFORE any collective or launch of that call, so a
        rank that raises has nothing in flight and no peer buffer can be overrun (a rank never
        sends more than max_tokens rows, so no rank receives more than its buffer holds)."""
        T = x_sorted.shape[0]
        if routing.perm.numel() != T:
            raise ValueError(f"token_ids has {routing.perm.numel()} entries for {T} tokens")
        if routing.num_experts != self.mlp.num_experts:
            raise ValueError("routing was computed for another expert count")
        if self.exchange == "peer":
            if self.max_tokens <= 0:
                raise ValueError("exchange='peer' needs max_tokens_per_rank")
            if T > self.max_tokens:
                raise ValueError(f"{T} tokens on this rank, but the exchange buffers were sized "
                                 f"for max_tokens_per_rank={self.max_tokens}")

    def _forward_sorted_peer(self, x_sorted, routing, residual, residual_lo, want_lo):
        mlp = self.mlp
        T, H = x_sorted.shape
        recv, ret, recv_h, ret_h = self._peer_buffers(H, x_sorted.device)
        push_base, seg, row_ptrs = self.peer_plan_for(routing, H)
        # dispatch: every row goes straight into its expert's GPU
        ops.push_rows(x_sorted, routing.offsets, push_base, mlp.num_experts,
                      self.experts_per_rank, recv_h.buffer_ptrs_dev)
        h_s = wd_s = None
        if mlp.use_shared_expert:          # local work while the pushes of the peers land
            packed_s, bn_s = mlp._packed_shared(T)
            h_s = ops.moe_up(x_sorted, None, 1, packed_s, mlp.shared_gate.weight.shape[0], bn_s)
            wd_s = mlp.shared_down.weight.detach()
        self._barrier(H, "peer_barrier_dispatch")   # all pushes visible; also: peers are done reading `ret`
        # The number of received rows is only known on the device: the GEMMs are launched over
        # the whole buffer and schedule tiles from `seg` (device), so rows past the last segment
        # are never touched.
        h_r = ops.moe_up(recv, seg, self.experts_per_rank, self.packed_local,
                         mlp.expert_intermediate_size, self.block_n)
        # the epilogue stores every finished row in its home GPU's return buffer
        ops.moe_down_push(h_r, self.down_local, seg, self.experts_per_rank, row_ptrs)
        self._barrier(H, "peer_barrier_return")     # all routed rows are home; peers are done reading `recv`
        y_sorted = ret[:T]
        if h_s is not None:
            return ops.moe_combine(h_s, wd_s, y_sorted, routing.perm, residual, residual_lo, want_lo)
        return self._unpermute_only(y_sorted, routing, residual, residual_lo, want_lo)

    @staticmethod
    def _unpermute_only(y_sorted, routing, residual, residual_lo, want_lo):
        """No shared expert: un-permute the routed rows (+ residual) with PyTorch operators."""
        out = ops.gather_rows(y_sorted, routing.inv_perm)
        if residual is None:
            return (out, None) if want_lo else out
        total = out.float() + residual.reshape(out.shape).float()
        if residual_lo is not None:
            total = total + residual_lo.reshape(out.shape).float()
        hi = total.to(out.dtype)
        return (hi, (total - hi.float()).to(out.dtype)) if want_lo else hi

    # ------------------------------------------------------------------ forward
    def forward_sorted(self, x_sorted: torch.Tensor, routing: ops.Routing,
                       residual: Optional[torch.Tensor],
                       residual_lo: Optional[torch.Tensor] = None, want_lo: bool = False):
        """x_sorted: this rank's rows in expert-sorted order [T_local, H]; returns rows in
        ORIGINAL order with shared + routed (+ residual) combined in fp32.  `residual_lo` /
        `want_lo`: split-bf16 residual stream as in TokenRoutedMLP.forward_sorted."""
        self._check_batch(x_sorted, routing)
        if self.exchange == "peer":
            return self._forward_sorted_peer(x_sorted, routing, residual, residual_lo, want_lo)
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
            return ops.moe_combine(h_s, wd_s, y_sorted, routing.perm, residual, residual_lo, want_lo)
        return self._unpermute_only(y_sorted, routing, residual, residual_lo, want_lo)

    def forward(self, hidden_states: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        """Drop-in for ``TokenRoutedMLP.forward`` on this rank's tokens."""
        shape = hidden_states.shape
        H = shape[-1]
        if token_ids.numel() != hidden_states.numel() // H:
            raise ValueError(f"token_ids has {token_ids.numel()} entries for "
                             f"{hidden_states.numel() // H} tokens")
        routing = self.routing(token_ids)
        x_sorted = ops.gather_rows(hidden_states.reshape(-1, H).contiguous(), routing.perm)
        return self.forward_sorted(x_sorted, routing, None).view(shape)

    __call__ = forward
