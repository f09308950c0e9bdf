"""Tensor-level wrappers over the libcdeep C ABI.

PyTorch is used for device memory and streams only: each function checks its arguments,
allocates outputs with ``torch.empty`` on the caller's device and enqueues the CUDA kernels
on ``torch.cuda.current_stream()``.  Nothing here computes on the CPU and nothing falls
back to PyTorch operators.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib

BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=BF16) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(
            f"{name}: expected a CUDA tensor; the complexity_deep_b200 kernels have no CPU path")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: expected a contiguous tensor")


def forward_only(x: torch.Tensor, what: str) -> None:
    """The kernels are forward-only.  An activation that carries autograd history would lose
    its gradient silently, so that case is refused instead."""
    if torch.is_grad_enabled() and isinstance(x, torch.Tensor) and x.requires_grad:
        raise RuntimeError(
            f"{what}: the complexity_deep_b200 kernels implement the forward pass only; call the "
            "model under torch.no_grad() / torch.inference_mode() (no backward is available)")


class _Profile:
    """Optional CUDA-event timing of the GEMM entry points (used by bench.py).

    Disabled by default: then `span` costs one attribute check.  When enabled, every call of
    an instrumented entry point records an event before and after its launch on the current
    stream; `collect` synchronises and returns per-entry launch counts and device time.
    """

    def __init__(self) -> None:
        self.enabled = False
        self.events = []
        self.kernel_launches = 0

    def reset(self, enabled: bool) -> None:
        self.enabled = enabled
        self.events = []
        self.kernel_launches = 0

    def collect(self):
        """name -> (calls, total_ms, kernels launched)."""
        torch.cuda.synchronize()
        out = {}
        for name, a, b, n in self.events:
            c, ms, k = out.get(name, (0, 0.0, 0))
            out[name] = (c + 1, ms + a.elapsed_time(b), k + n)
        return out


PROFILE = _Profile()


class _Span:
    def __init__(self, name: str, kernels: int = 1) -> None:
        self.name, self.kernels = name, kernels

    def __enter__(self):
        if PROFILE.enabled:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if PROFILE.enabled:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            PROFILE.events.append((self.name, self.start, end, self.kernels))
        return False


def status_fetch() -> int:
    """Synchronises and returns the kernels' status word (0 = ok); raises on a timeout."""
    lib = _lib.load()
    st = ctypes.c_int(0)
    _lib.check(lib.cd_status_fetch(ctypes.byref(st)), "cd_status_fetch")
    if st.value == 4:
        raise _lib.CdeepError("checking build: a libcdeep kernel met an index, address or segment "
                              "table out of range and skipped the access")
    if st.value != 0:
        raise _lib.CdeepError("a libcdeep kernel gave up on a bounded wait (pipeline error)")
    return st.value


# --------------------------------------------------------------------------- dispatch
@dataclass
class Routing:
    """Routing artefacts of one batch of token ids (all int32, on the device)."""
    expert_ids: torch.Tensor   # [T]
    counts: torch.Tensor       # [E]
    offsets: torch.Tensor      # [E + 1]
    perm: torch.Tensor         # [T] sorted position -> source row
    inv_perm: torch.Tensor     # [T] source row -> sorted position
    num_experts: int


def route(token_ids: torch.Tensor, table: torch.Tensor, num_experts: int) -> Routing:
    lib = _lib.load()
    ids = token_ids.reshape(-1)
    _need(ids, "token_ids", torch.int64)
    _need(table, "token_to_expert", torch.int64)
    T, V, E = ids.numel(), table.numel(), int(num_experts)
    dev = ids.device
    i32 = dict(dtype=torch.int32, device=dev)
    expert_ids = torch.empty(T, **i32)
    perm = torch.empty(T, **i32)
    inv_perm = torch.empty(T, **i32)
    counts = torch.empty(E, **i32)
    offsets = torch.empty(E + 1, **i32)
    ws_bytes = lib.cd_route_workspace_bytes(T, E)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    with _Span("route", 2):
        _lib.check(lib.cd_route(ids.data_ptr(), table.data_ptr(), V, E, T, expert_ids.data_ptr(),
                                counts.data_ptr(), offsets.data_ptr(), perm.data_ptr(),
                                inv_perm.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                   "cd_route")
    return Routing(expert_ids, counts, offsets, perm, inv_perm, E)


# --------------------------------------------------------------------------- row-wise
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float,
            residual: Optional[torch.Tensor] = None, dst_rows: Optional[torch.Tensor] = None,
            want_sum: bool = False, x_lo: Optional[torch.Tensor] = None):
    """``norm(x (+ residual)) * weight``; returns ``out`` or ``(sum, out)`` when want_sum.

    With ``dst_rows`` row i of the result is written to row ``dst_rows[i]``.  With ``x_lo``
    (the low part of a split-bf16 value, see ``SplitStream``) the input is ``x + x_lo`` in fp32.
    """
    lib = _lib.load()
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    _need(x2, "x")
    _need(weight, "weight")
    T = x2.shape[0]
    if x_lo is not None:
        if residual is not None or want_sum:
            raise RuntimeError("x_lo cannot be combined with residual / want_sum")
        lo2 = x_lo.reshape(-1, H)
        _need(lo2, "x_lo")
        if lo2.shape[0] != T:
            raise RuntimeError("x_lo does not match x")
        if dst_rows is not None:
            _need(dst_rows, "dst_rows", torch.int32)
            if dst_rows.numel() != T:
                raise RuntimeError("dst_rows must have one entry per row")
        out = torch.empty_like(x2)
        with _Span("rmsnorm"):
            _lib.check(lib.cd_rmsnorm_split(x2.data_ptr(), lo2.data_ptr(), weight.data_ptr(),
                                            float(eps), out.data_ptr(), _ptr(dst_rows), T, H,
                                            _stream()), "cd_rmsnorm_split")
        return out.view(x.shape)
    res2 = None
    if residual is not None:
        res2 = residual.reshape(-1, H)
        _need(res2, "residual")
    if dst_rows is not None:
        _need(dst_rows, "dst_rows", torch.int32)
        if dst_rows.numel() != T:
            raise RuntimeError("dst_rows must have one entry per row")
    out = torch.empty_like(x2)
    s = torch.empty_like(x2) if (want_sum and res2 is not None) else None
    with _Span("rmsnorm"):
        _lib.check(lib.cd_rmsnorm(x2.data_ptr(), _ptr(res2), weight.data_ptr(), float(eps),
                                  _ptr(s), out.data_ptr(), _ptr(dst_rows), T, H, _stream()),
                   "cd_rmsnorm")
    out = out.view(x.shape)
    if want_sum:
        return (s.view(x.shape) if s is not None else x), out
    return out


def gather_rows(x: torch.Tensor, src_rows: torch.Tensor) -> torch.Tensor:
    lib = _lib.load()
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    _need(x2, "x")
    _need(src_rows, "src_rows", torch.int32)
    out = torch.empty_like(x2)
    with _Span("gather_rows"):
        _lib.check(lib.cd_gather_rows(x2.data_ptr(), src_rows.data_ptr(), out.data_ptr(),
                                      x2.shape[0], H, _stream()), "cd_gather_rows")
    return out


def qk_norm_rope_(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                  cos: torch.Tensor, sin: torch.Tensor, eps: float, seq_len: int, pos0: int,
                  hq: int, hkv: int, head_dim: int) -> torch.Tensor:
    """In-place Q/K RMSNorm + RoPE on the fused projection buffer [T, (hq + 2 hkv) * D]."""
    lib = _lib.load()
    _need(qkv, "qkv")
    _need(cos, "cos", torch.float32)
    _need(sin, "sin", torch.float32)
    if q_w is not None:
        _need(q_w, "q_norm.weight")
        _need(k_w, "k_norm.weight")
    T = qkv.shape[0]
    if qkv.shape[1] != (hq + 2 * hkv) * head_dim:
        raise RuntimeError("qkv width does not match the head layout")
    if cos.shape[0] < pos0 + seq_len or cos.shape[1] != head_dim:
        raise RuntimeError("cos/sin tables too short for the requested positions")
    with _Span("qk_norm_rope"):
        _lib.check(lib.cd_qk_norm_rope(qkv.data_ptr(), _ptr(q_w), _ptr(k_w), cos.data_ptr(),
                                       sin.data_ptr(), float(eps), T, seq_len, pos0, hq, hkv,
                                       head_dim, _stream()), "cd_qk_norm_rope")
    return qkv


def decode_rope_append(qkv: torch.Tensor, q_w: Optional[torch.Tensor],
                       k_w: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor,
                       eps: float, hq: int, hkv: int, head_dim: int, k_cache: torch.Tensor,
                       v_cache: torch.Tensor, pos_dev: torch.Tensor) -> torch.Tensor:
    """Decode step (one row of qkv per sequence): Q/K RMSNorm + RoPE in place at the position
    held by the device scalar `pos_dev` (int32), and the row's rotated k and its v written
    into k_cache / v_cache [B, hkv, capacity, D] at that position."""
    lib = _lib.load()
    _need(qkv, "qkv")
    _need(cos, "cos", torch.float32)
    _need(sin, "sin", torch.float32)
    if q_w is not None:
        _need(q_w, "q_norm.weight")
        _need(k_w, "k_norm.weight")
    B, D = qkv.shape[0], head_dim
    cap = k_cache.shape[2]
    if qkv.shape[1] != (hq + 2 * hkv) * D:
        raise RuntimeError("qkv width does not match the head layout")
    for t, name in ((k_cache, "k cache"), (v_cache, "v cache")):
        if not t.is_cuda or t.dtype != BF16 or t.stride(-1) != 1 or tuple(t.shape) != (B, hkv, cap, D):
            raise RuntimeError(f"{name}: expected a CUDA bf16 tensor [B, kv heads, capacity, D]")
    if k_cache.stride() != v_cache.stride():
        raise RuntimeError("k and v caches must share their strides")
    if cos.shape[0] < cap or cos.shape[1] != D or sin.shape != cos.shape:
        raise RuntimeError("cos/sin tables must cover the cache capacity")
    if pos_dev.dtype != torch.int32 or not pos_dev.is_cuda or pos_dev.numel() != 1:
        raise RuntimeError("pos_dev: expected one int32 on the device")
    with _Span("decode_rope_append"):
        _lib.check(lib.cd_decode_rope_append(
            qkv.data_ptr(), _ptr(q_w), _ptr(k_w), cos.data_ptr(), sin.data_ptr(), float(eps), B,
            hq, hkv, D, k_cache.data_ptr(), v_cache.data_ptr(), k_cache.stride(0),
            k_cache.stride(1), k_cache.stride(2), cap, pos_dev.data_ptr(), _stream()),
            "cd_decode_rope_append")
    return qkv


def decode_attention(qkv: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     mask: Optional[torch.Tensor], hq: int, hkv: int, head_dim: int,
                     kv_len_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-query attention: qkv [B, (hq + 2 hkv) * D] (its q columns are used), k / v
    [B, hkv, L, D] views of the cache (any batch / head / token strides, D contiguous),
    mask None or a bf16 additive mask viewable as [B or 1, L].  `kv_len_dev` (one int32 on the
    device): attend only the first min(L, value) cached tokens.  Returns [B, hq * D]."""
    lib = _lib.load()
    B, D = qkv.shape[0], head_dim
    L = k.shape[2]
    for t, name in ((qkv, "qkv"), (k, "k cache"), (v, "v cache")):
        if not t.is_cuda or t.dtype != BF16 or t.stride(-1) != 1:
            raise RuntimeError(f"{name}: expected a CUDA bf16 tensor with a contiguous last dim")
    if tuple(k.shape) != (B, hkv, L, D) or tuple(v.shape) != (B, hkv, L, D):
        raise RuntimeError("cache shapes do not match")
    if k.stride() != v.stride():
        raise RuntimeError("k and v caches must share their strides")
    mptr, mstride = None, 0
    if mask is not None:
        m2 = mask.reshape(-1, L)
        if m2.dtype != BF16 or not m2.is_cuda or m2.stride(1) != 1 or m2.shape[0] not in (1, B):
            raise RuntimeError("mask: expected a CUDA bf16 additive mask of shape [B or 1, 1, 1, L]")
        mptr, mstride = m2.data_ptr(), (m2.stride(0) if m2.shape[0] == B else 0)
    if kv_len_dev is not None and (kv_len_dev.dtype != torch.int32 or not kv_len_dev.is_cuda
                                   or kv_len_dev.numel() != 1):
        raise RuntimeError("kv_len_dev: expected one int32 on the device")
    ws_bytes = lib.cd_decode_attention_workspace_bytes(B, hq, hkv, L, D)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=qkv.device)
    out = torch.empty(B, hq * D, dtype=BF16, device=qkv.device)
    with _Span("decode_attention", 2):
        _lib.check(lib.cd_decode_attention(
            qkv.data_ptr(), qkv.stride(0), k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1),
            k.stride(2), mptr, mstride, float(head_dim) ** -0.5, B, hq, hkv, L, _ptr(kv_len_dev),
            D, out.data_ptr(), ws.data_ptr(), ws_bytes, _stream()), "cd_decode_attention")
    return out


def attention_prefill_supported(B: int, S: int, hq: int, hkv: int, head_dim: int) -> bool:
    return bool(_lib.load().cd_attention_prefill_supported(B, S, hq, hkv, head_dim))


def attention_prefill(qkv: torch.Tensor, batch: int, seq_len: int, hq: int, hkv: int,
                      head_dim: int) -> torch.Tensor:
    """Causal self-attention of a prompt: qkv [B * S, (hq + 2 hkv) * D] (after Q/K norm + RoPE)
    -> [B * S, hq * D]; softmax scale D ** -0.5 as scaled_dot_product_attention's default."""
    lib = _lib.load()
    _need(qkv, "qkv")
    if tuple(qkv.shape) != (batch * seq_len, (hq + 2 * hkv) * head_dim):
        raise RuntimeError("qkv shape does not match batch / sequence / head layout")
    out = torch.empty(batch * seq_len, hq * head_dim, dtype=BF16, device=qkv.device)
    with _Span("attention_prefill"):
        _lib.check(lib.cd_attention_prefill(qkv.data_ptr(), out.data_ptr(), batch, seq_len, hq, hkv,
                                            head_dim, float(head_dim) ** -0.5, _stream()),
                   "cd_attention_prefill")
    return out


# --------------------------------------------------------------------------- weights
def choose_block_n(width: int, rows: Optional[int] = None, groups: int = 1,
                   sm_count: Optional[int] = None) -> int:
    """Accumulator-tile width for the SwiGLU up-projection of an expert `width` wide.

    Many rows (prefill): 256 (128 gate + 128 up columns per tile) unless padding `width` to a
    multiple of 128 would waste more than a quarter of the tile columns; then 128 (64 + 64).
    Measured on B200 at width 704 (padded to 768, 9 % waste): 1146 TFLOP/s with 256-wide tiles
    against 672 TFLOP/s with 128-wide ones, which are bound by shared-memory bandwidth.
    Few rows (decode, `rows` <= 512): a tile is one chain of K/16 dependent MMA instructions
    whose cost hardly depends on the tile width, so the time is set by how many tiles the
    busiest SM runs back to back: the narrowest tile that leaves at most one tile per SM
    (every one of the `groups` experts has at least one row tile), else the widest.
    """
    if rows is not None and rows <= 512:
        if sm_count is None:
            sm_count = (torch.cuda.get_device_properties(torch.cuda.current_device())
                        .multi_processor_count if torch.cuda.is_available() else 148)
        m_tiles = max(groups, -(-rows // 128))
        for bn in (32, 64, 128, 256):
            if m_tiles * -(-width // (bn // 2)) <= sm_count:
                return bn
        return 256
    padded = -(-width // 128) * 128
    return 256 if (padded - width) / width <= 0.25 else 128


def pack_gate_up(gate: torch.Tensor, up: torch.Tensor, block_n: int,
                 feature_major: bool = True) -> torch.Tensor:
    """Interleaves gate and up rows per accumulator tile (cd_pack_gate_up).

    feature_major: gate, up are [G, I, H] (one output feature per row, nn.Linear layout);
    otherwise [G, H, I] (the reference's routed-expert layout ``x @ W[e]``).  Result
    [G, ceil(I / half) * block_n, H] with, for each tile, `half` gate rows then `half` up rows
    (half = block_n / 2); rows past I are zero.
    """
    lib = _lib.load()
    _need(gate, "gate weights")
    _need(up, "up weights")
    if gate.shape != up.shape or gate.dim() != 3:
        raise RuntimeError("gate and up must be 3-D tensors of the same shape")
    G = gate.shape[0]
    I, H = (gate.shape[1], gate.shape[2]) if feature_major else (gate.shape[2], gate.shape[1])
    rows = lib.cd_gate_up_packed_rows(I, block_n)
    packed = torch.empty(G, rows, H, dtype=BF16, device=gate.device)
    _lib.check(lib.cd_pack_gate_up(gate.data_ptr(), up.data_ptr(), packed.data_ptr(), G, I, H,
                                   block_n, 1 if feature_major else 0, _stream()),
               "cd_pack_gate_up")
    return packed


def pack_down(down: torch.Tensor) -> torch.Tensor:
    """[E, I, H] (``h @ W[e]``) -> [E, H, I] (one output feature per row) (cd_pack_down)."""
    lib = _lib.load()
    _need(down, "down weights")
    E, I, H = down.shape
    out = torch.empty(E, H, I, dtype=BF16, device=down.device)
    _lib.check(lib.cd_pack_down(down.data_ptr(), out.data_ptr(), E, I, H, _stream()),
               "cd_pack_down")
    return out


# --------------------------------------------------------------------------- GEMMs
def moe_up(x_sorted: torch.Tensor, seg_offsets: Optional[torch.Tensor], num_groups: int,
           packed_w: torch.Tensor, width: int, block_n: int) -> torch.Tensor:
    lib = _lib.load()
    _need(x_sorted, "x_sorted")
    _need(packed_w, "packed gate/up weights")
    T, H = x_sorted.shape
    rows = lib.cd_gate_up_packed_rows(width, block_n)
    if tuple(packed_w.shape) != (num_groups, rows, H):
        raise RuntimeError(f"packed weights have shape {tuple(packed_w.shape)}, expected "
                           f"{(num_groups, rows, H)}")
    if seg_offsets is not None:
        _need(seg_offsets, "seg_offsets", torch.int32)
    h = torch.empty(T, width, dtype=BF16, device=x_sorted.device)
    with _Span("moe_up_routed" if seg_offsets is not None else "moe_up_shared"):
        _lib.check(lib.cd_moe_up(x_sorted.data_ptr(), _ptr(seg_offsets), num_groups,
                                 packed_w.data_ptr(), h.data_ptr(), T, H, width, block_n,
                                 _stream()), "cd_moe_up")
    return h


def moe_up_pair(x_sorted: torch.Tensor, seg_offsets: torch.Tensor, num_groups: int,
                packed_w: torch.Tensor, width: int, packed_shared: torch.Tensor,
                width_shared: int, block_n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Routed (grouped) and shared (dense) SwiGLU up-projections of the same rows in one
    launch; returns (h_routed [T, width], h_shared [T, width_shared])."""
    lib = _lib.load()
    _need(x_sorted, "x_sorted")
    _need(packed_w, "packed gate/up weights")
    _need(packed_shared, "packed shared gate/up weights")
    _need(seg_offsets, "seg_offsets", torch.int32)
    T, H = x_sorted.shape
    rows = lib.cd_gate_up_packed_rows(width, block_n)
    rows_s = lib.cd_gate_up_packed_rows(width_shared, block_n)
    if tuple(packed_w.shape) != (num_groups, rows, H) or tuple(packed_shared.shape) != (1, rows_s, H):
        raise RuntimeError("packed weights do not match the widths / tile width")
    h = torch.empty(T, width, dtype=BF16, device=x_sorted.device)
    h_s = torch.empty(T, width_shared, dtype=BF16, device=x_sorted.device)
    with _Span("moe_up_pair"):
        _lib.check(lib.cd_moe_up_pair(x_sorted.data_ptr(), seg_offsets.data_ptr(), num_groups,
                                      packed_w.data_ptr(), h.data_ptr(), width,
                                      packed_shared.data_ptr(), h_s.data_ptr(), width_shared, T, H,
                                      block_n, _stream()), "cd_moe_up_pair")
    return h, h_s


def _split_args(residual, residual_lo, T, H, want_lo, device):
    """Checks the low part of a split residual and allocates the low part of the output."""
    lo2 = None
    if residual_lo is not None:
        if residual is None:
            raise RuntimeError("residual_lo without residual")
        lo2 = residual_lo.reshape(-1, H)
        _need(lo2, "residual_lo")
        if lo2.shape[0] != T:
            raise RuntimeError("residual_lo rows do not match")
    out_lo = torch.empty(T, H, dtype=BF16, device=device) if want_lo else None
    return lo2, out_lo


def moe_down(h_routed: torch.Tensor, wd_routed: torch.Tensor, h_shared: Optional[torch.Tensor],
             wd_shared: Optional[torch.Tensor], seg_offsets: Optional[torch.Tensor],
             num_experts: int, row_map: Optional[torch.Tensor],
             residual: Optional[torch.Tensor], residual_lo: Optional[torch.Tensor] = None,
             want_lo: bool = False):
    """wd_routed: [E, H, I_e] (feature rows, I_e contiguous); wd_shared: [H, I_s].
    `residual_lo` / `want_lo`: split-bf16 residual stream; with want_lo returns (out, out_lo)."""
    lib = _lib.load()
    _need(h_routed, "h_routed")
    _need(wd_routed, "routed down weights")
    T, I_e = h_routed.shape
    E, H, I_e2 = wd_routed.shape
    if E != num_experts or I_e2 != I_e:
        raise RuntimeError("routed down weights do not match h_routed")
    I_s = 0
    if h_shared is not None:
        _need(h_shared, "h_shared")
        _need(wd_shared, "shared down weight")
        I_s = h_shared.shape[1]
        if tuple(wd_shared.shape) != (H, I_s) or h_shared.shape[0] != T:
            raise RuntimeError("shared down weight does not match h_shared")
    if seg_offsets is not None:
        _need(seg_offsets, "seg_offsets", torch.int32)
    if row_map is not None:
        _need(row_map, "row_map", torch.int32)
    res2 = None
    if residual is not None:
        res2 = residual.reshape(-1, H)
        _need(res2, "residual")
        if res2.shape[0] != T:
            raise RuntimeError("residual rows do not match")
    if row_map is not None and row_map.numel() != T:
        raise RuntimeError("row_map must have one entry per row")
    lo2, out_lo = _split_args(res2, residual_lo, T, H, want_lo, h_routed.device)
    out = torch.empty(T, H, dtype=BF16, device=h_routed.device)
    with _Span("moe_down"):
        _lib.check(lib.cd_moe_down(h_routed.data_ptr(), I_e, wd_routed.data_ptr(), _ptr(h_shared),
                                   I_s, _ptr(wd_shared), _ptr(seg_offsets), E, _ptr(row_map),
                                   _ptr(res2), _ptr(lo2), out.data_ptr(), _ptr(out_lo), T, H,
                                   _stream()), "cd_moe_down")
    return (out, out_lo) if want_lo else out


def push_rows(x_sorted: torch.Tensor, offsets: torch.Tensor, push_base: torch.Tensor,
              num_experts: int, experts_per_rank: int, peer_ptrs_dev: int) -> None:
    """Writes every expert-sorted row into the receive buffer of the GPU that owns its expert
    (peer-mapped memory; `peer_ptrs_dev` = device address of the array of buffer addresses)."""
    lib = _lib.load()
    _need(x_sorted, "x_sorted")
    _need(offsets, "offsets", torch.int32)
    _need(push_base, "push_base", torch.int32)
    T, H = x_sorted.shape
    with _Span("push_rows"):
        _lib.check(lib.cd_push_rows(x_sorted.data_ptr(), None, offsets.data_ptr(),
                                    push_base.data_ptr(), num_experts, experts_per_rank,
                                    peer_ptrs_dev, T, H, _stream()), "cd_push_rows")


def peer_put_i32(src: torch.Tensor, peer_bufs: torch.Tensor, world: int, offset: int) -> None:
    """Stores the int32 vector `src` at element `offset` of every rank's (peer-mapped) buffer
    (cd_peer_put_i32); visible to the peers after the next peer_barrier."""
    lib = _lib.load()
    _need(src, "src", torch.int32)
    _need(peer_bufs, "peer buffer addresses", torch.int64)
    with _Span("peer_put"):
        _lib.check(lib.cd_peer_put_i32(src.data_ptr(), src.numel(), peer_bufs.data_ptr(), world,
                                       int(offset), _stream()), "cd_peer_put_i32")


def ep_plan(all_counts: torch.Tensor, rank: int, experts_per_rank: int, ret_ptrs: torch.Tensor,
            row_bytes: int, capacity: int):
    """Exchange plan of the expert-parallel layer from the [ranks, E] count matrix, one launch
    (cd_ep_plan): returns (push_base int32 [E], seg_offsets int32 [El + 1], row_ptrs int64 [capacity])."""
    lib = _lib.load()
    _need(all_counts, "counts of all ranks", torch.int32)
    _need(ret_ptrs, "return buffer addresses", torch.int64)
    G, E = all_counts.shape
    dev = all_counts.device
    push_base = torch.empty(E, dtype=torch.int32, device=dev)
    seg_offsets = torch.empty(experts_per_rank + 1, dtype=torch.int32, device=dev)
    row_ptrs = torch.empty(capacity, dtype=torch.int64, device=dev)
    with _Span("ep_plan"):
        _lib.check(lib.cd_ep_plan(all_counts.data_ptr(), G, E, experts_per_rank, rank,
                                  ret_ptrs.data_ptr(), row_bytes, capacity, push_base.data_ptr(),
                                  seg_offsets.data_ptr(), row_ptrs.data_ptr(), _stream()), "cd_ep_plan")
    return push_base, seg_offsets, row_ptrs


def peer_barrier(flag_ptrs: torch.Tensor, flags: torch.Tensor, rank: int, world: int,
                 limit_ms: int = 2000, tag: str = "peer_barrier") -> None:
    """Cross-GPU barrier kernel (cd_peer_barrier); `flag_ptrs` int64 [world] addresses of the
    ranks' signal pads, `flags` this rank's pad (int32 [>= 1 + world])."""
    lib = _lib.load()
    _need(flag_ptrs, "flag_ptrs", torch.int64)
    _need(flags, "flags", torch.int32)
    if flag_ptrs.numel() != world or flags.numel() < 1 + world:
        raise RuntimeError("signal pad too small for the group")
    with _Span(tag):
        _lib.check(lib.cd_peer_barrier(flag_ptrs.data_ptr(), flags.data_ptr(), rank, world,
                                       int(limit_ms), _stream()), "cd_peer_barrier")


def moe_down_push(h_routed: torch.Tensor, wd_routed: torch.Tensor, seg_offsets: torch.Tensor,
                  num_experts: int, out_row_ptrs: torch.Tensor) -> None:
    """Routed down projection whose epilogue stores each row at its own address."""
    lib = _lib.load()
    _need(h_routed, "h_routed")
    _need(wd_routed, "routed down weights")
    _need(seg_offsets, "seg_offsets", torch.int32)
    _need(out_row_ptrs, "out_row_ptrs", torch.int64)
    T, I_e = h_routed.shape
    E, H, _ = wd_routed.shape
    if E != num_experts or out_row_ptrs.numel() != T:
        raise RuntimeError("moe_down_push: shapes do not match")
    with _Span("moe_down"):
        _lib.check(lib.cd_moe_down_push(h_routed.data_ptr(), I_e, wd_routed.data_ptr(),
                                        seg_offsets.data_ptr(), E, out_row_ptrs.data_ptr(), T, H,
                                        _stream()), "cd_moe_down_push")


def moe_combine(h_shared: torch.Tensor, wd_shared: torch.Tensor,
                routed_sorted: Optional[torch.Tensor], row_map: Optional[torch.Tensor],
                residual: Optional[torch.Tensor], residual_lo: Optional[torch.Tensor] = None,
                want_lo: bool = False):
    """Shared down projection + routed part (sorted order, from the expert GPUs) + residual.
    `residual_lo` / `want_lo` as in moe_down."""
    lib = _lib.load()
    _need(h_shared, "h_shared")
    _need(wd_shared, "shared down weight")
    T, I_s = h_shared.shape
    H = wd_shared.shape[0]
    if wd_shared.shape[1] != I_s:
        raise RuntimeError("shared down weight does not match h_shared")
    if routed_sorted is not None:
        _need(routed_sorted, "routed_sorted")
        if tuple(routed_sorted.shape) != (T, H):
            raise RuntimeError("routed_sorted does not match")
    if row_map is not None:
        _need(row_map, "row_map", torch.int32)
    res2 = None
    if residual is not None:
        res2 = residual.reshape(-1, H)
        _need(res2, "residual")
    lo2, out_lo = _split_args(res2, residual_lo, T, H, want_lo, h_shared.device)
    out = torch.empty(T, H, dtype=BF16, device=h_shared.device)
    with _Span("moe_combine"):
        _lib.check(lib.cd_moe_combine(h_shared.data_ptr(), I_s, wd_shared.data_ptr(),
                                      _ptr(routed_sorted), _ptr(row_map), _ptr(res2), _ptr(lo2),
                                      out.data_ptr(), _ptr(out_lo), T, H, _stream()),
                   "cd_moe_combine")
    return (out, out_lo) if want_lo else out


# device index -> the split-K workspace registered with the library (kept alive here; None =
# switched off by the caller)
_SPLIT_K_WS: dict = {}
_SPLIT_K_ROWS = 512          # calls of more rows never qualify (their tiles fill the SMs)
# the workspace form is opt-in (split_k(True), or CDEEP_SPLIT_K=1 for registration at first use): its
# workspace is shared by every stream of the device; the cluster form needs none and is always on
_SPLIT_K_AUTO = os.environ.get("CDEEP_SPLIT_K", "0") == "1"


def split_k(enable: bool = True, device: Optional[torch.device] = None) -> None:
    """Registers (or withdraws) the workspace that lets the few-row projections of a decode step
    cut their K loop over several CTAs (cd_splitk_workspace_set).  The workspace is shared by
    every call on the device: keep launches that may split on one stream."""
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        if enable:
            ws = torch.empty(lib.cd_splitk_workspace_bytes(), dtype=torch.uint8, device=dev)
            _lib.check(lib.cd_splitk_workspace_set(ws.data_ptr(), ws.numel(), _stream()),
                       "cd_splitk_workspace_set")
            _SPLIT_K_WS[dev.index] = ws
        else:
            _lib.check(lib.cd_splitk_workspace_set(None, 0, _stream()), "cd_splitk_workspace_set")
            torch.cuda.current_stream().synchronize()
            _SPLIT_K_WS[dev.index] = None      # stays off: the automatic registration skips this device


def split_k_config(flags: int = -1) -> int:
    """Which forms of split-K the few-row projections may take (cd_splitk_config): bit 0 the
    cluster form, bit 1 the workspace form; negative = query.  Returns the previous flags."""
    return _lib.load().cd_splitk_config(int(flags))


def _split_k_auto(x: torch.Tensor) -> None:
    # first few-row projection on a device: register the workspace (not while a graph is being
    # captured; the model's warm-up pass before the capture comes through here)
    if (_SPLIT_K_AUTO and x.shape[0] <= _SPLIT_K_ROWS and x.device.index not in _SPLIT_K_WS
            and not torch.cuda.is_current_stream_capturing()):
        split_k(True, x.device)


def mu_qkv(x: torch.Tensor, mu_prev: Optional[torch.Tensor], w: torch.Tensor,
           w_mu: Optional[torch.Tensor]) -> torch.Tensor:
    lib = _lib.load()
    _split_k_auto(x)
    _need(x, "x")
    _need(w, "qkv weight")
    T, H = x.shape
    N = w.shape[0]
    if mu_prev is not None:
        _need(mu_prev, "mu_prev")
        _need(w_mu, "mu qkv weight")
        if tuple(mu_prev.shape) != (T, H) or tuple(w_mu.shape) != (N, H):
            raise RuntimeError("mu_prev / mu weights do not match x / qkv weights")
    out = torch.empty(T, N, dtype=BF16, device=x.device)
    with _Span("mu_qkv"):
        _lib.check(lib.cd_mu_qkv(x.data_ptr(), _ptr(mu_prev), w.data_ptr(),
                                 _ptr(w_mu) if mu_prev is not None else None, out.data_ptr(), T,
                                 H, N, _stream()), "cd_mu_qkv")
    return out


def mu_qkv_rope(x: torch.Tensor, mu_prev: Optional[torch.Tensor], w: torch.Tensor,
                w_mu: Optional[torch.Tensor], q_w: Optional[torch.Tensor],
                k_w: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor, eps: float,
                seq_len: int, pos0: int, hq: int, hkv: int, head_dim: int) -> torch.Tensor:
    """The mu-guided QKV projection with Q/K RMSNorm + RoPE applied before the output is
    rounded: the fused kernel where it applies, else cd_mu_qkv followed by cd_qk_norm_rope."""
    lib = _lib.load()
    T, H = x.shape
    N = w.shape[0]
    if not lib.cd_mu_qkv_rope_supported(T, N, hq, hkv, head_dim):
        qkv = mu_qkv(x, mu_prev, w, w_mu)
        return qk_norm_rope_(qkv, q_w, k_w, cos, sin, eps, seq_len, pos0, hq, hkv, head_dim)
    _need(x, "x")
    _need(w, "qkv weight")
    _need(cos, "cos", torch.float32)
    _need(sin, "sin", torch.float32)
    if mu_prev is not None:
        _need(mu_prev, "mu_prev")
        _need(w_mu, "mu qkv weight")
        if tuple(mu_prev.shape) != (T, H) or tuple(w_mu.shape) != (N, H):
            raise RuntimeError("mu_prev / mu weights do not match x / qkv weights")
    if q_w is not None:
        _need(q_w, "q_norm.weight")
        _need(k_w, "k_norm.weight")
    if cos.shape[0] < pos0 + seq_len or cos.shape[1] != head_dim:
        raise RuntimeError("cos/sin tables too short for the requested positions")
    out = torch.empty(T, N, dtype=BF16, device=x.device)
    with _Span("mu_qkv"):
        _lib.check(lib.cd_mu_qkv_rope(
            x.data_ptr(), _ptr(mu_prev), w.data_ptr(), _ptr(w_mu) if mu_prev is not None else None,
            out.data_ptr(), T, H, N, _ptr(q_w), _ptr(k_w), cos.data_ptr(), sin.data_ptr(),
            float(eps), seq_len, pos0, hq, hkv, head_dim, _stream()), "cd_mu_qkv_rope")
    return out


def mu_proj(h: torch.Tensor, w: torch.Tensor, mu_param: torch.Tensor, mu_min: float,
            mu_max: float, out_clamp: Optional[Tuple[float, float]] = None) -> torch.Tensor:
    lib = _lib.load()
    _need(h, "hidden_states")
    _need(w, "mu_proj.weight")
    _need(mu_param, "mu")
    _split_k_auto(h)
    T, H = h.shape
    out = torch.empty(T, H, dtype=BF16, device=h.device)
    lo, hi = out_clamp if out_clamp is not None else (0.0, 0.0)
    with _Span("mu_proj"):
        _lib.check(lib.cd_mu_proj(h.data_ptr(), w.data_ptr(), mu_param.data_ptr(), float(mu_min),
                                  float(mu_max), 1 if out_clamp is not None else 0, float(lo),
                                  float(hi), out.data_ptr(), T, H, _stream()), "cd_mu_proj")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor] = None,
           tag: str = "linear", residual_lo: Optional[torch.Tensor] = None,
           want_lo: bool = False):
    """``x @ w^T (+ residual)``.  `residual_lo` / `want_lo`: split-bf16 residual stream; with
    want_lo returns (out, out_lo)."""
    lib = _lib.load()
    _need(x, "x")
    _need(w, "weight")
    _split_k_auto(x)
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise RuntimeError("weight does not match x")
    if N % 8:
        # rows of the output must stay 16-byte aligned: compute into a padded buffer against
        # zero-padded weight rows and hand back the first N columns (e.g. an lm_head whose
        # vocabulary size is not a multiple of 8)
        if residual is not None or want_lo:
            raise RuntimeError("residual with an output width that is not a multiple of 8")
        pad = 8 - N % 8
        w_pad = torch.cat([w, w.new_zeros(pad, K)], dim=0)
        return linear(x, w_pad, None, tag)[:, :N]
    if residual is not None:
        _need(residual, "residual")
        if tuple(residual.shape) != (T, N):
            raise RuntimeError("residual does not match the output")
    lo2, out_lo = _split_args(residual, residual_lo, T, N, want_lo, x.device)
    out = torch.empty(T, N, dtype=BF16, device=x.device)
    with _Span(tag):
        _lib.check(lib.cd_linear(x.data_ptr(), w.data_ptr(), _ptr(residual), _ptr(lo2),
                                 out.data_ptr(), _ptr(out_lo), T, K, N, _stream()), "cd_linear")
    return (out, out_lo) if want_lo else out
