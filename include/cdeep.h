/*
 * libcdeep — C ABI of the B200 (sm_100a) kernels for Complexity-Deep's token-routed MoE
 * layer and mu-guided attention projection.
 *
 * The reference (Complexity-ML/complexity-deep) has no FFI: the boundary it exposes is the
 * nn.Module API of complexity_deep/core and complexity_deep/models.  The Python package in
 * this repository keeps that API and calls the entry points below through ctypes; each
 * entry point names the reference code it replaces (path inside the reference project).
 *
 * Conventions
 *   - every function returns a CD_* status (0 = ok) and never throws;
 *   - all pointers are DEVICE pointers unless the name starts with h_;
 *   - activations and weights are bf16 (uint16 storage), row-major, contiguous, 16-byte
 *     aligned; ids and the routing table are int64 as in the reference; routing artefacts
 *     are int32;
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream); kernels are only
 *     enqueued, nothing synchronises except cd_status_fetch;
 *   - the library allocates no device memory on these paths: scratch is passed in.
 */
#ifndef CDEEP_H_
#define CDEEP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CD_OK 0
#define CD_ERR_INVALID 1      /* bad argument (null pointer, size or alignment rule broken) */
#define CD_ERR_CUDA 2         /* a CUDA runtime / driver call failed; see cd_last_cuda_error */
#define CD_ERR_UNSUPPORTED 3  /* shape outside what the kernels implement */
#define CD_ERR_TIMEOUT 4      /* a kernel gave up on a bounded wait (reported by cd_status_fetch) */
#define CD_ERR_BOUNDS 5       /* checking build only: an index / address / segment table read from device
                                 memory was out of range (reported by cd_status_fetch) */

/* ABI version of this header (bumped on any signature change; currently 3). */
int cd_version(void);
/* Static text for a CD_* code. */
const char* cd_error_string(int status);
/* Text of the last CUDA error seen by the calling thread's last failing call. */
const char* cd_last_cuda_error(void);
/* Largest number of row groups (experts) one grouped GEMM launch accepts; cd_moe_up,
 * cd_moe_up_pair, cd_moe_down and cd_moe_down_push return CD_ERR_UNSUPPORTED (text in
 * cd_last_cuda_error) beyond it.  The dispatch entry points accept up to 256 experts. */
int cd_max_groups(void);
/* Split-K for projections of few rows (decode; no counterpart in the reference).  A dense
 * projection whose output tiles would leave most SMs idle cuts the K loop of every tile into
 * ranges computed by different CTAs, which then combine their fp32 partial tiles and run the same
 * fused epilogue; results differ from the unsplit launch only by the order of the fp32 additions,
 * and do not depend on timing.  Two forms:
 *  - cluster form (cd_linear, cd_mu_qkv, cd_mu_proj; on by default, needs nothing from the
 *    caller): 128-wide tiles, 2 or 4 ranges per tile computed by the CTAs of one thread-block
 *    cluster, which exchange the partial tiles through distributed shared memory; each CTA
 *    finishes a slice of the tile's columns.
 *  - workspace form (also cd_moe_up with one group; up to 8 ranges): partial tiles go through a
 *    caller-provided workspace and the CTA that finishes a tile last adds them.  Off until a
 *    workspace is registered for the current device; cd_splitk_workspace_bytes() is a size that
 *    suits every eligible call.  The workspace is shared by all calls on the device: launches
 *    that may use it must be ordered on one stream (or by events), and the memory must stay valid
 *    until cd_splitk_workspace_set(NULL, 0, stream) or the last launch has finished.  `stream`
 *    orders the clearing of the workspace's counters.
 * cd_splitk_config(flags) chooses the forms a launch may take (bit 0 cluster, bit 1 workspace;
 * default 3; a negative argument only queries) and returns the previous flags. */
int cd_splitk_config(int flags);
size_t cd_splitk_workspace_bytes(void);
int cd_splitk_workspace_set(void* workspace, size_t bytes, void* stream);
/* Number of K ranges cd_linear (or cd_mu_proj; cd_mu_qkv with K = the sum of its two K extents)
 * would use for a [T, K] x [N, K]^T call on the current device as it is set up now (1 = unsplit). */
int cd_splitk_ranges(int T, int K, int N);
/* 1 when this library is the checking build (libcdeep_checks.so, compiled with -DCDEEP_CHECKS),
 * else 0.  The checking build validates what its kernels read from device memory before using it
 * as an index or address — row_map of cd_moe_down / cd_moe_combine (entries in [0, T)), dst_rows of
 * cd_rmsnorm / cd_rmsnorm_split and src_rows of cd_gather_rows (in [0, T)), out_row_ptrs of
 * cd_moe_down_push (non-null, 16-byte aligned), seg_offsets of every grouped call
 * (0 <= s[0] <= ... <= s[G] <= T) — and, on a violation, skips the access (a bad segment table:
 * the whole launch) and raises the status word to 4.  It is the stand-in for a memory checker on
 * machines where none may run; the normal build trusts its caller. */
int cd_checks_enabled(void);
/* Synchronises the current device, copies the kernels' status word to *h_status and clears it.
 * 0 = nothing to report; 1 = a bounded pipeline wait ran out; 2 = cd_peer_barrier ran out;
 * 4 = the checking build met an index out of range (the largest value seen is kept). */
int cd_status_fetch(int* h_status);

/* Self-test of the kernels' failure detection (no counterpart in the reference).  Every wait of
 * the GEMM pipeline is bounded; this launches one 128 x 128 x 64 tile whose loader is switched
 * off, with the limit set to limit_ms (1..1000): the kernel must give up, free its resources and
 * return, after which cd_status_fetch reports 1 and the device remains usable.  Nothing faults,
 * traps or spins forever.  a, b: [128, 64] bf16, out: [128, 128] bf16 (contents unspecified). */
int cd_selftest_wait_timeout(const void* a, const void* b, void* out, int limit_ms, void* stream);

/* ---- dispatch -------------------------------------------------------------------------
 * Replaces TokenRoutedMLP.forward's lookup and mask loop,
 * complexity_deep/core/token_routed_mlp.py:149-150 (clamp + table lookup) and :166-170,
 * :174 (per-expert boolean mask, gather, scatter).  Outputs, all bit-exact with what the
 * mask loop implies:
 *   expert_ids[T]  table[clamp(ids, 0, V-1)]
 *   counts[E]      tokens per expert
 *   offsets[E+1]   exclusive prefix sum of counts
 *   perm[T]        sorted position -> source row (rows of expert e in ascending row order)
 *   inv_perm[T]    source row -> sorted position
 * ws: scratch of at least cd_route_workspace_bytes(T, E) bytes.  E <= 256. */
size_t cd_route_workspace_bytes(int T, int E);
int cd_route(const int64_t* ids, const int64_t* table, int V, int E, int T, int32_t* expert_ids,
             int32_t* counts, int32_t* offsets, int32_t* perm, int32_t* inv_perm, void* ws,
             size_t ws_bytes, void* stream);

/* ---- dispatch for callers that cannot allocate ---------------------------------------------
 * (No counterpart in the reference.)  Same computation and outputs as cd_route, but the
 * scratch is a fixed 512 KiB array inside the library instead of a caller buffer, and the
 * call allocates nothing — no cudaMalloc/cudaFree, no allocating library routine.  Meant for
 * hosts that must not touch a device allocator where they route a batch: a serving loop
 * pinned to a fixed memory budget, or a framework plugin that is handed only input and
 * output buffers.
 *   - Limit: ceil(T / 2048) * E <= 131072; cd_route_static_max_tokens(E) gives the largest T.
 *     Larger requests return CD_ERR_UNSUPPORTED (text in cd_last_cuda_error) — use cd_route.
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array.  It keeps the previous call's contents, which
 *     is harmless (each call overwrites every slot it later reads), but two calls whose
 *     kernels overlap on the GPU (different streams, no ordering) race on it: order them.
 *   - Every GPU that loads the library holds the array until the process exits. */
int cd_route_static_max_tokens(int E);
int cd_route_static(const int64_t* ids, const int64_t* table, int V, int E, int T,
                    int32_t* expert_ids, int32_t* counts, int32_t* offsets, int32_t* perm,
                    int32_t* inv_perm, void* stream);

/* ---- RMSNorm ---------------------------------------------------------------------------
 * Replaces RMSNorm.forward, complexity_deep/core/normalization.py:29-32, optionally fused
 * with the residual add in front of it (complexity_deep/core/layer.py:174) and with the
 * scatter of rows into expert-sorted order behind it (the gather of
 * token_routed_mlp.py:170).
 *   h = x (+ residual, rounded to bf16);  sum_out = h (if non-null)
 *   out[dst_rows ? dst_rows[i] : i, :] = weight * h[i] * rsqrt(mean(h[i]^2) + eps)
 * residual, sum_out, dst_rows may be NULL.  sum_out is only written together with a residual
 * (without one h is x itself) and must not alias x: both cases return CD_ERR_INVALID. */
int cd_rmsnorm(const void* x, const void* residual, const void* weight, float eps, void* sum_out,
               void* out, const int32_t* dst_rows, int T, int H, void* stream);

/* RMSNorm of a split-bf16 residual stream.  Between the kernels of a block the residual stream
 * (complexity_deep/core/layer.py:174, :183) is carried as two bf16 tensors, hi = bf16(v) and
 * lo = bf16(v - hi) — 16 significant bits, so the 2 * num_layers additions into the stream do
 * not each cost a bf16 rounding of the whole stream (what keeps the logits of an 18-layer
 * model inside mean |err| <= 2e-3 of the fp32 reference):
 *   h = x_hi + x_lo in fp32 (x_lo may be NULL = 0);  out as in cd_rmsnorm. */
int cd_rmsnorm_split(const void* x_hi, const void* x_lo, const void* weight, float eps, void* out,
                     const int32_t* dst_rows, int T, int H, void* stream);

/* out[j, :] = x[src_rows[j], :] — the gather `flat_x[mask]` of token_routed_mlp.py:170 for
 * all experts at once, used when the MoE layer is called without the fused norm. */
int cd_gather_rows(const void* x, const int32_t* src_rows, void* out, int T, int H, void* stream);

/* ---- Q/K RMSNorm + rotary embedding, in place -------------------------------------------
 * Replaces complexity_deep/core/attention.py:138-155 (q_norm/k_norm, cos/sin slicing,
 * apply_rotary_pos_emb of complexity_deep/core/rotary.py:64-86) on the fused
 * [T, (hq + 2*hkv) * D] projection buffer; the V columns are left untouched.  Token t sits
 * at position pos0 + (t % S).  q_w / k_w ([D] bf16) may both be NULL (use_qk_norm=False).
 * cos_t / sin_t are fp32 [>= pos0 + S, D].  D % 4 == 0. */
int cd_qk_norm_rope(void* qkv, const void* q_w, const void* k_w, const float* cos_t,
                    const float* sin_t, float eps, int T, int S, int pos0, int hq, int hkv, int D,
                    void* stream);

/* ---- decode step: Q/K RMSNorm + rotary embedding + KV-cache append --------------------------
 * One new token per sequence (row b of qkv belongs to sequence b).  cd_qk_norm_rope's
 * arithmetic at the position stored in DEVICE memory (*pos_dev, the number of tokens already
 * cached), and the rotated k heads and the v heads of every row are also written into the
 * caches at that position: k_cache[b, h, *pos_dev, :], same for v (element strides batch / kv
 * head / token, D contiguous, multiples of 8).  Replaces complexity_deep/core/attention.py:138-161
 * for q_len == 1: the reference grows the cache with torch.cat, which copies all of it every
 * step; here the cache is a fixed buffer of `capacity` tokens and the position is a device
 * scalar, so the same launch (same arguments) serves every step and can be replayed from a
 * CUDA graph.  Nothing is written when *pos_dev is outside [0, capacity); cos_t / sin_t hold
 * `capacity` rows. */
int cd_decode_rope_append(void* qkv, const void* q_w, const void* k_w, const float* cos_t,
                          const float* sin_t, float eps, int B, int hq, int hkv, int D,
                          void* k_cache, void* v_cache, long long kv_stride_b,
                          long long kv_stride_h, long long kv_stride_t, int capacity,
                          const int32_t* pos_dev, void* stream);

/* ---- single-query attention over a KV cache (decode) ---------------------------------------
 * Replaces, for q_len == 1, complexity_deep/core/attention.py:163-177 (repeat_interleave of the
 * KV heads + scaled_dot_product_attention with an additive mask):
 *   out[b, h, :] = softmax(scale * q[b, h] . K[b, h / G]^T + mask[b]) V[b, h / G],  G = hq / hkv
 * q: row b at q + b * q_stride_b, heads contiguous [hq, D] (the q columns of the fused
 * projection buffer).  k, v: element strides (batch, kv head, token), D contiguous — the
 * cache is read in place, whatever buffer it lives in.  mask: bf16 additive [B, L] with row
 * stride mask_stride_b (0 = one row for all), or NULL.  out: [B, hq * D] bf16.
 * ws: cd_decode_attention_workspace_bytes(...) bytes.  D is 64 or 128, G <= 4; all strides
 * multiples of 8 elements.  kv_len_dev (may be NULL): a device scalar; when given, only the
 * first min(L, *kv_len_dev) cached tokens are attended (L then is the capacity the launch is
 * sized for), with the same split of the rows over blocks, hence the same bits, as a call
 * with that L. */
size_t cd_decode_attention_workspace_bytes(int B, int hq, int hkv, int L, int D);
int cd_decode_attention(const void* q, long long q_stride_b, const void* k, const void* v,
                        long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                        const void* mask, long long mask_stride_b, float scale, int B, int hq,
                        int hkv, int L, const int32_t* kv_len_dev, int D, void* out, void* ws,
                        size_t ws_bytes, void* stream);

/* ---- causal self-attention over a prompt (prefill) --------------------------------------------
 * Replaces, for a prompt without cached keys and without an additive mask,
 * complexity_deep/core/attention.py:163-177 (repeat_interleave of the KV heads +
 * scaled_dot_product_attention(is_causal=True)); the reference's Triton analogue is
 * complexity_deep/cuda/fused_attention.py:121-233.
 *   out[b*S + s, h*D : (h+1)*D] = softmax_{t <= s}(scale * q[b,s,h] . k[b,t,h/G]) v[b,t,h/G],  G = hq / hkv
 * qkv: [B * S, (hq + 2*hkv) * D] — the fused projection buffer after Q/K norm + RoPE (q heads,
 * then k heads, then v heads along a row); q, k, v are read in place from its column slices and
 * grouped KV heads are never copied.  out: [B * S, hq * D] (the operand of o_proj).  Any S
 * (ragged last tiles are masked); D is 64 or 128; hq % hkv == 0.  QK^T and PV run on tcgen05
 * with the scores, probabilities and the output accumulator in tensor memory.
 * cd_attention_prefill_supported returns 1 for shapes the kernel takes. */
int cd_attention_prefill_supported(int B, int S, int hq, int hkv, int D);
int cd_attention_prefill(const void* qkv, void* out, int B, int S, int hq, int hkv, int D,
                         float scale, void* stream);

/* ---- expert up-projection with fused SwiGLU ---------------------------------------------
 * Replaces gate/up GEMMs and silu(gate)*up of the routed experts
 * (token_routed_mlp.py:171-173) or, with num_groups = 1 and seg_offsets = NULL, of the
 * shared expert (:157-160) / the dense SwiGLU (complexity_deep/core/mlp.py:40).
 *   h[r, :I] = silu(x[r] @ Wg[g]) * (x[r] @ Wu[g])   for rows r of group g
 * x_sorted: [T, H] rows grouped by expert (seg_offsets[g] .. seg_offsets[g+1]).
 * packed_w: [num_groups, cd_gate_up_packed_rows(I, block_n), H] — per group, for each tile
 *   of block_n/2 output columns, block_n/2 gate rows followed by block_n/2 up rows (each
 *   row = one output feature, H contiguous), zero rows padding the last tile.
 * h: [T, I].  block_n is 32, 64, 128 or 256 (narrow tiles for few rows: more CTAs share the
 * weight stream).  H % 8 == 0, I % 8 == 0. */
int cd_gate_up_packed_rows(int I, int block_n);
int cd_moe_up(const void* x_sorted, const int32_t* seg_offsets, int num_groups,
              const void* packed_w, void* h, int T, int H, int I, int block_n, void* stream);

/* Routed AND shared up-projections in ONE launch (token_routed_mlp.py:171-173 and :157-160):
 * cd_moe_up over the groups, followed in the same persistent tile schedule by the dense
 * product of the same T rows against the shared expert's packed gate/up rows
 * (packed_shared: [cd_gate_up_packed_rows(I_s, block_n), H]) into h_shared [T, I_s].  One launch
 * has one tail instead of two, which matters when a GPU holds few rows (small data-parallel
 * shards).  Both weight sets are packed for the same block_n. */
int cd_moe_up_pair(const void* x_sorted, const int32_t* seg_offsets, int num_groups,
                   const void* packed_w, void* h, int I, const void* packed_shared, void* h_shared,
                   int I_s, int T, int H, int block_n, void* stream);

/* ---- one-off weight layout transforms ------------------------------------------------------
 * What a host has to do once per weight version to get from the reference's parameter layouts
 * (token_routed_mlp.py:62-77) to the operands of the entry points above; outputs go to
 * caller-owned buffers.
 * cd_pack_gate_up: packed [G, cd_gate_up_packed_rows(I, block_n), H] from gate and up.
 *   feature_major = 0: gate / up are [G, H, I] (gate_proj_w / up_proj_w, used as x @ W[e]);
 *   feature_major = 1: gate / up are [G, I, H] (nn.Linear weights, G = 1 for the shared expert).
 * cd_pack_down: packed [E, H, I] from down_proj_w [E, I, H] (the wd_routed operand of
 *   cd_moe_down).  The shared expert's down weight [H, I_s] is used as it is. */
int cd_pack_gate_up(const void* gate, const void* up, void* packed, int G, int I, int H,
                    int block_n, int feature_major, void* stream);
int cd_pack_down(const void* down, void* packed, int E, int I, int H, void* stream);

/* ---- expert down-projection, combine, un-permute, residual -------------------------------
 * Replaces the routed down GEMM and scatter (token_routed_mlp.py:174), the shared down GEMM
 * (:157-160), `routed_out + shared_out` (:177) and the block's residual add
 * (complexity_deep/core/layer.py:183) with ONE fp32 accumulation per output element:
 *   out[row_map[r], :] = h_routed[r] @ Wd[g]^T + h_shared[r] @ Sd^T + residual[row_map[r], :]
 * h_routed [T, I_e], h_shared [T, I_s] (NULL = no shared expert), rows in sorted order;
 * wd_routed [E * H, I_e] (for expert e rows e*H..: one output feature per row, I_e
 * contiguous); wd_shared [H, I_s]; row_map = perm (NULL = identity); residual (NULL = none)
 * and out are [T, H] in ORIGINAL row order.  I_e % 8 == 0, I_s % 8 == 0, H % 8 == 0.
 * Split-bf16 residual stream (see cd_rmsnorm_split): residual_lo (NULL = 0, needs residual) is
 * the low part of the residual and is added too; with out_lo non-NULL the fp32 result v is
 * stored as out = bf16(v), out_lo = bf16(v - out).  Both are indexed like residual / out. */
int cd_moe_down(const void* h_routed, int I_e, const void* wd_routed, const void* h_shared,
                int I_s, const void* wd_shared, const int32_t* seg_offsets, int E,
                const int32_t* row_map, const void* residual, const void* residual_lo, void* out,
                void* out_lo, int T, int H, void* stream);

/* ---- expert-parallel combine ---------------------------------------------------------------
 * Home-GPU half of the layer when the routed experts live on other GPUs: the shared expert's
 * down projection (token_routed_mlp.py:157-160) plus `routed_out + shared_out` (:177) and the
 * block's residual add (complexity_deep/core/layer.py:183), where the routed part arrives
 * from the expert GPUs (already down-projected there with cd_moe_down, h_shared = NULL):
 *   out[row_map[r], :] = h_shared[r] @ Sd^T + routed_sorted[r, :] + residual[row_map[r], :]
 * h_shared [T, I_s] and routed_sorted [T, H] in sorted order (routed_sorted may be NULL);
 * row_map / residual / residual_lo / out_lo as in cd_moe_down. */
int cd_moe_combine(const void* h_shared, int I_s, const void* wd_shared, const void* routed_sorted,
                   const int32_t* row_map, const void* residual, const void* residual_lo, void* out,
                   void* out_lo, int T, int H, void* stream);

/* ---- expert-parallel exchange by peer stores --------------------------------------------------
 * (The reference has no distributed code; the entry points of this section replace the NCCL
 * all-to-alls of the expert-parallel layer with stores into peer-mapped memory, issued by the
 * kernels that produce the rows.  The caller provides peer-mapped buffers, e.g. CUDA IPC or symmetric
 * memory, and orders the phases with a barrier across the GPUs.)
 *
 * cd_peer_put_i32: copies n int32 from src to element offset `offset` of the buffer of EVERY
 * rank (peer_bufs: device array of the world buffers' addresses as seen from this GPU).  With
 * offset = rank * n, followed by cd_peer_barrier, it is an all-gather of a small table (the
 * counts of cd_route) without a collective library call.
 *
 * cd_ep_plan: the exchange plan of a routed batch in one launch, from the count matrix of all
 * ranks (counts[g * num_experts + e] = rows of expert e among rank g's tokens; one all-gather of
 * cd_route's counts).  Receive buffers are laid out expert-major, source-minor.  Outputs for THIS
 * rank: push_base[num_experts] (see cd_push_rows), seg_offsets[experts_per_rank + 1] (segments of
 * this rank's receive buffer, the seg_offsets of cd_moe_up / cd_moe_down_push) and
 * row_ptrs[capacity] (out_row_ptrs of cd_moe_down_push: for received row r the address
 * ret_ptrs[home] + (home's sorted offset of the row) * row_bytes in its home rank's return buffer;
 * entries past the received rows are never used).  world * experts_per_rank == num_experts,
 * world * num_experts <= 8192.
 *
 * cd_push_rows: sorted row j (= x[src_rows[j]], or x[j] when src_rows is NULL) of expert e
 * (offsets[e] <= j < offsets[e+1]) is written to row push_base[e] + (j - offsets[e]) of the
 * buffer whose address is peer_ptrs[e / experts_per_rank] (device array of E /
 * experts_per_rank addresses).
 *
 * cd_moe_down_push: the routed down projection of cd_moe_down (no shared expert, no residual)
 * whose epilogue writes sorted row r to the ADDRESS out_row_ptrs[r] (device array, one per row;
 * rows may live in another GPU's memory), so each finished tile leaves for its home GPU while
 * the next one is being computed.
 *
 * cd_peer_barrier: the barrier between the phases.  Every GPU of the group owns a signal pad of
 * 1 + world int32 (zero-initialised, peer-mapped); peer_flags is a device array of the world
 * pads' addresses as seen from this GPU, flags this GPU's own pad.  The kernel (one block)
 * advances this GPU's barrier count in flags[0], announces it in every pad and waits until every
 * GPU has announced the same count.  All stores issued on this GPU before the barrier are then
 * visible to the kernels the other GPUs launch after theirs.  The wait gives up after limit_ms
 * (1..60000): the status word is raised (cd_status_fetch reports it) and the kernel returns, so a
 * GPU that left the group cannot leave the others spinning.  All GPUs must call it the same
 * number of times; the launch arguments never change, so it can be captured in a CUDA graph. */
int cd_peer_barrier(const uint64_t* peer_flags, int32_t* flags, int rank, int world, int limit_ms,
                    void* stream);
int cd_peer_put_i32(const int32_t* src, int n, const uint64_t* peer_bufs, int world, int64_t offset,
                    void* stream);
int cd_ep_plan(const int32_t* counts, int world, int num_experts, int experts_per_rank, int rank,
               const int64_t* ret_ptrs, int64_t row_bytes, int capacity, int32_t* push_base,
               int32_t* seg_offsets, int64_t* row_ptrs, void* stream);
int cd_push_rows(const void* x, const int32_t* src_rows, const int32_t* offsets,
                 const int32_t* push_base, int E, int experts_per_rank, const uint64_t* peer_ptrs,
                 int T, int H, void* stream);
int cd_moe_down_push(const void* h_routed, int I_e, const void* wd_routed,
                     const int32_t* seg_offsets, int E, const int64_t* out_row_ptrs, int T, int H,
                     void* stream);

/* ---- mu-guided QKV -------------------------------------------------------------------------
 * Replaces complexity_deep/core/attention.py:120-131: torch.cat([x, mu_prev]) against the
 * re-concatenated weights, three F.linear calls.  One GEMM whose K loop walks x then
 * mu_prev; nothing is concatenated in memory:
 *   qkv[t, :N] = x[t] @ w^T + mu_prev[t] @ w_mu^T,   N = q_dim + 2 * kv_dim
 * w, w_mu: [N, H] = rows of q_proj, k_proj, v_proj (resp. mu_to_q, mu_to_k, mu_to_v) stacked.
 * mu_prev / w_mu may be NULL (no mu guidance: plain q/k/v projections). */
int cd_mu_qkv(const void* x, const void* mu_prev, const void* w, const void* w_mu, void* qkv,
              int T, int H, int N, void* stream);

/* ---- mu-guided QKV with Q/K RMSNorm + rotary embedding in the epilogue ---------------------
 * cd_mu_qkv followed by cd_qk_norm_rope, in one kernel: the norm and the rotation are applied
 * to the fp32 accumulators before the single bf16 rounding (replaces
 * complexity_deep/core/attention.py:120-131 and :138-155).  Arguments as in those two entry
 * points.  Only for head size 128 with q and k column ranges that are multiples of 256 and
 * enough rows for 256-wide tiles: cd_mu_qkv_rope_supported(...) returns 1 when the fused
 * kernel applies, otherwise call the two entry points one after the other. */
int cd_mu_qkv_rope_supported(int T, int N, int hq, int hkv, int D);
int cd_mu_qkv_rope(const void* x, const void* mu_prev, const void* w, const void* w_mu, void* qkv,
                   int T, int H, int N, const void* q_w, const void* k_w, const float* cos_t,
                   const float* sin_t, float eps, int S, int pos0, int hq, int hkv, int D,
                   void* stream);

/* ---- mu projection ------------------------------------------------------------------------
 * Replaces MuGuidance.forward, complexity_deep/core/layer.py:54-61, and optionally the
 * model's clamp of the result, complexity_deep/models/modeling.py:199-200:
 *   out[t, n] = clamp(mu_param[n], mu_min, mu_max) + h[t] @ w[n]      (w = mu_proj.weight [H, H])
 *   if clamp_out: out = clamp(out, out_lo, out_hi) */
int cd_mu_proj(const void* h, const void* w, const void* mu_param, float mu_min, float mu_max,
               int clamp_out, float out_lo, float out_hi, void* out, int T, int H, void* stream);

/* ---- plain projection with optional residual ---------------------------------------------
 * out[t, :N] = x[t, :K] @ w^T (+ residual[t, :N]);  w = nn.Linear weight [N, K].
 * Replaces o_proj + residual (complexity_deep/core/attention.py:181 with layer.py:174) and
 * lm_head (complexity_deep/models/modeling.py:206).  K % 8 == 0, N % 8 == 0.
 * residual_lo / out_lo: split-bf16 residual stream as in cd_moe_down (both may be NULL). */
int cd_linear(const void* x, const void* w, const void* residual, const void* residual_lo,
              void* out, void* out_lo, int T, int K, int N, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CDEEP_H_ */
