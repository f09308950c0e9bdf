// Causal self-attention for prefill on sm_100a: S = Q K^T and O = P V on the tcgen05 tensor
// cores with S / P / O in tensor memory, online softmax in dedicated warps, K / V tiles fed by
// TMA (never with cluster multicast), grouped-query heads without materialising repeated KV.
//
// Replaces, for a prompt without cached keys and without an additive mask,
// complexity_deep/core/attention.py:163-177 of the reference (repeat_interleave of the KV
// heads + scaled_dot_product_attention(is_causal=True)); the reference's Triton analogue is
// complexity_deep/cuda/fused_attention.py:121-233.  q, k, v are read in place as column
// slices of the fused projection buffer [T, (hq + 2 hkv) * D] (token-major, T = B * S) and
// the result is written as [T, hq * D], the operand layout of o_proj.
//
// Work decomposition: a work item is (sequence, query head, pair of 128-row query tiles); one
// persistent CTA per SM loops over items (heavy pairs first), keeping its TMEM allocation and
// barriers, so the loads and first products of the next item overlap the epilogue of the
// current one.  The two query tiles A and B of an item share the K / V tiles in shared memory
// and take turns on the tensor pipe: while the softmax warps of A work on their 128 x 128
// scores, the MMA warp issues B's products, and vice versa.
//
//   warps 0-3   softmax of tile A (a thread owns one query row = one TMEM lane)
//   warps 4-7   softmax of tile B
//   warp  8     TMA producer (Q once, then the K / V ring)
//   warp  9     MMA issuer + TMEM owner
//
// Per KV tile j and query tile X:  S_X = Q_X K_j^T  (accumulator in TMEM, 128 columns)
//   -> softmax warps: row max, p = exp2(scale * (s - m)), row sum; P (bf16) is written back
//      into the first 64 columns of S_X
//   -> O_X += P_X V_j  (A operand = P from TMEM, B operand = the V tile, N-major)
// The running maximum m is only raised when it grew by more than 2^8 in the exp2 domain
// (then O and the row sum are rescaled in TMEM); otherwise the stale maximum is kept, which
// is exact as long as the final division uses the matching row sum.
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "../../include/cdeep.h"
#include "kernels.h"
#include "ptx.cuh"

namespace cdeep {

namespace {

constexpr int kQTile = 128;      // query rows per tile = TMEM lanes
constexpr int kKvTile = 128;     // keys per tile
constexpr int kAttnThreads = 320;
constexpr float kRescaleThreshold = 8.0f;   // log2 of the growth of the maximum that forces a rescale

struct AttnParams {
  int S;            // sequence length
  int hq, hkv;      // query / kv heads
  int q_tiles;      // ceil(S / 128)
  int pairs;        // ceil(q_tiles / 2)
  int batch;        // sequences
  float scale_log2; // softmax scale * log2(e)
  __nv_bfloat16* out;   // [T, hq * D]
  int ldo;
  unsigned long long wait_limit_ns;
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int kBoxBytes = 128 * 64 * 2;           // one TMA box: 128 rows x 64 columns
  static constexpr int kTileBytes = (D / 64) * kBoxBytes;  // a Q, K or V tile
  static constexpr int kQOff = 0;                          // Q_A, Q_B
  static constexpr int kKOff = 2 * kTileBytes;             // K ring (2 stages)
  static constexpr int kVOff = 4 * kTileBytes;             // V ring (2 stages)
  static constexpr int kBarOff = 6 * kTileBytes;
  static constexpr int kNumBars = 2 + 8 + 8;               // q_full/q_empty, k/v full/empty x2, s_full/p_full/o_done/o_free x2
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap tm_qkv, const AttnParams p) {
  using L = AttnSmem<D>;
  constexpr int kDBlocks = D / 64;                 // 64-column boxes per tile
  constexpr uint32_t kTmemCols = 512;   // S_A, S_B (128 columns each), O_A, O_B (D each)
  auto s_col = [](int x) { return static_cast<uint32_t>(x * 128); };
  auto o_col = [](int x) { return static_cast<uint32_t>(256 + x * D); };

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2] per query tile
  uint64_t* p_full = bars + 11;       // [2]
  uint64_t* o_done = bars + 13;       // [2]
  uint64_t* o_free = bars + 15;       // [2]
  uint64_t* q_empty = bars + 17;      // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t wait_limit = p.wait_limit_ns ? p.wait_limit_ns : kWaitLimitNs;

  // Work items = (pair of query tiles, head, sequence), numbered heavy pairs first (late rows see
  // the most keys); this CTA takes items blockIdx.x, blockIdx.x + gridDim.x, ...  TMEM, barriers
  // and their phase counters live across items, so the loads and first products of item i + 1
  // run under the softmax tail and the epilogue of item i.
  const int per_pair = p.hq * p.batch;
  const int total_items = p.pairs * per_pair;
  struct Item {
    int pair, head, batch, kv_head, n_a, n_b, n_max, q_col, k_col, v_col;
    long long row0;
  };
  auto decode_item = [&](int item) {
    Item w;
    w.pair = p.pairs - 1 - item / per_pair;
    const int rem = item % per_pair;
    w.head = rem % p.hq;
    w.batch = rem / p.hq;
    w.kv_head = w.head / (p.hq / p.hkv);
    // query tiles 2 * pair (A) and 2 * pair + 1 (B); tile t sees KV tiles 0 .. t
    w.n_a = 2 * w.pair + 1;
    w.n_b = (2 * w.pair + 1 < p.q_tiles) ? 2 * w.pair + 2 : 0;     // 0: B does not exist
    w.n_max = w.n_b > w.n_a ? w.n_b : w.n_a;
    w.row0 = static_cast<long long>(w.batch) * p.S;
    w.q_col = w.head * D;
    w.k_col = (p.hq + w.kv_head) * D;
    w.v_col = (p.hq + p.hkv + w.kv_head) * D;
    return w;
  };

  if (warp == 8 && lane == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);     // one arrival per softmax warp of the tile
      mbar_init(&o_done[s], 1);
      mbar_init(&o_free[s], 4);     // the tile's softmax warps have read O of the finished item
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_qkv);
  } else if (warp == 9) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  griddep_wait();
  griddep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      uint32_t kv = 0;     // K / V tiles loaded so far (ring position)
      uint32_t it = 0;     // items started by this CTA
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
        const Item w = decode_item(item);
        // Q may be overwritten once every S product of the previous item has read it
        if (it > 0 && !mbar_wait(q_empty, (it - 1) & 1u, abort_flag, wait_limit)) { ok = false; break; }
        const int q_tiles_here = w.n_b > 0 ? 2 : 1;
        mbar_arrive_expect_tx(q_full, q_tiles_here * L::kTileBytes);
        for (int x = 0; x < q_tiles_here; ++x)
          for (int d = 0; d < kDBlocks; ++d)
            tma_load_2d(smem + L::kQOff + x * L::kTileBytes + d * L::kBoxBytes, &tm_qkv, q_full,
                        w.q_col + d * 64, static_cast<int>(w.row0) + (2 * w.pair + x) * kQTile);
        for (int j = 0; j < w.n_max && ok; ++j, ++kv) {
          const int s = kv & 1;
          const uint32_t ph = (kv >> 1) & 1u;
          const int kv_row = static_cast<int>(w.row0) + j * kKvTile;
          if (!mbar_wait(&k_empty[s], ph ^ 1u, abort_flag, wait_limit)) { ok = false; break; }
          mbar_arrive_expect_tx(&k_full[s], L::kTileBytes);
          for (int d = 0; d < kDBlocks; ++d)
            tma_load_2d(smem + L::kKOff + s * L::kTileBytes + d * L::kBoxBytes, &tm_qkv, &k_full[s],
                        w.k_col + d * 64, kv_row);
          if (!mbar_wait(&v_empty[s], ph ^ 1u, abort_flag, wait_limit)) { ok = false; break; }
          mbar_arrive_expect_tx(&v_full[s], L::kTileBytes);
          for (int d = 0; d < kDBlocks; ++d)
            tma_load_2d(smem + L::kVOff + s * L::kTileBytes + d * L::kBoxBytes, &tm_qkv, &v_full[s],
                        w.v_col + d * 64, kv_row);
        }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kQTile, kKvTile);         // S = Q K^T
      constexpr uint32_t idesc_o = make_idesc_bf16(kQTile, D, true);         // O = P V (V N-major)
      const uint32_t q_addr = smem_u32(smem + L::kQOff);
      const uint32_t k_addr = smem_u32(smem + L::kKOff);
      const uint32_t v_addr = smem_u32(smem + L::kVOff);
      bool ok = true;
      uint32_t kv = 0;               // ring position of the item's first K / V tile
      uint32_t it = 0;               // items started
      uint32_t cnt[2] = {0, 0};      // tiles of A / B finished in earlier items (barrier phases)
      uint32_t items_x[2] = {0, 0};  // earlier items in which A / B existed (o_free phases)
      // S_X = Q_X K^T for the K tile in ring stage `stage`: D / 16 MMAs over the 64-column boxes
      auto issue_s = [&](int x, int stage) {
        const uint32_t qa = q_addr + x * L::kTileBytes;
        const uint32_t ka = k_addr + stage * L::kTileBytes;
#pragma unroll
        for (int d = 0; d < kDBlocks; ++d) {
          const uint64_t da = make_smem_desc_sw128(qa + d * L::kBoxBytes);
          const uint64_t db = make_smem_desc_sw128(ka + d * L::kBoxBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + s_col(x), da + 2u * k, db + 2u * k, idesc_s, (d | k) != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[x]);
      };
      // O_X (+)= P_X V: 8 MMAs of 16 keys; P sits in the first 64 columns of S_X (two bf16 per
      // column), the V tile is read N-major: 16 key rows = 2048 bytes further per step
      auto issue_pv = [&](int x, int stage, bool first) {
        const uint64_t db0 = make_smem_desc_mn_sw128(v_addr + stage * L::kTileBytes, L::kBoxBytes);
        const uint32_t acc0 = first ? 0u : 1u;
#pragma unroll
        for (int k = 0; k < kKvTile / 16; ++k)
          umma_bf16_tmem_a(tmem_base + o_col(x), tmem_base + s_col(x) + 8u * k, db0 + k * 128u, idesc_o,
                           k != 0 ? 1u : acc0);
      };
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++it) {
        const Item w = decode_item(item);
        const int n_of[2] = {w.n_a, w.n_b};
        int s_left = w.n_a + w.n_b;     // S products of this item still to issue (then Q is free)
        if (!mbar_wait(q_full, it & 1u, abort_flag, wait_limit)) { ok = false; break; }
        if (!mbar_wait(&k_full[kv & 1], (kv >> 1) & 1u, abort_flag, wait_limit)) { ok = false; break; }
        tc_fence_after();
        issue_s(0, kv & 1);
        --s_left;
        if (w.n_b > 0) { issue_s(1, kv & 1); --s_left; }
        umma_commit(&k_empty[kv & 1]);   // K_0 is free once both first products have read it
        if (s_left == 0) umma_commit(q_empty);
        for (int j = 0; j < w.n_max && ok; ++j) {
          const uint32_t g = kv + j;                 // ring position of K_j / V_j
          const int s = g & 1;
          const uint32_t ph = (g >> 1) & 1u;
          for (int x = 0; x < 2 && ok; ++x) {
            if (j >= n_of[x]) continue;
            const bool last_user = (x == 1) || (j >= w.n_b);   // of V_j among the two tiles
            if (!mbar_wait(&p_full[x], (cnt[x] + j) & 1u, abort_flag, wait_limit)) { ok = false; break; }
            if (x == 0 || j >= w.n_a) {   // first PV of this KV tile: V_j must have landed
              if (!mbar_wait(&v_full[s], ph, abort_flag, wait_limit)) { ok = false; break; }
            }
            if (j == 0 && items_x[x] > 0) {   // O_X of the previous item must have been read out
              if (!mbar_wait(&o_free[x], (items_x[x] - 1) & 1u, abort_flag, wait_limit)) { ok = false; break; }
            }
            tc_fence_after();
            issue_pv(x, s, j == 0);
            if (last_user) umma_commit(&v_empty[s]);
            umma_commit(&o_done[x]);
            if (j + 1 < n_of[x]) {
              const uint32_t g1 = g + 1;
              const int s1 = g1 & 1;
              if (x == 0 || j + 1 >= w.n_a) {   // first S of the next KV tile: K_{j+1} must have landed
                if (!mbar_wait(&k_full[s1], (g1 >> 1) & 1u, abort_flag, wait_limit)) { ok = false; break; }
                tc_fence_after();
              }
              issue_s(x, s1);
              // K_{j+1} is free once the last tile that uses it has issued its S
              if (x == 1 || j + 1 >= w.n_b) umma_commit(&k_empty[s1]);
              if (--s_left == 0) umma_commit(q_empty);
            }
          }
        }
        kv += w.n_max;
        for (int x = 0; x < 2; ++x) {
          cnt[x] += n_of[x];
          items_x[x] += n_of[x] > 0 ? 1u : 0u;
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int x = warp >> 2;                 // query tile of this warp group
    const int quarter = warp & 3;            // TMEM lane quarter this warp may access
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_addr + s_col(x);
    const uint32_t o_tmem = tmem_base + lane_addr + o_col(x);
    uint32_t cnt = 0;                        // tiles of this query-tile slot finished in earlier items
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const Item w = decode_item(item);
      const int n_mine = x ? w.n_b : w.n_a;
      if (n_mine == 0) continue;             // the sequence has an odd number of tiles: no tile B here
      const int q_pos = (2 * w.pair + x) * kQTile + quarter * 32 + lane;   // position of this thread's row
      float m_ref = -INFINITY;               // maximum the stored exponentials refer to (raw scores)
      float l_sum = 0.f;
      for (int j = 0; j < n_mine && ok; ++j) {
        const uint32_t g = cnt + j;          // index of this tile among all tiles of the slot
        if (!mbar_wait(&s_full[x], g & 1u, abort_flag, wait_limit)) { ok = false; break; }
        tc_fence_after();
        const bool diagonal = (j == n_mine - 1);
        const int k_pos0 = j * kKvTile;
        // keys of this tile the row may see: all 128, fewer on the diagonal tile (causal)
        const int n_vis = diagonal ? min(kKvTile, max(q_pos - k_pos0 + 1, 0)) : kKvTile;
        // pass 1: row maximum.  The load of chunk c + 1 is in flight while chunk c is reduced.
        float m_tile = -INFINITY;
        {
          uint32_t va[32], vb[32];
          tmem_ld32(s_tmem, va);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t (&cur)[32] = (c & 1) ? vb : va;
            uint32_t (&nxt)[32] = (c & 1) ? va : vb;
            tmem_ld_wait();
            if (c < 3) tmem_ld32(s_tmem + (c + 1) * 32, nxt);
            if (!diagonal) {
              float m0 = __uint_as_float(cur[0]), m1 = __uint_as_float(cur[1]);
              float m2 = __uint_as_float(cur[2]), m3 = __uint_as_float(cur[3]);
#pragma unroll
              for (int i = 4; i < 32; i += 4) {
                m0 = fmaxf(m0, __uint_as_float(cur[i]));
                m1 = fmaxf(m1, __uint_as_float(cur[i + 1]));
                m2 = fmaxf(m2, __uint_as_float(cur[i + 2]));
                m3 = fmaxf(m3, __uint_as_float(cur[i + 3]));
              }
              m_tile = fmaxf(m_tile, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i < n_vis) m_tile = fmaxf(m_tile, __uint_as_float(cur[i]));
            }
          }
        }
        const float m_new = fmaxf(m_ref, m_tile);
        const bool grow = (j == 0) || ((m_new - m_ref) * p.scale_log2 > kRescaleThreshold);
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          // O of this tile must be complete before it is rescaled: the product of the previous tile
          if (!mbar_wait(&o_done[x], (g - 1) & 1u, abort_flag, wait_limit)) { ok = false; break; }
          tc_fence_after();
          const float alpha = grow ? fast_exp2((m_ref - m_new) * p.scale_log2) : 1.0f;
          l_sum *= alpha;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_tmem + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_tmem + c * 32, o);
          }
          tmem_st_wait();
        }
        if (grow) m_ref = m_new;
        // pass 2: exponentials, row sum, P (bf16, two per column) into the first 64 columns of S
        // (chunk c's probabilities land on columns whose scores were consumed with chunk c / 2)
        const float m_scaled = m_ref * p.scale_log2;
        {
          uint32_t va[32], vb[32];
          float l0 = 0.f, l1 = 0.f;
          tmem_ld32(s_tmem, va);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t (&cur)[32] = (c & 1) ? vb : va;
            uint32_t (&nxt)[32] = (c & 1) ? va : vb;
            tmem_ld_wait();
            if (c < 3) tmem_ld32(s_tmem + (c + 1) * 32, nxt);
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float e0 = fast_exp2(fmaf(__uint_as_float(cur[2 * i]), p.scale_log2, -m_scaled));
              float e1 = fast_exp2(fmaf(__uint_as_float(cur[2 * i + 1]), p.scale_log2, -m_scaled));
              if (diagonal) {
                if (c * 32 + 2 * i >= n_vis) e0 = 0.f;
                if (c * 32 + 2 * i + 1 >= n_vis) e1 = 0.f;
              }
              l0 += e0;
              l1 += e1;
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
              pk[i] = *reinterpret_cast<const uint32_t*>(&b2);
            }
            tmem_st16(s_tmem + c * 16, pk);
          }
          l_sum += l0 + l1;
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[x]);
      }
      if (ok) {
        // epilogue: O / l -> bf16 -> out[row, head * D ...]; then O may be overwritten
        if (mbar_wait(&o_done[x], (cnt + n_mine - 1) & 1u, abort_flag, wait_limit)) {
          tc_fence_after();
          const float inv = 1.0f / l_sum;
          const bool row_ok = q_pos < p.S;
          __nv_bfloat16* dst = p.out + (w.row0 + q_pos) * p.ldo + w.q_col;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_tmem + c * 32, o);
            tmem_ld_wait();
            if (c == D / 32 - 1) {           // last read of O: the next item's first product may go
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&o_free[x]);
            }
            if (row_ok) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                uint4 wv;
                uint32_t* ww = reinterpret_cast<uint32_t*>(&wv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const __nv_bfloat162 b2 = __floats2bfloat162_rn(
                      __uint_as_float(o[q4 * 8 + 2 * i]) * inv, __uint_as_float(o[q4 * 8 + 2 * i + 1]) * inv);
                  ww[i] = *reinterpret_cast<const uint32_t*>(&b2);
                }
                *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = wv;
              }
            }
          }
        } else {
          ok = false;
        }
      }
      cnt += n_mine;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 3);
}

}  // namespace

cudaError_t launch_attention_prefill(const void* qkv, void* out, int B, int S, int hq, int hkv, int D,
                                     float scale, int* status, cudaStream_t stream) {
  const long long T = static_cast<long long>(B) * S;
  const int N = (hq + 2 * hkv) * D;
  CUtensorMap tm;
  if (!encode_map_2d(&tm, qkv, T, N, N, 128)) return cudaErrorInvalidValue;
  AttnParams p;
  p.S = S;
  p.hq = hq;
  p.hkv = hkv;
  p.q_tiles = (S + kQTile - 1) / kQTile;
  p.pairs = (p.q_tiles + 1) / 2;
  p.batch = B;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = hq * D;
  p.wait_limit_ns = 0;
  p.status = status;
  // persistent CTAs: one per SM (192 KB of shared memory and all of TMEM each), looping over items
  const long long items = static_cast<long long>(p.pairs) * hq * B;
  const int sms = current_sm_count();
  const dim3 grid(static_cast<unsigned>(items < sms ? items : sms), 1, 1);
  static bool attr_done[2] = {false, false};
  if (D == 128) {
    if (!attr_done[1]) {
      cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<128>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           AttnSmem<128>::kDynamic);
      if (e != cudaSuccess) return e;
      attr_done[1] = true;
    }
    return launch_kernel(attention_prefill_kernel<128>, grid, dim3(kAttnThreads),
                         AttnSmem<128>::kDynamic, stream, tm, p);
  }
  if (!attr_done[0]) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<64>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         AttnSmem<64>::kDynamic);
    if (e != cudaSuccess) return e;
    attr_done[0] = true;
  }
  return launch_kernel(attention_prefill_kernel<64>, grid, dim3(kAttnThreads), AttnSmem<64>::kDynamic,
                       stream, tm, p);
}

}  // namespace cdeep
