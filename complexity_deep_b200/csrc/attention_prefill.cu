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
// Work decomposition: one CTA per (sequence, query head, 128-row query tile), heavy tiles (late
// rows, which see the most keys) first.
//
//   warp  0     TMA producer (the K / V ring, 3 stages each)
//   warp  1     MMA issuer + TMEM owner
//   warps 2-9   softmax: two threads per query row (= TMEM lane), 64 score columns each
//
// Both products take their A operand from tensor memory, so the tensor cores read only ONE
// operand per instruction from shared memory (a 128 x 128 x 16 product fed from shared memory
// on both sides needs the full 128 bytes per clock of the SM and measured at half rate here):
//   * Q (bf16, two elements per column) is written to TMEM once per CTA by the softmax threads;
//   * S_j = Q K_j^T goes to one of TWO score buffers, so the product for tile j + 1 runs while
//     the softmax warps work on tile j;
//   * softmax warps: row max, p = exp2(scale * (s - m)), row sum; P (bf16) overwrites the first
//     columns of the thread's own score columns;
//   * O += P_j V_j with P from TMEM and the V tile read N-major from shared memory.
// The softmax of tile j + 1 does not wait for O: the running maximum m is only raised when it
// grew by more than 2^8 in the exp2 domain (then O and the row sum are rescaled in TMEM, after
// the pending product has finished); otherwise the stale maximum is kept, which is exact as long
// as the final division uses the matching row sum.
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
constexpr int kSoftmaxWarps = 8;
constexpr int kProducerWarp = 0;   // the two single-thread roles come first: lower warp ids are
constexpr int kMmaWarp = 1;        // favoured by the warp scheduler over the eight softmax warps
constexpr int kFirstSoftmaxWarp = 2;
constexpr int kAttnThreads = 320;
constexpr int kKvStages = 3;
constexpr float kRescaleThreshold = 8.0f;   // log2 of the growth of the maximum that forces a rescale

struct AttnParams {
  const __nv_bfloat16* qkv;   // [T, ld]
  int ld;
  long long T;      // B * S rows
  int S;            // sequence length
  int hq, hkv;      // query / kv heads
  int q_tiles;      // ceil(S / 128)
  float scale_log2; // softmax scale * log2(e)
  __nv_bfloat16* out;   // [T, hq * D]
  int ldo;
  unsigned long long wait_limit_ns;
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int kBoxBytes = 128 * 64 * 2;           // one TMA box: 128 rows x 64 columns
  static constexpr int kTileBytes = (D / 64) * kBoxBytes;  // a K or V tile
  static constexpr int kKOff = 0;                          // K ring
  static constexpr int kVOff = kKvStages * kTileBytes;     // V ring
  static constexpr int kBarOff = 2 * kKvStages * kTileBytes;
  static constexpr int kNumBars = 1 + 4 * kKvStages + 5;   // q_ready, k/v full/empty, s_full x2, p_full x2, o_done
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kXchOff = kMiscOff + 16;            // exchange between the two threads of a row:
  static constexpr int kTotal = kXchOff + 128 * 6 * 4;     // 128 rows x 6 floats
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
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kQCol = 0;                    // Q: D / 2 columns (two bf16 per column)
  constexpr uint32_t kSCol0 = 64;                  // two score buffers of 128 columns
  constexpr uint32_t kOCol = 320;                  // O: D columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* q_ready = bars;                       // [1]
  uint64_t* k_full = bars + 1;                    // [kKvStages]
  uint64_t* k_empty = k_full + kKvStages;
  uint64_t* v_full = k_empty + kKvStages;
  uint64_t* v_empty = v_full + kKvStages;
  uint64_t* s_full = v_empty + kKvStages;         // [2] per score buffer
  uint64_t* p_full = s_full + 2;                  // [2]
  uint64_t* o_done = p_full + 2;                  // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint64_t wait_limit = p.wait_limit_ns ? p.wait_limit_ns : kWaitLimitNs;

  // work item: heavy tiles (late rows of the sequence see the most keys) are scheduled first
  const int qt = p.q_tiles - 1 - static_cast<int>(blockIdx.x);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int kv_head = head / (p.hq / p.hkv);
  const int n_kv = qt + 1;                            // tile qt sees KV tiles 0 .. qt
  const long long row0 = static_cast<long long>(batch) * p.S;   // first token row of this sequence
  const int q_col = head * D;
  const int k_col = (p.hq + kv_head) * D;
  const int v_col = (p.hq + p.hkv + kv_head) * D;

  if (warp == kProducerWarp && lane == 0) {
    mbar_init(q_ready, kSoftmaxWarps);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], kSoftmaxWarps);     // one arrival per softmax warp
    }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm_qkv);
  } else if (warp == kMmaWarp) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  griddep_wait();
  griddep_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == kProducerWarp) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j % kKvStages;
        const uint32_t ph = (j / kKvStages) & 1u;
        const int kv_row = static_cast<int>(row0) + j * kKvTile;
        if (!mbar_wait(&k_empty[s], ph ^ 1u, abort_flag, wait_limit)) { ok = false; break; }
        mbar_arrive_expect_tx(&k_full[s], L::kTileBytes);
        for (int d = 0; d < kDBlocks; ++d)
          tma_load_2d(smem + L::kKOff + s * L::kTileBytes + d * L::kBoxBytes, &tm_qkv, &k_full[s],
                      k_col + d * 64, kv_row);
        if (!mbar_wait(&v_empty[s], ph ^ 1u, abort_flag, wait_limit)) { ok = false; break; }
        mbar_arrive_expect_tx(&v_full[s], L::kTileBytes);
        for (int d = 0; d < kDBlocks; ++d)
          tma_load_2d(smem + L::kVOff + s * L::kTileBytes + d * L::kBoxBytes, &tm_qkv, &v_full[s],
                      v_col + d * 64, kv_row);
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kQTile, kKvTile);         // S = Q K^T
      constexpr uint32_t idesc_o = make_idesc_bf16(kQTile, D, true);         // O = P V (V N-major)
      const uint32_t k_addr = smem_u32(smem + L::kKOff);
      const uint32_t v_addr = smem_u32(smem + L::kVOff);
      bool ok = true;
      // S_j = Q K_j^T into score buffer j & 1: D / 16 MMAs, Q from TMEM (8 columns per step of
      // 16 elements), K_j from the 64-column boxes of its stage
      auto issue_s = [&](int j) {
        // one descriptor per burst; a step of 16 elements along K is +2 (units of 16 bytes) inside
        // a 64-column box, the next box is kBoxBytes further (the address field cannot overflow:
        // shared-memory addresses stay below 256 KB)
        const uint64_t db0 = make_smem_desc_sw128(k_addr + (j % kKvStages) * L::kTileBytes);
        const uint32_t d_tmem = tmem_base + kSCol0 + (j & 1) * 128;
        const uint32_t a_tmem = tmem_base + kQCol;
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_tmem_a(d_tmem, a_tmem + 8u * k, db0 + ((k >> 2) * (L::kBoxBytes >> 4) + 2u * (k & 3)),
                           idesc_s, k != 0 ? 1u : 0u);
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[j % kKvStages]);   // K_j is free once these products have read it
      };
      // O (+)= P_j V_j: 8 MMAs of 16 keys; P (two bf16 per column) sits in columns 0-31 (keys
      // 0-63) and 64-95 (keys 64-127) of its score buffer, the V tile is read N-major: 16 key
      // rows = 2048 bytes further per step
      auto issue_pv = [&](int j) {
        const uint64_t db0 = make_smem_desc_mn_sw128(v_addr + (j % kKvStages) * L::kTileBytes, L::kBoxBytes);
        const uint32_t p_tmem = tmem_base + kSCol0 + (j & 1) * 128;
        const uint32_t o_acc = tmem_base + kOCol;
        const uint32_t first = j != 0 ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < kKvTile / 16; ++k)
          umma_bf16_tmem_a(o_acc, p_tmem + (k < 4 ? 8u * k : 32u + 8u * k), db0 + k * (2048u >> 4), idesc_o,
                           k != 0 ? 1u : first);
        umma_commit(&v_empty[j % kKvStages]);
        umma_commit(o_done);
      };
      if (!mbar_wait(q_ready, 0, abort_flag, wait_limit)) ok = false;
      // The scores run TWO tiles ahead of the softmax: S(j + 2) is issued in the same burst as
      // PV(j) (it overwrites the buffer of P(j), which the in-order tensor pipe has consumed by
      // then), so the pipe's start-up latency is paid once per burst of 16 instructions and
      // the softmax warps always find their next scores ready.
      for (int j = 0; j < 2 && j < n_kv && ok; ++j) {
        if (!mbar_wait(&k_full[j % kKvStages], 0, abort_flag, wait_limit)) { ok = false; break; }
        tc_fence_after();
        issue_s(j);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        // operands that were requested long ago first, then the probabilities
        if (!mbar_wait(&v_full[j % kKvStages], (j / kKvStages) & 1u, abort_flag, wait_limit)) { ok = false; break; }
        if (j + 2 < n_kv &&
            !mbar_wait(&k_full[(j + 2) % kKvStages], ((j + 2) / kKvStages) & 1u, abort_flag, wait_limit)) { ok = false; break; }
        if (!mbar_wait(&p_full[j & 1], (j >> 1) & 1u, abort_flag, wait_limit)) { ok = false; break; }
        tc_fence_after();
        issue_pv(j);
        if (j + 2 < n_kv) {
          issue_s(j + 2);
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax warps
    // Two threads per query row: softmax warps w and w + 4 share a TMEM lane quarter and take the two
    // halves of the 128 score columns (and of the D output columns); the halves exchange their
    // row maxima through shared memory, ordered by a named barrier of the two warps.  Each
    // thread only ever writes tensor-memory columns it alone reads.
    const int quarter = warp & 3;            // TMEM lane quarter this warp may access
    const int half = (warp - kFirstSoftmaxWarp) >> 2;   // column half
    const int row = quarter * 32 + lane;     // row within the tile
    const int q_pos = qt * kQTile + row;     // position of this thread's row in its sequence
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t o_tmem = tmem_base + lane_addr + kOCol + half * (D / 2);
    const uint32_t pair_bar = 1 + quarter;   // named barrier of the two warps of a lane quarter
    float* xch = reinterpret_cast<float*>(smem + L::kXchOff) + row * 6;   // maxima [parity][half], row sums [half]

    {
      // this thread's half of its Q row -> TMEM (two bf16 per column, the A operand layout)
      const long long grow_ = row0 + q_pos;
      const uint4* src = reinterpret_cast<const uint4*>(p.qkv + grow_ * p.ld + q_col + half * (D / 2));
      uint32_t qv[D / 4];
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        uint4 t = make_uint4(0, 0, 0, 0);
        if (grow_ < p.T) t = src[i];
        qv[4 * i] = t.x; qv[4 * i + 1] = t.y; qv[4 * i + 2] = t.z; qv[4 * i + 3] = t.w;
      }
      const uint32_t q_tmem = tmem_base + lane_addr + kQCol + half * (D / 4);
      if constexpr (D == 128) tmem_st32(q_tmem, qv); else tmem_st16(q_tmem, qv);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);
    }

    float m_ref = -INFINITY;                 // maximum the stored exponentials refer to (raw scores)
    float l_sum = 0.f;                       // this thread's half of the row sum
    bool ok = true;
    // (after a wait gave up, `ok` is false and the remaining iterations only keep the pair
    // barrier counts of the two warps equal, so nobody is left waiting at a named barrier)
    for (int j = 0; j < n_kv; ++j) {
      if (ok && !mbar_wait(&s_full[j & 1], (j >> 1) & 1u, abort_flag, wait_limit)) ok = false;
      ok = __all_sync(0xffffffffu, ok);   // warp-uniform: the tensor-memory instructions below are warp-wide
                  tc_fence_after();
      const bool diagonal = (j == n_kv - 1);
      // keys of this thread's 64 columns the row may see: all, fewer on the diagonal tile
      const int n_vis = diagonal ? min(64, max(q_pos - j * kKvTile - half * 64 + 1, 0)) : 64;
      const uint32_t s_mine = tmem_base + lane_addr + kSCol0 + (j & 1) * 128 + half * 64;
      uint32_t v[64];
      tmem_ld32(s_mine, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
      tmem_ld32(s_mine + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
      tmem_ld_wait();   // (harmless on stale data when !ok: nothing below is stored then)
      float m_part;
      if (!diagonal) {
        float m0 = __uint_as_float(v[0]), m1 = __uint_as_float(v[1]);
        float m2 = __uint_as_float(v[2]), m3 = __uint_as_float(v[3]);
#pragma unroll
        for (int i = 4; i < 64; i += 4) {
          m0 = fmaxf(m0, __uint_as_float(v[i]));
          m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
          m2 = fmaxf(m2, __uint_as_float(v[i + 2]));
          m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
        }
        m_part = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      } else {
        m_part = -INFINITY;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i < n_vis) m_part = fmaxf(m_part, __uint_as_float(v[i]));
      }
      // exchange with the thread that holds the other half of the row
      xch[(j & 1) * 2 + half] = m_part;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      const float m_tile = fmaxf(m_part, xch[(j & 1) * 2 + (half ^ 1)]);
      const float m_new = fmaxf(m_ref, m_tile);
      const bool grow = (j == 0) || ((m_new - m_ref) * p.scale_log2 > kRescaleThreshold);
      if (!ok) continue;
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // O must be complete before it is rescaled: PV(j - 1) is the j-th product
        if (!mbar_wait(o_done, (j - 1) & 1u, abort_flag, wait_limit)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) continue;
        tc_fence_after();
        const float alpha = grow ? fast_exp2((m_ref - m_new) * p.scale_log2) : 1.0f;
        l_sum *= alpha;
#pragma unroll 1
        for (int c = 0; c < D / 64; ++c) {     // this thread's D / 2 output columns
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
      // exponentials, row sum, P (bf16, two per column): this half's 64 probabilities go to the
      // first 32 of ITS OWN score columns; the MMA warp reads keys 0-63 at column 0 and keys
      // 64-127 at column 64 of the buffer
            const float m_scaled = m_ref * p.scale_log2;
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float e0 = fast_exp2(fmaf(__uint_as_float(v[c * 32 + 2 * i]), p.scale_log2, -m_scaled));
          float e1 = fast_exp2(fmaf(__uint_as_float(v[c * 32 + 2 * i + 1]), p.scale_log2, -m_scaled));
          if (diagonal) {
            if (c * 32 + 2 * i >= n_vis) e0 = 0.f;
            if (c * 32 + 2 * i + 1 >= n_vis) e1 = 0.f;
          }
          l0 += e0;
          l1 += e1;
          const __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
          pk[i] = *reinterpret_cast<const uint32_t*>(&b2);
        }
        tmem_st16(s_mine + c * 16, pk);
      }
      l_sum += l0 + l1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[j & 1]);
          }
    {
      // full row sum = this half + the other half
      xch[4 + half] = l_sum;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      l_sum += xch[4 + (half ^ 1)];
    }
    if (ok) {
      // epilogue: O / l -> bf16 -> out[row, head * D + this thread's D / 2 columns]
      if (__all_sync(0xffffffffu, mbar_wait(o_done, (n_kv - 1) & 1u, abort_flag, wait_limit))) {
        tc_fence_after();
        const float inv = 1.0f / l_sum;
        const bool row_ok = q_pos < p.S;
        __nv_bfloat16* dst = p.out + (row0 + q_pos) * p.ldo + q_col + half * (D / 2);
#pragma unroll 1
        for (int c = 0; c < D / 64; ++c) {
          uint32_t o[32];
          tmem_ld32(o_tmem + c * 32, o);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 w;
              uint32_t* ww = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 b2 = __floats2bfloat162_rn(
                    __uint_as_float(o[q4 * 8 + 2 * i]) * inv, __uint_as_float(o[q4 * 8 + 2 * i + 1]) * inv);
                ww[i] = *reinterpret_cast<const uint32_t*>(&b2);
              }
              *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = w;
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
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
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.ld = N;
  p.T = T;
  p.S = S;
  p.hq = hq;
  p.hkv = hkv;
  p.q_tiles = (S + kQTile - 1) / kQTile;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = hq * D;
  p.wait_limit_ns = 0;
  p.status = status;
  const dim3 grid(static_cast<unsigned>(p.q_tiles), static_cast<unsigned>(hq), static_cast<unsigned>(B));
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
