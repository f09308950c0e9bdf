// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA-fed shared-memory pipeline,
// tcgen05.mma accumulating in TMEM (two accumulators, so the epilogue of one tile runs
// under the main loop of the next), ragged per-expert row segments, two K segments
// (K-concatenation without materialising the concatenated operand), fused epilogues.
//
//   C[rows of group g, :] = A0[rows, :K0] * B0[g]^T  +  A1[rows, :K1] * B1[g]^T
//
// A0/A1 are row-major [M, K*] activations, B0/B1 are K-major weights [groups * N, K*]
// (nn.Linear layout: one output feature per row).  Groups are contiguous row ranges of A
// given by `seg_offsets` on the device, so no host synchronisation is needed to schedule
// ragged expert segments.  Rows of a 128-row tile that lie past the end of its segment are
// computed (they are real rows of the next segment, or TMA zero fill) and never stored.
//
// This one kernel covers, through its epilogue and operand set-up:
//   * the routed and the shared SwiGLU up-projections with silu(gate)*up fused
//     (reference: complexity_deep/core/token_routed_mlp.py:157-160,171-173),
//   * the down projections of routed + shared experts as ONE fp32 accumulation, the
//     un-permutation of rows and the block's residual add (token_routed_mlp.py:174-178,
//     complexity_deep/core/layer.py:183),
//   * the mu-guided QKV projection [x | mu_prev] @ [W ; W_mu]^T
//     (complexity_deep/core/attention.py:120-127),
//   * mu_proj with the clamp(mu) term (complexity_deep/core/layer.py:61) and the model's
//     output clamp (complexity_deep/models/modeling.py:199-200),
//   * plain projections with an optional residual (o_proj, lm_head).
#pragma once
#include <cuda_bf16.h>
#include "checks.cuh"
#include "ptx.cuh"

namespace cdeep {

constexpr int kBlockM = 128;       // rows per tile = TMEM lanes
constexpr int kBoxK = 64;          // bf16 elements per TMA box row = one 128-byte swizzle row
// Boxes per operand and pipeline stage.  The thread that issues the MMAs pays a fixed price per
// stage (barrier wait, fence, commit: about 300 cycles measured) on top of 40 .. 64 cycles per
// tcgen05.mma of a tile up to 128 columns wide, so the single-CTA tiles up to 128 wide — few-row
// calls, whose K loop is bound by that thread — take two boxes (128 elements of K) per stage:
// 0.29 -> 0.21 us per 64 elements of K for 32-wide tiles; for 128-wide tiles (grouped few-row
// calls, the cluster form of split-K) the gain is a few per cent.  256-wide tiles are bound by the
// tensor pipe and want many fine stages instead (with two boxes the 1B prefill step was 5 % slower).
__host__ __device__ constexpr int gemm_k_boxes(int bn, int cg) { return (cg == 1 && bn <= 128) ? 2 : 1; }
constexpr int kUmmaK = 16;         // K of one tcgen05.mma for 16-bit inputs
constexpr int kMaxGroups = 128;
constexpr int kEpiCols = 64;          // output columns per epilogue sub-tile (128 bytes of bf16)
constexpr int kEpiStageBytes = 4096;  // 32 rows x 128 bytes, per warp and buffer

enum GemmEpilogue : int {
  kEpiStore = 0,      // out[row_map(r), n] = clamp(acc + bias[n] + residual[row_map(r), n])
  kEpiSwiGLU = 1,     // out[r, j] = silu(acc[r, gate(j)]) * acc[r, up(j)]
  kEpiStoreRope = 2,  // store with per-head RMSNorm + rotary embedding (256-wide tiles only)
  kEpiStoreSplit = 3, // store of a split-bf16 value: out = bf16(v), out_lo = bf16(v - out); the
                      // residual may be split the same way (residual + residual_lo)
};

// Warp roles: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2 .. 2 + EW - 1
// epilogue.  A warp may only read the TMEM lane quarter (warp id % 4); with EW = 8 two warps
// share each quarter and take alternate 64-column sub-tiles.  Eight warps halve the part of
// the epilogue that nothing overlaps (the last tile of every CTA), which matters when a CTA
// runs only three or four tiles: 1B prefill step at 8 192 tokens 16.33 -> 15.93 ms on B200,
// unchanged at 65 536 tokens (there the epilogue already ran under the next tile's main
// loop).  The fused RoPE epilogue keeps four warps and its 255 registers per thread.
template <int BN, int EPI>
__host__ __device__ constexpr int gemm_epi_warps() {
  return (BN == 256 && EPI != kEpiStoreRope) ? 8 : 4;
}
template <int BN, int EPI>
__host__ __device__ constexpr int gemm_threads() {
  return 64 + 32 * gemm_epi_warps<BN, EPI>();
}

struct GemmParams {
  int M;                   // rows of A
  int N;                   // rows of B per group (= accumulator columns per group)
  int K0, K1;              // K extents of the two segments (K1 == 0: one segment)
  int num_groups;          // row segments; 1 = dense
  const int* seg_offsets;  // device [num_groups + 1]; nullptr = one segment [0, M)
  int b0_group_rows;       // B0 row offset per group (0: all groups share B0)
  int b1_group_rows;       // same for B1
  int band;                // m-tiles per scheduling band (L2 reuse of the A band)
  // epilogue
  __nv_bfloat16* out;
  int ldo;
  int out_cols;            // valid output columns (N for store, N/2-ish width I for SwiGLU)
  const int* row_map;      // sorted row -> destination row (nullptr = identity)
  int out_rows;            // rows of the destination (checking build: row_map entries must lie below; 0 = unknown)
  const long long* out_row_ptrs;  // sorted row -> ADDRESS of its destination row (overrides out /
                                  // row_map; rows may live in another GPU's peer-mapped memory)
  const __nv_bfloat16* residual;  // indexed like out (nullptr = none)
  int ldr;
  // split-bf16 residual stream (kEpiStoreSplit): the value carried between kernels is
  // hi + lo with hi = bf16(v), lo = bf16(v - hi) (16 significant bits instead of 8)
  const __nv_bfloat16* residual_lo;  // low part of the residual, indexed like residual (nullptr = none)
  __nv_bfloat16* out_lo;             // low part of the result, indexed like out (nullptr = not stored)
  // optional second problem over the same A rows (SwiGLU epilogue, one K segment): a dense
  // [M, N2] product against B1 whose tiles follow the grouped ones in the same launch
  int N2;                  // accumulator columns of the second problem (0 = none)
  __nv_bfloat16* out2;
  int ldo2;
  int out_cols2;
  const __nv_bfloat16* residual2;  // second addend, indexed by the tile row itself (nullptr = none)
  int ldr2;
  const __nv_bfloat16* bias;      // per output column, clamped to [bias_lo, bias_hi] (nullptr = none)
  float bias_lo, bias_hi;
  int do_clamp;            // clamp the result to [clamp_lo, clamp_hi]
  float clamp_lo, clamp_hi;
  // optional: per-head RMSNorm + rotary embedding on the first rope_cols output columns
  // (heads of 128 columns; store epilogue with 256-wide tiles only, no residual / bias)
  const float* rope_cos;   // [positions, 128] fp32 (nullptr = off)
  const float* rope_sin;
  const __nv_bfloat16* rope_qw;   // [128] norm weights of the q / k heads (both nullptr = no norm)
  const __nv_bfloat16* rope_kw;
  float rope_eps;
  int rope_S, rope_pos0;   // row r sits at position rope_pos0 + r % rope_S
  int rope_q_cols;         // columns [0, rope_q_cols) are q heads, [rope_q_cols, rope_cols) k heads
  int rope_cols;
  // split-K for few-row calls (CG = 1): the K loop of every output tile is cut into `splits`
  // ranges computed by different CTAs; each writes its fp32 partial tile to sk_scratch and
  // counts in sk_counters[tile]; the CTA that arrives last adds the partials and runs the fused
  // epilogue (and puts the counter back to zero for the next launch)
  int splits;              // 1 = off
  float* sk_scratch;       // [tiles * splits][128][BN] fp32
  int* sk_counters;        // [tiles], zero between launches
  // split-K inside a cluster (store epilogues, BN / splits a multiple of 32): the launch has
  // tiles x splits CTAs in clusters of `splits`; the CTAs of a cluster hold the partial tiles of
  // one output tile in their shared memory, CTA s reduces and stores the columns
  // [s * BN / splits, (s + 1) * BN / splits) of it, reading the others' partials through
  // distributed shared memory.  No workspace, no atomics.
  int sk_cluster;          // 1 = the cluster form (sk_scratch / sk_counters unused)
  // self-test of the failure path: with `selftest_stall` the producer issues no loads, so the
  // pipeline waits run into `wait_limit_ns` (0 = the default limit) and the kernel must leave
  // cleanly with the status word raised
  unsigned long long wait_limit_ns;
  int selftest_stall;
  int* status;             // device word; set non-zero when a bounded wait ran out
};

// CG = 1: one CTA per 128-row tile.  CG = 2: a CTA pair per 256-row tile (cta_group::2); each
// CTA stages its 128 rows of A and its BN / 2 rows of B.
template <int BN, int CG, int EW = 4>
struct GemmSmem {
  static constexpr int kKBoxes = gemm_k_boxes(BN, CG);
  static constexpr int kBlockK = kBoxK * kKBoxes;   // bf16 elements of K per pipeline stage (k-block)
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = (BN / CG) * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // epilogue staging: EW warps x 2 buffers
  static constexpr int kEpiBytes = EW * 2 * kEpiStageBytes;
  // as many stages as fit beside it in 224 KB (with four epilogue warps: 4 x 48 KB, 6 x 32 KB,
  // 8 x 24 KB, 9 x 20 KB): narrow tiles run with few rows, where the K loop is bound by load
  // latency, not bandwidth
  static constexpr int kTileBudget = 196608 + 4 * 2 * kEpiStageBytes - kEpiBytes;
  static constexpr int kStages = (kTileBudget / kStageBytes) > 12 ? 12 : (kTileBudget / kStageBytes);
  static constexpr int kTileBytes = kStages * kStageBytes;
  // after the tiles: epilogue staging, barriers, TMEM base, abort flag, schedule tables
  static constexpr int kEpiOff = kTileBytes;
  static constexpr int kBarOff = kEpiOff + kEpiBytes;
  static constexpr int kNumBars = 2 * kStages + 5;   // full, empty, tmem_full[2], tmem_empty[2], split-K
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kPrefixOff = kMiscOff + 16;
  static constexpr int kSegOff = kPrefixOff + (kMaxGroups + 2) * 4;
  static constexpr int kTotal = kSegOff + (kMaxGroups + 1) * 4;
  static constexpr int kDynamic = kTotal + 1024;  // slack for 1024-byte alignment
};

struct TileCoord {
  int group;
  int m0;       // first row of the tile (global row of A)
  int n0;       // first accumulator column within the group
  int row_end;  // one past the last valid row of the segment
};

// Maps a linear tile index to its coordinates.  Within a group, tiles are ordered in bands
// of `band` m-tiles; inside a band the m index runs fastest, so the CTAs that run together
// share a small set of B tiles while the A band stays in L2.  Group index `num_groups` is the
// optional second problem: all M rows as one segment, `n_tiles2` tiles wide.
__device__ __forceinline__ TileCoord decode_tile(int t, int& gcur, const int* prefix,
                                                 const int* seg, int num_groups, int M,
                                                 int n_tiles, int n_tiles2, int band,
                                                 int bn, int block_m) {
  while (t >= prefix[gcur + 1]) ++gcur;
  const bool second = gcur >= num_groups;
  const int local = t - prefix[gcur];
  const int lo = second ? 0 : seg[gcur], hi = second ? M : seg[gcur + 1];
  const int nt = second ? n_tiles2 : n_tiles;
  const int m_tiles = (hi - lo + block_m - 1) / block_m;
  const int per_band = band * nt;
  const int b = local / per_band;
  const int within = local - b * per_band;
  const int m_first = b * band;
  const int bh = min(band, m_tiles - m_first);
  const int n_idx = within / bh;
  const int m_idx = m_first + (within - n_idx * bh);
  TileCoord c;
  c.group = gcur;
  c.m0 = lo + m_idx * block_m;
  c.n0 = n_idx * bn;
  c.row_end = hi;
  return c;
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

template <int BN, int EPI, int CG>
__global__ void __launch_bounds__(gemm_threads<BN, EPI>(), 1)
gemm_bf16_sm100_kernel(const __grid_constant__ CUtensorMap tmA0,
                       const __grid_constant__ CUtensorMap tmB0,
                       const __grid_constant__ CUtensorMap tmA1,
                       const __grid_constant__ CUtensorMap tmB1, const GemmParams p) {
  constexpr int EW = gemm_epi_warps<BN, EPI>();
  constexpr int kEpiHalves = EW / 4;               // epilogue warps per TMEM lane quarter
  constexpr bool kStore = (EPI == kEpiStore || EPI == kEpiStoreRope || EPI == kEpiStoreSplit);
  constexpr bool kSplit = (EPI == kEpiStoreSplit);
  using L = GemmSmem<BN, CG, EW>;
  constexpr int S = L::kStages;
  constexpr int kKBoxes = L::kKBoxes;
  constexpr int kBlockK = L::kBlockK;
  constexpr int kTileM = kBlockM * CG;             // rows per tile (per CTA pair when CG = 2)
  const uint32_t crank = (CG == 2) ? cluster_ctarank() : 0u;  // 0 = leader
  const int tile0 = blockIdx.x / CG;               // both CTAs of a pair walk the same tiles
  const int tstride = gridDim.x / CG;
  // Tiles up to 128 wide (few-row calls: an output tile is one chain of K/16 dependent MMA
  // instructions) accumulate even and odd K steps in two TMEM accumulators that the epilogue
  // adds: two independent chains, measured 2-4 % less time per launch (K = 2048 ... 8192).
  constexpr int kChains = (BN <= 128 && CG == 1) ? 2 : 1;
  constexpr uint32_t kAccCols = kChains * BN;     // TMEM columns of one tile's accumulator(s)
  // two tiles in flight (main loop / epilogue); 32-wide tiles allocate more than they need
  // because the epilogue always reads 32-column groups
  constexpr uint32_t kTmemCols = (BN == 32) ? 256 : 2 * kAccCols;
  static_assert(kTmemCols == 64 || kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512,
                "TMEM allocation must be a power of two >= 32");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* empty_bar = full_bar + S;
  uint64_t* tmem_full = empty_bar + S;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;  // [2]
  uint64_t* sk_bar = tmem_empty + 2;     // cluster split-K: every partial tile of the cluster is written
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  int* prefix = reinterpret_cast<int*>(smem + L::kPrefixOff);
  int* seg = reinterpret_cast<int*>(smem + L::kSegOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int n_tiles2 = (p.N2 + BN - 1) / BN;   // 0 without a second problem
  const int kb0 = (p.K0 + kBlockK - 1) / kBlockK;
  const int kb1 = (p.K1 + kBlockK - 1) / kBlockK;
  const int kb_total = kb0 + kb1;
  const uint64_t wait_limit = p.wait_limit_ns ? p.wait_limit_ns : kWaitLimitNs;

  // ---------------------------------------------------------------- set-up
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], EW * CG);  // one arrival per epilogue warp (of both CTAs)
    }
    mbar_init(sk_bar, (p.splits > 1 ? p.splits : 1) * EW);  // one arrival per epilogue warp of the cluster
    *abort_flag = 0;
    *reinterpret_cast<int*>(smem + L::kMiscOff + 8) = 0;
    *reinterpret_cast<int*>(smem + L::kMiscOff + 12) = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA0);
    tma_prefetch_desc(&tmB0);
    if (p.K1 > 0) tma_prefetch_desc(&tmA1);
    if (p.K1 > 0 || p.N2 > 0) tma_prefetch_desc(&tmB1);
  } else if (warp == 1) {
    if constexpr (CG == 2) {
      tmem_alloc_pair(tmem_base_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_base_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  // Everything above touched only this CTA's shared memory, TMEM and the kernel parameters,
  // so it may run while the previous kernel of the stream is still finishing.
  griddep_wait();
  griddep_launch_dependents();
  if (warp == 2 && lane == 0) {
    int acc = 0;
    bool bad = false;
    prefix[0] = 0;
    for (int g = 0; g < p.num_groups; ++g) {
      const int lo = p.seg_offsets ? p.seg_offsets[g] : 0;
      const int hi = p.seg_offsets ? p.seg_offsets[g + 1] : p.M;
      if (kChecks && (lo < 0 || hi < lo || hi > p.M)) bad = true;
      seg[g] = lo;
      seg[g + 1] = hi;
      acc += ((hi - lo + kTileM - 1) / kTileM) * n_tiles;
      prefix[g + 1] = acc;
    }
    if (p.N2 > 0) prefix[p.num_groups + 1] = acc + ((p.M + kTileM - 1) / kTileM) * n_tiles2;
    if (kChecks && bad) {
      // checking build: a segment table that is not 0 <= s[0] <= s[1] <= ... <= M schedules nothing
      atomicMax(p.status, kStatusBounds);
      for (int g = 0; g <= p.num_groups + 1; ++g) prefix[g] = 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  constexpr bool kSplitK = (CG == 1 && BN <= 128);
  // the cluster form of split-K exists for 128-wide store tiles only (uniform over the launch)
  constexpr bool kClusterSplitK = kSplitK && kStore && BN == 128;
  const bool csk = kClusterSplitK && p.splits > 1 && p.sk_cluster != 0;
  if constexpr (CG == 2) cluster_sync_all();  // the peer's barriers exist before anyone signals them
  else if (csk) cluster_sync_all();
  tc_fence_after();

  const uint32_t tmem_base = *tmem_base_slot;
  const int total_tiles = prefix[p.num_groups + (p.N2 > 0 ? 1 : 0)];
  // split-K only in the narrow single-CTA instantiations (the few-row problems it is for never
  // take the 256-wide tile, whose epilogue has no registers to spare)
  const int splits = (kSplitK && p.splits > 1) ? p.splits : 1;
  const int total_units = total_tiles * splits;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      int gcur = 0;
      bool ok = true;
      for (int u = tile0; u < total_units && ok; u += tstride) {
        const int t = u / splits;
        const int sp = u - t * splits;
        const int kb_lo = (sp * kb_total) / splits, kb_hi = ((sp + 1) * kb_total) / splits;
        const TileCoord c = decode_tile(t, gcur, prefix, seg, p.num_groups, p.M, n_tiles, n_tiles2,
                                        p.band, BN, kTileM);
        const bool second = c.group >= p.num_groups;   // dense problem against B1, K segment 0 only
        const int a_row = c.m0 + static_cast<int>(crank) * kBlockM;
        const int b0_row = c.group * p.b0_group_rows + c.n0 + static_cast<int>(crank) * (BN / CG);
        const int b1_row = (second ? 0 : c.group * p.b1_group_rows) + c.n0 +
                           static_cast<int>(crank) * (BN / CG);
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const uint32_t s = it % S;
          const uint32_t ph = (it / S) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag, wait_limit)) {
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * L::kStageBytes;
          uint8_t* b_dst = a_dst + L::kABytes;
          if (p.selftest_stall) continue;  // nothing is loaded: the consumers' waits must expire
          if constexpr (CG == 2) {
            // the leader's barrier collects the bytes of both CTAs
            if (crank == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * L::kStageBytes);
            const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
            if (second) {
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d_pair(a_dst + h * (L::kABytes / kKBoxes), &tmA0, bar, kb * kBlockK + h * kBoxK, a_row);
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d_pair(b_dst + h * (L::kBBytes / kKBoxes), &tmB1, bar, kb * kBlockK + h * kBoxK, b1_row);
            } else if (kb < kb0) {
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d_pair(a_dst + h * (L::kABytes / kKBoxes), &tmA0, bar, kb * kBlockK + h * kBoxK, a_row);
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d_pair(b_dst + h * (L::kBBytes / kKBoxes), &tmB0, bar, kb * kBlockK + h * kBoxK, b0_row);
            } else {
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d_pair(a_dst + h * (L::kABytes / kKBoxes), &tmA1, bar, (kb - kb0) * kBlockK + h * kBoxK, a_row);
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d_pair(b_dst + h * (L::kBBytes / kKBoxes), &tmB1, bar, (kb - kb0) * kBlockK + h * kBoxK, b1_row);
            }
          } else {
            mbar_arrive_expect_tx(&full_bar[s], L::kStageBytes);
            if (second) {
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d(a_dst + h * (L::kABytes / kKBoxes), &tmA0, &full_bar[s], kb * kBlockK + h * kBoxK, a_row);
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d(b_dst + h * (L::kBBytes / kKBoxes), &tmB1, &full_bar[s], kb * kBlockK + h * kBoxK, b1_row);
            } else if (kb < kb0) {
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d(a_dst + h * (L::kABytes / kKBoxes), &tmA0, &full_bar[s], kb * kBlockK + h * kBoxK, a_row);
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d(b_dst + h * (L::kBBytes / kKBoxes), &tmB0, &full_bar[s], kb * kBlockK + h * kBoxK, b0_row);
            } else {
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d(a_dst + h * (L::kABytes / kKBoxes), &tmA1, &full_bar[s], (kb - kb0) * kBlockK + h * kBoxK, a_row);
              for (int h = 0; h < kKBoxes; ++h) tma_load_2d(b_dst + h * (L::kBBytes / kKBoxes), &tmB1, &full_bar[s], (kb - kb0) * kBlockK + h * kBoxK, b1_row);
            }
          }
        }
      }
      if (ok) {
        // Drain: wait until the MMA warp has consumed every stage this thread filled, so
        // no bulk copy is still writing shared memory when the CTA exits.
        const uint32_t filled = it < static_cast<uint32_t>(S) ? it : static_cast<uint32_t>(S);
        for (uint32_t d = 0; d < filled && ok; ++d) {
          const uint32_t j = it - filled + d;  // the last `filled` fills
          ok = mbar_wait(&empty_bar[j % S], (j / S) & 1u, abort_flag, wait_limit);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && crank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kTileM, BN);
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool ok = true;
      for (int u = tile0; u < total_units && ok; u += tstride, ++tcount) {
        const int sp = u % splits;
        const int kb_lo = (sp * kb_total) / splits, kb_hi = ((sp + 1) * kb_total) / splits;
        const uint32_t acc = tcount & 1u;
        const uint32_t acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1u, abort_flag, wait_limit)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const uint32_t s = it % S;
          const uint32_t ph = (it / S) & 1u;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, wait_limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * L::kStageBytes);
          const uint64_t da0 = make_smem_desc_sw128(a_addr);
          const uint64_t db0 = make_smem_desc_sw128(a_addr + L::kABytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // box k / 4 of the stage (descriptor addresses are in 16-byte units); inside the box,
            // advancing 16 bf16 (32 bytes) along K within the swizzle row is +2
            constexpr int kPerBox = kBoxK / kUmmaK;
            const uint64_t da = da0 + static_cast<uint64_t>((k / kPerBox) * (L::kABytes / kKBoxes / 16) + 2 * (k % kPerBox));
            const uint64_t db = db0 + static_cast<uint64_t>((k / kPerBox) * (L::kBBytes / kKBoxes / 16) + 2 * (k % kPerBox));
            if constexpr (CG == 2)
              umma_bf16_pair(d_tmem, da, db, idesc, ((kb - kb_lo) | k) != 0 ? 1u : 0u);
            else
              umma_bf16(d_tmem + (k % kChains) * BN, da, db, idesc,
                        ((kb - kb_lo) | (k / kChains)) != 0 ? 1u : 0u);
          }
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if constexpr (CG == 2) umma_commit_pair(&empty_bar[s]); else umma_commit(&empty_bar[s]);
        }
        if (ok) {  // accumulator complete
          if constexpr (CG == 2) umma_commit_pair(&tmem_full[acc]); else umma_commit(&tmem_full[acc]);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (EW warps)
    // A thread owns one accumulator row (TMEM lane), but rows are 32 different cache lines:
    // results are therefore staged through a per-warp shared-memory buffer (32 rows x 64
    // bf16 columns = 4 KB, 16-byte chunks XOR-swizzled by row so both access patterns are
    // conflict-free) and leave in a coalesced pattern: 8 lanes cover the 128 bytes of one
    // row, a warp instruction covers 4 rows.  The residual enters the same way, fetched with
    // cp.async one and two sub-tiles ahead — the first two before the accumulator is even
    // complete — so its latency stays off the critical path.
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    const int ehalf = (warp - 2) >> 2;   // which of the quarter's warps (takes sub-tiles ehalf, ehalf + kEpiHalves, ...)
    uint8_t* stage0 = smem + L::kEpiOff + (warp - 2) * (2 * kEpiStageBytes);
    const int crow_l = lane >> 3;   // row within a group of 4 rows (coalesced phase)
    const int cchunk = lane & 7;    // 16-byte chunk within the 128-byte row
    const uint32_t own_off = static_cast<uint32_t>(lane) * 128u;  // this lane's row (owner phase)
    uint32_t tcount = 0;
    int gcur = 0;
    bool ok = true;
    int* sk_arrivals = reinterpret_cast<int*>(smem + L::kMiscOff + 12);   // split-K: epilogue-warp barrier
    int sk_target = 0;
    for (int u = tile0; u < total_units && ok; u += tstride, ++tcount) {
      const int t = u / splits;
      const int sp = u - t * splits;
      const TileCoord c = decode_tile(t, gcur, prefix, seg, p.num_groups, p.M, n_tiles, n_tiles2,
                                      p.band, BN, kTileM);
      const bool second = c.group >= p.num_groups;
      __nv_bfloat16* const out_base = second ? p.out2 : p.out;
      const int out_ld = second ? p.ldo2 : p.ldo;
      const int out_cols = second ? p.out_cols2 : p.out_cols;
      const uint32_t acc = tcount & 1u;
      const uint32_t acc_ph = (tcount >> 1) & 1u;
      const int r = c.m0 + static_cast<int>(crank) * kBlockM + quarter * 32 + lane;
      bool row_ok = r < c.row_end;
      int orow = 0;
      if constexpr (kStore) {
        orow = row_ok ? (p.row_map ? p.row_map[r] : r) : 0;
        if (kChecks && row_ok && p.row_map && p.out_rows > 0 && !index_ok(orow, p.out_rows, p.status)) {
          row_ok = false;   // checking build: a row whose destination is out of range is not stored
          orow = 0;
        }
      } else {
        orow = row_ok ? r : 0;
      }
      // destination row addresses when rows are pushed to arbitrary (peer) memory
      const bool use_ptrs = kStore && p.out_row_ptrs != nullptr;
      long long my_ptr = 0;
      if (use_ptrs) {
        my_ptr = row_ok ? p.out_row_ptrs[r] : 0;
        if (kChecks && row_ok && !row_address_ok(my_ptr, p.status)) row_ok = false;
      }
      // destination rows in the coalesced mapping: it * 4 + lane / 8
      int crow[8];
      uint32_t cvalid = 0;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        crow[it] = __shfl_sync(0xffffffffu, orow, it * 4 + crow_l);
        cvalid |= (__shfl_sync(0xffffffffu, row_ok ? 1 : 0, it * 4 + crow_l) ? 1u : 0u) << it;
      }
      long long cptr[8];
      if (use_ptrs) {
        const long long mine = my_ptr;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const unsigned lo = __shfl_sync(0xffffffffu, static_cast<unsigned>(mine), it * 4 + crow_l);
          const unsigned hi = __shfl_sync(0xffffffffu, static_cast<unsigned>(mine >> 32), it * 4 + crow_l);
          cptr[it] = static_cast<long long>((static_cast<unsigned long long>(hi) << 32) | lo);
        }
      }
      // output columns of this tile and the number of sub-tiles (64 columns; 32 for the split
      // store, whose staged rows hold 64 bytes of high parts followed by 64 bytes of low parts)
      constexpr int kSubCols = kSplit ? 32 : kEpiCols;
      // cluster split-K: this CTA finishes only its slice of the tile's columns
      const int sk_col_lo = csk ? sp * (BN / splits) : 0;
      const int ocol_base = (kStore ? c.n0 : c.n0 / 2) + sk_col_lo;
      const int ocol_span = csk ? BN / splits : (kStore ? BN : BN / 2);
      const int ocols = min(ocol_span, out_cols - ocol_base);
      const int nsub = (ocols + kSubCols - 1) / kSubCols;
      const int col_end = ocol_base + ocols;   // one past the last output column of this tile
      const bool has_res = kStore && p.residual != nullptr;

      // i-th sub-tile of THIS warp (sub-tile index ehalf + i * kEpiHalves of the tile)
      auto fetch_residual = [&](int i) {
        uint8_t* buf = stage0 + (i & 1) * kEpiStageBytes;
        // split store: chunks 0-3 of a staged row come from the high part, 4-7 from the low part
        const __nv_bfloat16* src = (kSplit && cchunk >= 4) ? p.residual_lo : p.residual;
        const int col = ocol_base + (ehalf + i * kEpiHalves) * kSubCols +
                        (kSplit ? (cchunk & 3) : cchunk) * 8;
        if (col < col_end && src != nullptr) {
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            if ((cvalid >> it) & 1u) {
              const int rr = it * 4 + crow_l;
              cp_async_16(buf + rr * 128 + ((cchunk ^ (rr & 7)) << 4),
                          src + static_cast<long long>(crow[it]) * p.ldr + col);
            }
          }
        }
        cp_async_commit();
      };
      if (splits == 1 && has_res && ehalf < nsub) {
        fetch_residual(0);
        if (ehalf + kEpiHalves < nsub) fetch_residual(1);
      }
      const __nv_bfloat16* res2_row = nullptr;
      if constexpr (kStore) {
        if (p.residual2 && row_ok) {
          // read lane-per-row (uncoalesced): pull the row's bytes into L2 ahead of time
          res2_row = p.residual2 + static_cast<long long>(r) * p.ldr2;
          for (int cc = 0; cc < ocols; cc += 64) prefetch_l2(res2_row + ocol_base + cc);
        }
      }

      if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag, wait_limit)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kAccCols;

      // split-K: hand this CTA's partial tile over; only the CTA that arrives last goes on
      const float* sk_row = nullptr;    // this lane's row in partial 0 of the tile (last CTA only)
      uint32_t sk_part = 0;             // cluster form: shared-memory address of this lane's partial row
      constexpr uint32_t kPartMask = (BN / 4 - 1) & 31;   // 16-byte chunks of a row are XOR-swizzled by row
      if (csk) {
        // this thread's accumulator row, all BN columns, to the start of the (now idle) tile ring
        const uint32_t prow = static_cast<uint32_t>(quarter * 32 + lane);
        sk_part = smem_u32(smem) + prow * (BN * 4);
#pragma unroll 1
        for (int cc = 0; cc < BN / 32; ++cc) {
          uint32_t v[32];
          tmem_ld32(t_row + cc * 32, v);
          if constexpr (kChains == 2) {
            uint32_t v2[32];
            tmem_ld32(t_row + BN + cc * 32, v2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
          }
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t chunk = static_cast<uint32_t>(cc * 8 + q);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                             sk_part + ((chunk ^ (prow & kPartMask)) << 4)),
                         "r"(v[4 * q]), "r"(v[4 * q + 1]), "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                         : "memory");
          }
        }
        fence_acq_rel_cluster();
        __syncwarp();
        if (lane == 0) {
          for (int q = 0; q < splits; ++q)
            mbar_arrive_cluster(map_to_cta(smem_u32(sk_bar), static_cast<uint32_t>(q)));
        }
        if (!mbar_wait_cluster(sk_bar, 0, abort_flag, wait_limit)) {
          ok = false;
          break;
        }
        fence_acq_rel_cluster();
        {
          // Sum this CTA's column slice over the partial tiles of the cluster, in rank order, and
          // leave the sums in place of the slice in this CTA's own partial tile (nobody else
          // reads those columns of it).  Remote shared memory is read in whole 128-byte row
          // pieces: `cpr` lanes cover the slice of one row, a warp instruction covers 32 / cpr
          // rows (a lane-per-row pattern costs 32 remote transactions per instruction: 7 us).
          // 16-byte chunks per row slice: 8 or 16
          const uint32_t cpr = kClusterSplitK ? (static_cast<uint32_t>(BN / splits) >> 2) : 8u;
          const uint32_t rpl = 32u / cpr;
          const uint32_t chunk = (static_cast<uint32_t>(sk_col_lo) >> 2) + (static_cast<uint32_t>(lane) % cpr);
          const uint32_t ring = smem_u32(smem);
          // two row groups per round, so eight remote loads are in flight before the first is used
          for (uint32_t it = 0; it < 32u / rpl; it += 2) {
            uint32_t addr[2];
            float4 f[2][4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t row = static_cast<uint32_t>(quarter * 32) + (it + h) * rpl + static_cast<uint32_t>(lane) / cpr;
              addr[h] = ring + row * (BN * 4) + ((chunk ^ (row & kPartMask)) << 4);
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (q < splits) f[h][q] = ld_shared_cluster_f4(map_to_cta(addr[h], static_cast<uint32_t>(q)));
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              float4 a = f[h][0];
#pragma unroll
              for (int q = 1; q < 4; ++q)
                if (q < splits) { a.x += f[h][q].x; a.y += f[h][q].y; a.z += f[h][q].z; a.w += f[h][q].w; }
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr[h]), "f"(a.x), "f"(a.y),
                           "f"(a.z), "f"(a.w)
                           : "memory");
            }
          }
          __syncwarp();
        }
        if (has_res && ehalf < nsub) {
          fetch_residual(0);
          if (ehalf + kEpiHalves < nsub) fetch_residual(1);
        }
      } else if (splits > 1) {
        constexpr int kTileFloats = kBlockM * BN;
        float* mine = p.sk_scratch + (static_cast<size_t>(t) * splits + sp) * kTileFloats +
                      (quarter * 32 + lane) * BN;
#pragma unroll 1
        for (int cc = 0; cc < BN / 32; ++cc) {
          if (((cc >> 1) % kEpiHalves) != ehalf) continue;
          uint32_t v[32];
          tmem_ld32(t_row + cc * 32, v);
          if constexpr (kChains == 2) {
            uint32_t v2[32];
            tmem_ld32(t_row + BN + cc * 32, v2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
          }
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            *reinterpret_cast<uint4*>(mine + cc * 32 + q * 4) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        }
        __threadfence();
        volatile int* sk_flag = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 8);
        // barrier of the epilogue warps on a shared-memory counter; like every wait of this
        // kernel it gives up when another role has raised the abort flag (a named barrier would
        // wait forever for a warp that left its loop)
        auto epi_sync = [&]() {
          __syncwarp();
          if (lane == 0) atomicAdd(sk_arrivals, 1);
          sk_target += EW;
          while (*reinterpret_cast<volatile int*>(sk_arrivals) < sk_target) {
            if (*abort_flag) { ok = false; break; }
          }
          __syncwarp();
        };
        epi_sync();
        if (warp == 2 && lane == 0) {
          const int old = atomicAdd(p.sk_counters + t, 1);
          __threadfence();                    // the other CTAs' partials are visible before they are read
          const int last = (old == splits - 1) ? 1 : 0;
          if (last) p.sk_counters[t] = 0;     // every other CTA of the tile has counted: ready for the next launch
          *sk_flag = last;
        }
        epi_sync();
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const bool sk_last = *sk_flag != 0;
        if (!sk_last) {                     // not the last: the accumulator is free again, next unit
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
          continue;
        }
        __threadfence();
        sk_row = p.sk_scratch + static_cast<size_t>(t) * splits * kTileFloats + (quarter * 32 + lane) * BN;
        if (has_res && ehalf < nsub) {
          fetch_residual(0);
          if (ehalf + kEpiHalves < nsub) fetch_residual(1);
        }
      }
      // the accumulator values of 32 columns starting at `col`, summed over the partial tiles
      auto sk_sum = [&](int col, uint32_t (&v)[32]) {
        float a[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) a[j] = 0.f;
        if (csk) {
          // 32 columns of this CTA's slice, already summed over the cluster (see above)
          const uint32_t prow = static_cast<uint32_t>(quarter * 32 + lane);
          const uint32_t chunk0 = static_cast<uint32_t>(sk_col_lo + col) >> 2;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            float4 f;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(f.x), "=f"(f.y), "=f"(f.z), "=f"(f.w)
                         : "r"(sk_part + (((chunk0 + q) ^ (prow & kPartMask)) << 4))
                         : "memory");
            a[4 * q] = f.x; a[4 * q + 1] = f.y; a[4 * q + 2] = f.z; a[4 * q + 3] = f.w;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(a[j]);
          return;
        }
        for (int sidx = 0; sidx < splits; ++sidx) {
          const float4* src = reinterpret_cast<const float4*>(sk_row + static_cast<size_t>(sidx) * (kBlockM * BN) + col);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 f = __ldcg(src + q);
            a[4 * q] += f.x; a[4 * q + 1] += f.y; a[4 * q + 2] += f.z; a[4 * q + 3] += f.w;
          }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(a[j]);
      };

      // coalesced copy-out of one staged 32 x 64 sub-tile: 4 rows x 128 bytes per warp instruction
      auto copy_out = [&](const uint8_t* buf, int col0) {
        // split store: lanes with chunks 0-3 write the high parts to `out`, 4-7 the low parts to
        // `out_lo` (64 bytes per row and destination)
        __nv_bfloat16* base = (kSplit && cchunk >= 4) ? p.out_lo : out_base;
        const int col = col0 + (kSplit ? (cchunk & 3) : cchunk) * 8;
        if (col < col_end && (use_ptrs || base != nullptr)) {
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            if ((cvalid >> it) & 1u) {
              const int rr = it * 4 + crow_l;
              const uint4 o = *reinterpret_cast<const uint4*>(buf + rr * 128 + ((cchunk ^ (rr & 7)) << 4));
              __nv_bfloat16* drow = use_ptrs ? reinterpret_cast<__nv_bfloat16*>(cptr[it])
                                             : base + static_cast<long long>(crow[it]) * out_ld;
              *reinterpret_cast<uint4*>(drow + col) = o;
            }
          }
        }
      };

      bool rope_tile = false;
      if constexpr (EPI == kEpiStoreRope && BN == 256) {
        rope_tile = p.rope_cos != nullptr && c.n0 < p.rope_cols;
      }
      if (rope_tile) {
        if constexpr (EPI == kEpiStoreRope && BN == 256) {
          // Q/K RMSNorm + RoPE on the fp32 accumulators (reference: attention.py:138-155): the
          // tile holds two heads of 128 columns; a thread owns a row, so the norm is a plain
          // per-thread sum and rotate-half pairs column j with j + 64 of the same thread.
          const int pos = p.rope_pos0 + (row_ok ? r % p.rope_S : 0);
          const float* cs = p.rope_cos + static_cast<size_t>(pos) * 128;
          const float* sn = p.rope_sin + static_cast<size_t>(pos) * 128;
          uint8_t* buf_a = stage0;                    // columns [0, 64) of the head
          uint8_t* buf_b = stage0 + kEpiStageBytes;   // columns [64, 128)
#pragma unroll 1
          for (int hh = 0; hh < 2; ++hh) {
            const int hcol = c.n0 + hh * 128;
            if (hcol >= col_end) break;               // uniform
            const __nv_bfloat16* nw = (hcol < p.rope_q_cols) ? p.rope_qw : p.rope_kw;
            float rstd = 1.0f;
            if (nw) {
              float ss = 0.f;
#pragma unroll 1
              for (int cch = 0; cch < 4; ++cch) {
                uint32_t v[32];
                tmem_ld32(t_row + hh * 128 + cch * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) ss += __uint_as_float(v[j]) * __uint_as_float(v[j]);
              }
              rstd = rsqrtf(ss * (1.0f / 128.0f) + p.rope_eps);
            }
#pragma unroll 1
            for (int cch = 0; cch < 2; ++cch) {
              uint32_t a[32], b[32];
              tmem_ld32(t_row + hh * 128 + cch * 32, a);
              tmem_ld32(t_row + hh * 128 + 64 + cch * 32, b);
              tmem_ld_wait();
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int j0 = cch * 32 + q * 8;
                float w1[8], w2[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) w1[e] = w2[e] = rstd;
                if (nw) {
                  const uint4 wa = *reinterpret_cast<const uint4*>(nw + j0);
                  const uint4 wb = *reinterpret_cast<const uint4*>(nw + 64 + j0);
                  const uint32_t wwa[4] = {wa.x, wa.y, wa.z, wa.w}, wwb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    w1[2 * e] *= bf16_lo(wwa[e]); w1[2 * e + 1] *= bf16_hi(wwa[e]);
                    w2[2 * e] *= bf16_lo(wwb[e]); w2[2 * e + 1] *= bf16_hi(wwb[e]);
                  }
                }
                float o1[8], o2[8];
#pragma unroll
                for (int v4 = 0; v4 < 2; ++v4) {
                  const float4 ca = __ldg(reinterpret_cast<const float4*>(cs + j0) + v4);
                  const float4 sa = __ldg(reinterpret_cast<const float4*>(sn + j0) + v4);
                  const float4 cb = __ldg(reinterpret_cast<const float4*>(cs + 64 + j0) + v4);
                  const float4 sb = __ldg(reinterpret_cast<const float4*>(sn + 64 + j0) + v4);
                  const float cav[4] = {ca.x, ca.y, ca.z, ca.w}, sav[4] = {sa.x, sa.y, sa.z, sa.w};
                  const float cbv[4] = {cb.x, cb.y, cb.z, cb.w}, sbv[4] = {sb.x, sb.y, sb.z, sb.w};
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const int e = v4 * 4 + i;
                    const float x1 = __uint_as_float(a[q * 8 + e]) * w1[e];
                    const float x2 = __uint_as_float(b[q * 8 + e]) * w2[e];
                    o1[e] = x1 * cav[i] - x2 * sav[i];   // x cos + rotate_half(x) sin, first half
                    o2[e] = x2 * cbv[i] + x1 * sbv[i];   // second half
                  }
                }
                uint4 oa, ob;
                oa.x = pack_bf16x2(o1[0], o1[1]); oa.y = pack_bf16x2(o1[2], o1[3]);
                oa.z = pack_bf16x2(o1[4], o1[5]); oa.w = pack_bf16x2(o1[6], o1[7]);
                ob.x = pack_bf16x2(o2[0], o2[1]); ob.y = pack_bf16x2(o2[2], o2[3]);
                ob.z = pack_bf16x2(o2[4], o2[5]); ob.w = pack_bf16x2(o2[6], o2[7]);
                const uint32_t slot = own_off + (((cch * 4 + q) ^ (lane & 7)) << 4);
                *reinterpret_cast<uint4*>(buf_a + slot) = oa;
                *reinterpret_cast<uint4*>(buf_b + slot) = ob;
              }
            }
            __syncwarp();
            copy_out(buf_a, hcol);
            copy_out(buf_b, hcol + 64);
            __syncwarp();
          }
        }
      } else {
#pragma unroll 1
      for (int i = 0, sub = ehalf; sub < nsub; ++i, sub += kEpiHalves) {
        uint8_t* buf = stage0 + (i & 1) * kEpiStageBytes;
        const int col0 = ocol_base + sub * kSubCols;
        if constexpr (kSplit) {
          // one round of 32 accumulator columns: v = acc + bias + residual (high + low) + residual2,
          // stored as hi = bf16(v) and lo = bf16(v - hi)
          uint4 r2[4];
          if (res2_row) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (col0 + q * 8 < col_end) r2[q] = ld_nc_v4(res2_row + col0 + q * 8);
          }
          uint4 bb[4];
          if (p.bias) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (col0 + q * 8 < col_end) bb[q] = *reinterpret_cast<const uint4*>(p.bias + col0 + q * 8);
          }
          uint32_t v[32];
          tmem_ld32(t_row + sub * 32, v);
          if constexpr (kChains == 2) {
            uint32_t v2[32];
            tmem_ld32(t_row + BN + sub * 32, v2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
          }
          if (has_res) {
            if (sub + kEpiHalves < nsub) cp_async_wait<1>(); else cp_async_wait<0>();
            __syncwarp();
          }
          tmem_ld_wait();
          if (sk_row || csk) sk_sum(sub * 32, v);
          const bool has_lo = p.residual_lo != nullptr;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int col = col0 + q * 8;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[q * 8 + j]);
            uint8_t* slot_hi = buf + own_off + ((q ^ (lane & 7)) << 4);
            uint8_t* slot_lo = buf + own_off + (((4 + q) ^ (lane & 7)) << 4);
            if (col < col_end) {
              if (p.bias) {
                const uint32_t bw[4] = {bb[q].x, bb[q].y, bb[q].z, bb[q].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  f[2 * j] += fminf(fmaxf(bf16_lo(bw[j]), p.bias_lo), p.bias_hi);
                  f[2 * j + 1] += fminf(fmaxf(bf16_hi(bw[j]), p.bias_lo), p.bias_hi);
                }
              }
              if (has_res && row_ok) {
                const uint4 rr = *reinterpret_cast<const uint4*>(slot_hi);
                const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  f[2 * j] += bf16_lo(rw[j]);
                  f[2 * j + 1] += bf16_hi(rw[j]);
                }
                if (has_lo) {
                  const uint4 rl = *reinterpret_cast<const uint4*>(slot_lo);
                  const uint32_t lw[4] = {rl.x, rl.y, rl.z, rl.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    f[2 * j] += bf16_lo(lw[j]);
                    f[2 * j + 1] += bf16_hi(lw[j]);
                  }
                }
              }
              if (res2_row) {
                const uint32_t rw[4] = {r2[q].x, r2[q].y, r2[q].z, r2[q].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  f[2 * j] += bf16_lo(rw[j]);
                  f[2 * j + 1] += bf16_hi(rw[j]);
                }
              }
              if (p.do_clamp) {
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = fminf(fmaxf(f[j], p.clamp_lo), p.clamp_hi);
              }
            }
            uint4 o, l;
            o.x = pack_bf16x2(f[0], f[1]);
            o.y = pack_bf16x2(f[2], f[3]);
            o.z = pack_bf16x2(f[4], f[5]);
            o.w = pack_bf16x2(f[6], f[7]);
            l.x = pack_bf16x2(f[0] - bf16_lo(o.x), f[1] - bf16_hi(o.x));
            l.y = pack_bf16x2(f[2] - bf16_lo(o.y), f[3] - bf16_hi(o.y));
            l.z = pack_bf16x2(f[4] - bf16_lo(o.z), f[5] - bf16_hi(o.z));
            l.w = pack_bf16x2(f[6] - bf16_lo(o.w), f[7] - bf16_hi(o.w));
            *reinterpret_cast<uint4*>(slot_hi) = o;
            *reinterpret_cast<uint4*>(slot_lo) = l;
          }
        } else if constexpr (kStore) {
          // two rounds of 32 accumulator columns (keeps the register count of the
          // eight-warp variants inside their budget)
#pragma unroll 1
          for (int hh = 0; hh < 2; ++hh) {
            const int colh = col0 + hh * 32;
            if (colh >= col_end) break;   // uniform: nothing of this round is stored
            uint4 r2[4];
            if (res2_row) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (colh + q * 8 < col_end) r2[q] = ld_nc_v4(res2_row + colh + q * 8);
            }
            uint4 bb[4];
            if (p.bias) {   // same for every row: issued before the TMEM loads, L1 hits
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (colh + q * 8 < col_end) bb[q] = *reinterpret_cast<const uint4*>(p.bias + colh + q * 8);
            }
            uint32_t v[32];
            tmem_ld32(t_row + sub * 64 + hh * 32, v);
            if constexpr (kChains == 2) {
              uint32_t v2[32];
              tmem_ld32(t_row + BN + sub * 64 + hh * 32, v2);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
            }
            if (has_res && hh == 0) {
              if (sub + kEpiHalves < nsub) cp_async_wait<1>(); else cp_async_wait<0>();
              __syncwarp();
            }
            tmem_ld_wait();
            if (sk_row || csk) sk_sum(sub * 64 + hh * 32, v);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int col = colh + q * 8;
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(v[q * 8 + j]);
              uint8_t* slot = buf + own_off + (((hh * 4 + q) ^ (lane & 7)) << 4);
              if (col < col_end) {
                if (p.bias) {
                  const uint32_t bw[4] = {bb[q].x, bb[q].y, bb[q].z, bb[q].w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    f[2 * j] += fminf(fmaxf(bf16_lo(bw[j]), p.bias_lo), p.bias_hi);
                    f[2 * j + 1] += fminf(fmaxf(bf16_hi(bw[j]), p.bias_lo), p.bias_hi);
                  }
                }
                if (has_res && row_ok) {
                  const uint4 rr = *reinterpret_cast<const uint4*>(slot);
                  const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    f[2 * j] += bf16_lo(rw[j]);
                    f[2 * j + 1] += bf16_hi(rw[j]);
                  }
                }
                if (res2_row) {
                  const uint32_t rw[4] = {r2[q].x, r2[q].y, r2[q].z, r2[q].w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    f[2 * j] += bf16_lo(rw[j]);
                    f[2 * j + 1] += bf16_hi(rw[j]);
                  }
                }
                if (p.do_clamp) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) f[j] = fminf(fmaxf(f[j], p.clamp_lo), p.clamp_hi);
                }
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]);
              o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]);
              o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(slot) = o;
            }
          }
        } else {
          // SwiGLU: accumulator columns [0, BN/2) hold gate, [BN/2, BN) hold up, for output
          // columns (n0 / 2) .. (n0 / 2) + BN / 2; 32 output columns per TMEM round trip.
          // narrow tiles (BN / 2 <= 32 output columns) need a single round trip; columns read
          // past the tile's own are never stored
          constexpr int kRounds = (BN / 2 > 32) ? 2 : 1;
#pragma unroll
          for (int half = 0; half < kRounds; ++half) {
            uint32_t g[32], u[32];
            tmem_ld32(t_row + sub * 64 + half * 32, g);
            tmem_ld32(t_row + BN / 2 + sub * 64 + half * 32, u);
            if constexpr (kChains == 2) {
              uint32_t g2[32], u2[32];
              tmem_ld32(t_row + BN + sub * 64 + half * 32, g2);
              tmem_ld32(t_row + BN + BN / 2 + sub * 64 + half * 32, u2);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                g[j] = __float_as_uint(__uint_as_float(g[j]) + __uint_as_float(g2[j]));
                u[j] = __float_as_uint(__uint_as_float(u[j]) + __uint_as_float(u2[j]));
              }
            }
            tmem_ld_wait();
            if (sk_row) {
              sk_sum(sub * 64 + half * 32, g);
              sk_sum(BN / 2 + sub * 64 + half * 32, u);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float h[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                h[j] = silu_f(__uint_as_float(g[q * 8 + j])) * __uint_as_float(u[q * 8 + j]);
              uint4 o;
              o.x = pack_bf16x2(h[0], h[1]);
              o.y = pack_bf16x2(h[2], h[3]);
              o.z = pack_bf16x2(h[4], h[5]);
              o.w = pack_bf16x2(h[6], h[7]);
              *reinterpret_cast<uint4*>(buf + own_off + (((half * 4 + q) ^ (lane & 7)) << 4)) = o;
            }
          }
        }
        __syncwarp();
        copy_out(buf, col0);
        __syncwarp();  // the buffer may be refilled from here on
        if (has_res && sub + 2 * kEpiHalves < nsub) fetch_residual(i + 2);
      }
      }  // plain tiles
      // this warp is done reading the accumulator
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 2)
          mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));  // the leader's barrier
        else
          mbar_arrive(&tmem_empty[acc]);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();  // the leader's MMAs read the peer's memory until here
  else if (csk) cluster_sync_all();           // the cluster's CTAs read each other's partial tiles until here
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if constexpr (CG == 2) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

}  // namespace cdeep
