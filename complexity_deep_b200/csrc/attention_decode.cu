// Single-query (decode) attention over a KV cache, HBM-bound: every cached K and V row is
// read exactly once, straight from the cache's own layout, for all the query heads that
// share it (grouped-query attention without repeating the KV heads).
//
// Replaces, for q_len == 1, complexity_deep/core/attention.py:163-177 (repeat_interleave of
// K/V + scaled_dot_product_attention): out[b, h] = softmax(q[b, h] . K[b, h / G]^T * scale
// + mask[b]) V[b, h / G].
//
// Split-KV: grid (splits, kv heads, batch); a block owns one chunk of the cache for one
// (batch, kv head) and all G query heads of the group.  8 lanes share a cached row: for
// every 64 dimensions lane s owns dimensions 8 s .. 8 s + 7, so one 16-byte access per lane
// covers 128 contiguous bytes of the row (whole sectors, no re-fetch); a warp streams 4 rows
// per step; every lane group
// keeps an online-softmax state (running max, sum, weighted V) per query head, merged across
// the block through shared memory and across splits by a second small kernel.
#include <cfloat>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "kernels.h"

namespace cdeep {

namespace {

constexpr int kAttnThreads = 128;
constexpr int kMaxGroup = 4;    // query heads per KV head handled by one block (the entry point refuses more)
constexpr int kLanesPerRow = 8;

__device__ __forceinline__ float lo_f(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi_f(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Blocks per (batch, kv head) pair.  Also evaluated on the device when the cache length is
// read from device memory, so both forms split (and therefore round) identically.
// kTargetBlocks is a tuning constant (16 blocks for each of a B200's 148 SMs), not a limit: any
// other SM count only changes how many blocks share the work.
constexpr int kTargetBlocks = 16 * 148;
__host__ __device__ inline int choose_splits(int B, int hkv, int L) {
  const int pairs = B * hkv;
  int splits = (kTargetBlocks + pairs - 1) / pairs;   // several waves of blocks: small tail
  // at least 512 rows per block (measured against 128 and 256: 10-15 % faster for short
  // caches and few sequences, equal elsewhere)
  const int max_splits = (L + 511) / 512;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  return splits;
}

__host__ __device__ inline int chunk_rows(int L, int splits) {
  return (((L + splits - 1) / splits) + 15) / 16 * 16;
}

// programmatic dependent launch: wait for the previous kernel of the stream before touching
// memory, then let the next kernel be scheduled (its launch hides under this one)
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kStages = 4;   // row steps staged in shared memory per thread (3 in flight)

// DPL = dimensions per lane = D / 8 (8 or 16 -> D = 64 or 128), G = query heads per KV head.
// len_dev (optional): the number of cached rows is min(L, *len_dev) and the split of the rows
// over blocks is recomputed from it; the grid and the workspace layout stay those of L.
//
// A row step = 16 cached rows of the block (4 warps x 4 lane groups), 2 * DPL bytes of K and
// of V per lane.  Every lane copies its own slices of the next kStages - 1 steps into a
// private slot of shared memory with cp.async (bytes in flight without holding registers:
// 4 blocks per SM keep ~100 KB on the way) and reads them back with 16-byte loads, so no
// block-level synchronisation is needed inside the loop.
template <int DPL, int G>
__global__ void __launch_bounds__(kAttnThreads, (G * DPL > 48) ? 2 : (G * DPL > 32) ? 3 : 4)
decode_attn_partial_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride_b,
                           const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                           long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                           const __nv_bfloat16* __restrict__ mask, long long mask_stride_b,
                           float scale, int L, int chunk, int hq, float* __restrict__ part_acc,
                           float* __restrict__ part_ml, const int* __restrict__ len_dev) {
  constexpr int D = DPL * kLanesPerRow;
  constexpr int kV = DPL / 8;                               // 16-byte pieces of K (and of V) per lane
  constexpr int kStepBytes = kAttnThreads * 2 * kV * 16;    // one row step of the block
  constexpr int kMergeBytes = 16 * G * D * 4;               // the block-level merge re-uses the slots
  constexpr int kSmemBytes = kStages * kStepBytes > kMergeBytes ? kStages * kStepBytes : kMergeBytes;
  __shared__ __align__(16) unsigned char s_raw[kSmemBytes];
  __shared__ float s_m[16][G], s_l[16][G];

  griddep_wait();
  griddep_launch_dependents();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int splits = gridDim.x;
  if (len_dev) {
    L = max(0, min(L, __ldg(len_dev)));
    const int live = choose_splits(gridDim.z, gridDim.y, L);
    if (split >= live) return;       // whole block; the combine kernel skips these slots
    chunk = chunk_rows(L, live);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7;          // which D/8 slice of the row
  const int rgrp = lane >> 3;        // which of the warp's 4 concurrent rows
  const int t_begin = split * chunk;
  const int t_end = min(L, t_begin + chunk);

  // query fragments of the G heads, pre-scaled
  float qf[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const __nv_bfloat16* qp = q + b * q_stride_b + static_cast<long long>(kvh * G + g) * D + sub * 8;
#pragma unroll
    for (int i = 0; i < DPL; i += 8) {
      const uint4 w = *reinterpret_cast<const uint4*>(qp + i * 8);
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        qf[g][i + 2 * e] = lo_f(ww[e]) * scale;
        qf[g][i + 2 * e + 1] = hi_f(ww[e]) * scale;
      }
    }
  }
  float m_run[G], l_run[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -FLT_MAX;
    l_run[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i] = 0.f;
  }
  const __nv_bfloat16* kb = k + b * kv_stride_b + kvh * kv_stride_h + sub * 8;
  const __nv_bfloat16* vb = v + b * kv_stride_b + kvh * kv_stride_h + sub * 8;
  const __nv_bfloat16* mb = mask ? mask + b * mask_stride_b : nullptr;

  // slot of (stage, piece) for this thread: consecutive threads are 16 bytes apart, so both
  // the asynchronous writes and the reads are free of bank conflicts
  auto slot = [&](int stage, int piece) -> uint4* {
    return reinterpret_cast<uint4*>(s_raw + stage * kStepBytes) + piece * kAttnThreads + threadIdx.x;
  };
  const int t_lane = t_begin + warp * 4 + rgrp;             // this lane's row of step 0
  const int n_steps = (t_end - t_begin + 15) >> 4;          // same for the whole block
  auto issue = [&](int step) {
    const int t = t_lane + step * 16;
    if (step < n_steps && t < t_end) {
      const int stage = step % kStages;
#pragma unroll
      for (int i = 0; i < kV; ++i) {
        cp_async16(slot(stage, i), kb + t * kv_stride_t + i * 64);
        cp_async16(slot(stage, kV + i), vb + t * kv_stride_t + i * 64);
      }
    }
    cp_async_commit();                                      // one group per step, even if empty
  };
#pragma unroll
  for (int s0 = 0; s0 < kStages - 1; ++s0) issue(s0);

  // Additive mask: once per 8 steps lane l fetches the value of row group (l & 3) of step
  // (window + l / 4) of this warp, one window ahead of its use; a step then takes its value
  // from the owning lane with a shuffle, so no step waits for a global load.
  auto mask_window = [&](int step0) -> float {
    const int t = t_begin + 16 * (step0 + (lane >> 2)) + warp * 4 + (lane & 3);
    return (mb && t < t_end) ? __bfloat162float(mb[t]) : 0.f;
  };
  float mwin = mask_window(0), mwin_next = mask_window(8);

  for (int step = 0; step < n_steps; ++step) {
    issue(step + kStages - 1);
    float madd = 0.f;
    if (mb) {                                               // uniform
      const int j = step & 7;
      if (j == 0 && step > 0) {
        mwin = mwin_next;
        mwin_next = mask_window(step + 8);
      }
      madd = __shfl_sync(0xffffffffu, mwin, (j << 2) | rgrp);
    }
    cp_async_wait<kStages - 1>();                           // this step's group has landed
    const int t = t_lane + step * 16;
    const bool valid = t < t_end;
    const int stage = step % kStages;
    float kf[DPL], vf[DPL];
#pragma unroll
    for (int i = 0; i < kV; ++i) {
      uint4 kr = make_uint4(0, 0, 0, 0), vr = kr;
      if (valid) {
        kr = *slot(stage, i);
        vr = *slot(stage, kV + i);
      }
      const uint32_t kw[4] = {kr.x, kr.y, kr.z, kr.w};
      const uint32_t vw[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        kf[i * 8 + 2 * e] = lo_f(kw[e]); kf[i * 8 + 2 * e + 1] = hi_f(kw[e]);
        vf[i * 8 + 2 * e] = lo_f(vw[e]); vf[i * 8 + 2 * e + 1] = hi_f(vw[e]);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) s += qf[g][i] * kf[i];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (valid) {
        s += madd;
        if (s > m_run[g]) {            // new running maximum: rescale (rare after the first rows)
          const float corr = __expf(m_run[g] - s);
          l_run[g] *= corr;
#pragma unroll
          for (int i = 0; i < DPL; ++i) acc[g][i] *= corr;
          m_run[g] = s;
        }
        // s = -inf (masked) gives pr = 0 and leaves the state untouched
        const float pr = __expf(s - m_run[g]);
        l_run[g] += pr;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[g][i] += pr * vf[i];
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();                     // every lane is done with its slots: re-use them

  // merge the 16 row streams of the block (4 warps x 4 lane groups) in shared memory
  float (*s_acc)[G][D] = reinterpret_cast<float (*)[G][D]>(s_raw);
  const int stream = warp * 4 + rgrp;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (sub == 0) {
      s_m[stream][g] = m_run[g];
      s_l[stream][g] = l_run[g];
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) s_acc[stream][g][(i >> 3) * 64 + sub * 8 + (i & 7)] = acc[g][i];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += kAttnThreads) {
    const int g = idx / D, d = idx - g * D;
    float m = -FLT_MAX;
#pragma unroll
    for (int s = 0; s < 16; ++s) m = fmaxf(m, s_m[s][g]);
    float l = 0.f, a = 0.f;
#pragma unroll
    for (int s = 0; s < 16; ++s) {
      const float w = (s_m[s][g] > -FLT_MAX) ? __expf(s_m[s][g] - m) : 0.f;
      l += s_l[s][g] * w;
      a += s_acc[s][g][d] * w;
    }
    const long long row = (static_cast<long long>(b) * hq + kvh * G + g) * splits + split;
    part_acc[row * D + d] = a;
    if (d == 0) {
      part_ml[row * 2] = m;
      part_ml[row * 2 + 1] = l;
    }
  }
}

// out[b, h, :] = sum_s w_s acc_s / sum_s w_s l_s, w_s = exp(m_s - max m)
__global__ void __launch_bounds__(128)
decode_attn_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                           int splits, int D, __nv_bfloat16* __restrict__ out, int B, int hkv,
                           int L, const int* __restrict__ len_dev) {
  griddep_wait();
  griddep_launch_dependents();
  const long long row0 = static_cast<long long>(blockIdx.x) * splits;   // (b, h)
  if (len_dev) splits = choose_splits(B, hkv, max(0, min(L, __ldg(len_dev))));
  float m = -FLT_MAX;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(row0 + s) * 2]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float l = 0.f, a = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = part_ml[(row0 + s) * 2];
      const float w = (ms > -FLT_MAX) ? __expf(ms - m) : 0.f;
      l += part_ml[(row0 + s) * 2 + 1] * w;
      a += part_acc[(row0 + s) * D + d] * w;
    }
    out[static_cast<long long>(blockIdx.x) * D + d] = __float2bfloat16_rn(l > 0.f ? a / l : 0.f);
  }
}

template <int DPL>
cudaError_t launch_partial(int G, dim3 grid, cudaStream_t st, const __nv_bfloat16* q,
                           long long qsb, const __nv_bfloat16* k, const __nv_bfloat16* v,
                           long long sb, long long sh, long long stt, const __nv_bfloat16* mask,
                           long long msb, float scale, int L, int chunk, int hq, float* pa,
                           float* pml, const int* len_dev) {
#define CDEEP_ATTN_CASE(GG)                                                                     \
  case GG:                                                                                      \
    return launch_kernel(decode_attn_partial_kernel<DPL, GG>, grid, dim3(kAttnThreads), 0, st,  \
                         q, qsb, k, v, sb, sh, stt, mask, msb, scale, L, chunk, hq, pa, pml,    \
                         len_dev);
  switch (G) {
    CDEEP_ATTN_CASE(1)
    CDEEP_ATTN_CASE(2)
    CDEEP_ATTN_CASE(3)
    CDEEP_ATTN_CASE(4)
    default:
      return cudaErrorInvalidValue;
  }
#undef CDEEP_ATTN_CASE
  return cudaGetLastError();
}

}  // namespace

size_t decode_attention_workspace_bytes(int B, int hq, int hkv, int L, int D) {
  const size_t splits = choose_splits(B, hkv, L);
  return static_cast<size_t>(B) * hq * splits * (D + 2) * sizeof(float);
}

cudaError_t launch_decode_attention(const void* q, long long q_stride_b, const void* k,
                                    const void* v, long long kv_stride_b, long long kv_stride_h,
                                    long long kv_stride_t, const void* mask,
                                    long long mask_stride_b, float scale, int B, int hq, int hkv,
                                    int L, int D, void* out, void* ws, cudaStream_t stream,
                                    const int* kv_len_dev) {
  const int G = hq / hkv;
  const int splits = choose_splits(B, hkv, L);
  const int chunk = chunk_rows(L, splits);
  float* part_acc = static_cast<float*>(ws);
  float* part_ml = part_acc + static_cast<size_t>(B) * hq * splits * D;
  dim3 grid(splits, hkv, B);
  auto qb = static_cast<const __nv_bfloat16*>(q);
  auto kb = static_cast<const __nv_bfloat16*>(k);
  auto vb = static_cast<const __nv_bfloat16*>(v);
  auto mb = static_cast<const __nv_bfloat16*>(mask);
  cudaError_t e;
  if (D == 128)
    e = launch_partial<16>(G, grid, stream, qb, q_stride_b, kb, vb, kv_stride_b, kv_stride_h,
                           kv_stride_t, mb, mask_stride_b, scale, L, chunk, hq, part_acc, part_ml,
                           kv_len_dev);
  else if (D == 64)
    e = launch_partial<8>(G, grid, stream, qb, q_stride_b, kb, vb, kv_stride_b, kv_stride_h,
                          kv_stride_t, mb, mask_stride_b, scale, L, chunk, hq, part_acc, part_ml,
                           kv_len_dev);
  else
    return cudaErrorInvalidValue;
  if (e != cudaSuccess) return e;
  return launch_kernel(decode_attn_combine_kernel, dim3(B * hq), dim3(128), 0, stream, part_acc,
                       part_ml, splits, D, static_cast<__nv_bfloat16*>(out), B, hkv, L, kv_len_dev);
}

}  // namespace cdeep
