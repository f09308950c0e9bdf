// Single-query (decode) attention over a KV cache, HBM-bound: every cached K and V row is
// read exactly once, straight from the cache's own layout, for all the query heads that
// share it (grouped-query attention without repeating the KV heads).
//
// Replaces, for q_len == 1, complexity_deep/core/attention.py:163-177 (repeat_interleave of
// K/V + scaled_dot_product_attention): out[b, h] = softmax(q[b, h] . K[b, h / G]^T * scale
// + mask[b]) V[b, h / G].
//
// Split-KV: grid (splits, kv heads, batch); a block owns one chunk of the cache for one
// (batch, kv head) and all G query heads of the group.  8 lanes share a cached row (each
// owns D/8 dimensions, 16-byte loads), so a warp streams 4 rows per step; every lane group
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
constexpr int kMaxGroup = 8;    // query heads per KV head handled by one block
constexpr int kLanesPerRow = 8;

__device__ __forceinline__ float lo_f(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi_f(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Blocks per (batch, kv head) pair.  Also evaluated on the device when the cache length is
// read from device memory, so both forms split (and therefore round) identically.
__host__ __device__ inline int choose_splits(int B, int hkv, int L) {
  const int pairs = B * hkv;
  int splits = (16 * 148 + pairs - 1) / pairs;      // several waves of blocks: small tail
  const int max_splits = (L + 255) / 256;           // at least 256 rows per block
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  return splits;
}

__host__ __device__ inline int chunk_rows(int L, int splits) {
  return (((L + splits - 1) / splits) + 15) / 16 * 16;
}

// DPL = dimensions per lane = D / 8 (8 or 16 -> D = 64 or 128), G = query heads per KV head.
// len_dev (optional): the number of cached rows is min(L, *len_dev) and the split of the rows
// over blocks is recomputed from it; the grid and the workspace layout stay those of L.
template <int DPL, int G>
__global__ void __launch_bounds__(kAttnThreads)
decode_attn_partial_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride_b,
                           const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                           long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                           const __nv_bfloat16* __restrict__ mask, long long mask_stride_b,
                           float scale, int L, int chunk, int hq, float* __restrict__ part_acc,
                           float* __restrict__ part_ml, const int* __restrict__ len_dev) {
  constexpr int D = DPL * kLanesPerRow;
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
    const __nv_bfloat16* qp = q + b * q_stride_b + static_cast<long long>(kvh * G + g) * D + sub * DPL;
#pragma unroll
    for (int i = 0; i < DPL; i += 8) {
      const uint4 w = *reinterpret_cast<const uint4*>(qp + i);
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
  const __nv_bfloat16* kb = k + b * kv_stride_b + kvh * kv_stride_h + sub * DPL;
  const __nv_bfloat16* vb = v + b * kv_stride_b + kvh * kv_stride_h + sub * DPL;
  const __nv_bfloat16* mb = mask ? mask + b * mask_stride_b : nullptr;

  // Rows of this block: t_begin + 16 * i + (warp * 4 + rgrp), two steps (rows t and t + 16) per
  // iteration; the loads of the next iteration are issued before the arithmetic of the current
  // one, so 8 x 16 bytes per lane are in flight.  The loop bound is the same for every lane of
  // a warp (the shuffles need the whole warp).
  constexpr int kV = DPL / 8;
  uint4 kn[2][kV], vn[2][kV];
  auto load_rows = [&](int t, int s) {
#pragma unroll
    for (int i = 0; i < kV; ++i) {
      kn[s][i] = make_uint4(0, 0, 0, 0);
      vn[s][i] = make_uint4(0, 0, 0, 0);
      if (t < t_end) {
        kn[s][i] = *reinterpret_cast<const uint4*>(kb + t * kv_stride_t + i * 8);
        vn[s][i] = *reinterpret_cast<const uint4*>(vb + t * kv_stride_t + i * 8);
      }
    }
  };
  auto process = [&](const uint4 (&kr)[kV], const uint4 (&vr)[kV], int t) {
    const bool valid = t < t_end;
    float kf[DPL], vf[DPL];
#pragma unroll
    for (int i = 0; i < kV; ++i) {
      const uint32_t kw[4] = {kr[i].x, kr[i].y, kr[i].z, kr[i].w};
      const uint32_t vw[4] = {vr[i].x, vr[i].y, vr[i].z, vr[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        kf[i * 8 + 2 * e] = lo_f(kw[e]); kf[i * 8 + 2 * e + 1] = hi_f(kw[e]);
        vf[i * 8 + 2 * e] = lo_f(vw[e]); vf[i * 8 + 2 * e + 1] = hi_f(vw[e]);
      }
    }
    const float madd = (valid && mb) ? __bfloat162float(mb[t]) : 0.f;
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
        const float m_new = fmaxf(m_run[g], s);
        // a fully masked prefix (-inf scores) keeps the state untouched
        if (m_new > -FLT_MAX) {
          const float corr = __expf(m_run[g] - m_new);
          const float pr = __expf(s - m_new);
          l_run[g] = l_run[g] * corr + pr;
#pragma unroll
          for (int i = 0; i < DPL; ++i) acc[g][i] = acc[g][i] * corr + pr * vf[i];
          m_run[g] = m_new;
        }
      }
    }
  };
  const int t_first = t_begin + warp * 4 + rgrp;
  load_rows(t_first, 0);
  load_rows(t_first + 16, 1);
  for (int tb = t_begin + warp * 4; tb < t_end; tb += 32) {
    const int t = tb + rgrp;
    uint4 k0[kV], v0[kV], k1[kV], v1[kV];
#pragma unroll
    for (int i = 0; i < kV; ++i) {
      k0[i] = kn[0][i]; v0[i] = vn[0][i];
      k1[i] = kn[1][i]; v1[i] = vn[1][i];
    }
    load_rows(t + 32, 0);
    load_rows(t + 48, 1);
    process(k0, v0, t);
    process(k1, v1, t + 16);
  }

  // merge the 16 row streams of the block (4 warps x 4 lane groups) in shared memory
  __shared__ float s_m[16][G], s_l[16][G];
  __shared__ float s_acc[16][G][D];
  const int stream = warp * 4 + rgrp;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (sub == 0) {
      s_m[stream][g] = m_run[g];
      s_l[stream][g] = l_run[g];
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) s_acc[stream][g][sub * DPL + i] = acc[g][i];
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
    decode_attn_partial_kernel<DPL, GG><<<grid, kAttnThreads, 0, st>>>(                         \
        q, qsb, k, v, sb, sh, stt, mask, msb, scale, L, chunk, hq, pa, pml, len_dev);                    \
    break;
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
  decode_attn_combine_kernel<<<B * hq, 128, 0, stream>>>(part_acc, part_ml, splits, D,
                                                        static_cast<__nv_bfloat16*>(out), B, hkv,
                                                        L, kv_len_dev);
  return cudaGetLastError();
}

}  // namespace cdeep
