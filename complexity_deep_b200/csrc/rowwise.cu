// Row-wise, HBM-bound kernels of the block: RMSNorm (optionally fused with the residual add
// before it and with the scatter of rows into expert-sorted order after it), the row
// gather used when the MoE layer is called on its own, and the per-head Q/K RMSNorm +
// rotary embedding applied in place on the fused QKV buffer.
//
// Reference semantics:
//   RMSNorm            complexity_deep/core/normalization.py:29-32  (w * x * rsqrt(mean(x^2) + eps))
//   residual add       complexity_deep/core/layer.py:174
//   Q/K norm, RoPE     complexity_deep/core/attention.py:138-155, complexity_deep/core/rotary.py:57-86
// The reference evaluates these in the activation dtype; here every reduction and product
// is fp32 and each output is rounded to bf16 once.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "checks.cuh"
#include "kernels.h"

namespace cdeep {

namespace {

// programmatic dependent launch (same two instructions as in ptx.cuh, which this file does
// not include): wait for the previous kernel of the stream, then let the next one be scheduled
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float lo_f(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi_f(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kNormWarps = 4;
constexpr int kMaxVec = 16;  // register path: H <= 16 * 256 = 4096, H % 256 == 0

// One warp per row; the row lives in registers between the reduction and the scaling, so
// x is read from HBM exactly once.  kSplit: `res` is the low part of a split-bf16 value
// (x + res carries 16 significant bits); the sum then stays in fp32 and nothing is written back.
// NV: uint4 per lane (H / 256) when known at compile time — the row then needs exactly NV (2 NV
// for a split row) 16-byte registers per lane, which keeps enough warps resident to cover HBM
// latency; NV = 0 is the generic form for any H <= 4096 with H % 256 == 0.
template <bool kSplit, int NV>
__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                    const __nv_bfloat16* __restrict__ w, float eps,
                    __nv_bfloat16* __restrict__ sum_out, __nv_bfloat16* __restrict__ out,
                    const int* __restrict__ dst_rows, int T, int H, int* status) {
  griddep_wait();               // the previous kernel's writes are visible from here
  griddep_launch_dependents();  // the next kernel may be scheduled
  const int row = blockIdx.x * kNormWarps + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  constexpr int kVec = NV ? NV : kMaxVec;
  const int nv = NV ? NV : (H >> 8);  // uint4 (8 bf16) per lane
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + static_cast<size_t>(row) * H)
                        : nullptr;
  uint4 buf[kVec];
  uint4 low[kSplit ? kVec : 1];
#pragma unroll
  for (int v = 0; v < kVec; ++v)
    if (v < nv) buf[v] = xr[v * 32 + lane];
  if constexpr (kSplit) {
#pragma unroll
    for (int v = 0; v < kVec; ++v)
      if (v < nv) low[v] = rr ? rr[v * 32 + lane] : make_uint4(0, 0, 0, 0);
  } else if (rr) {
#pragma unroll
    for (int v = 0; v < kVec; ++v)
      if (v < nv) {
        const uint4 r = rr[v * 32 + lane];
        uint32_t* a = reinterpret_cast<uint32_t*>(&buf[v]);
        const uint32_t b[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) a[j] = pack2(lo_f(a[j]) + lo_f(b[j]), hi_f(a[j]) + hi_f(b[j]));
      }
    if (sum_out) {
      uint4* so = reinterpret_cast<uint4*>(sum_out + static_cast<size_t>(row) * H);
#pragma unroll
      for (int v = 0; v < kVec; ++v)
        if (v < nv) so[v * 32 + lane] = buf[v];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < kVec; ++v)
    if (v < nv) {
      const uint32_t* a = reinterpret_cast<const uint32_t*>(&buf[v]);
      const uint32_t* b = reinterpret_cast<const uint32_t*>(&low[kSplit ? v : 0]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float l = lo_f(a[j]), h = hi_f(a[j]);
        if constexpr (kSplit) {
          l += lo_f(b[j]);
          h += hi_f(b[j]);
        }
        ss += l * l + h * h;
      }
    }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
  const int orow = dst_rows ? dst_rows[row] : row;
  if (kChecks && dst_rows && !index_ok(orow, T, status)) return;   // checking build: row not stored
  uint4* orw = reinterpret_cast<uint4*>(out + static_cast<size_t>(orow) * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int v = 0; v < kVec; ++v)
    if (v < nv) {
      const uint4 wv = wr[v * 32 + lane];
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
      const uint32_t* a = reinterpret_cast<const uint32_t*>(&buf[v]);
      const uint32_t* b = reinterpret_cast<const uint32_t*>(&low[kSplit ? v : 0]);
      uint4 o;
      uint32_t* oo = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float l = lo_f(a[j]), h = hi_f(a[j]);
        if constexpr (kSplit) {
          l += lo_f(b[j]);
          h += hi_f(b[j]);
        }
        oo[j] = pack2(lo_f(ww[j]) * (l * rstd), hi_f(ww[j]) * (h * rstd));
      }
      orw[v * 32 + lane] = o;
    }
}

// Any H: one block per row, scalar accesses, the row is re-read from L1/L2 for the scaling.
__global__ void __launch_bounds__(128)
rmsnorm_generic_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                       const __nv_bfloat16* __restrict__ w, float eps,
                       __nv_bfloat16* __restrict__ sum_out, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ dst_rows, int T, int H, int split, int* status) {
  griddep_wait();               // the previous kernel's writes are visible from here
  griddep_launch_dependents();  // the next kernel may be scheduled
  __shared__ float s_part[4];
  const int row = blockIdx.x;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
  const __nv_bfloat16* rr = res ? res + static_cast<size_t>(row) * H : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = __bfloat162float(xr[c]);
    if (rr && split) {
      v += __bfloat162float(rr[c]);
    } else if (rr) {
      const __nv_bfloat16 s = __float2bfloat16_rn(v + __bfloat162float(rr[c]));
      if (sum_out) sum_out[static_cast<size_t>(row) * H + c] = s;
      v = __bfloat162float(s);
    }
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float tot = s_part[0] + s_part[1] + s_part[2] + s_part[3];
  const float rstd = rsqrtf(tot / static_cast<float>(H) + eps);
  const int orow = dst_rows ? dst_rows[row] : row;
  if (kChecks && dst_rows && !index_ok(orow, T, status)) return;   // checking build: row not stored
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = __bfloat162float(xr[c]);
    if (rr && split) v += __bfloat162float(rr[c]);
    else if (rr) v = __bfloat162float(__float2bfloat16_rn(v + __bfloat162float(rr[c])));
    out[static_cast<size_t>(orow) * H + c] = __float2bfloat16_rn(__bfloat162float(w[c]) * (v * rstd));
  }
}

// out[j, :] = x[src_rows[j], :]
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src_rows,
                   __nv_bfloat16* __restrict__ out, int T, int H, int* status) {
  griddep_wait();               // the previous kernel's writes are visible from here
  griddep_launch_dependents();  // the next kernel may be scheduled
  const int warps_per_block = blockDim.x >> 5;
  const int j = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (j >= T) return;
  const int lane = threadIdx.x & 31;
  const int src_row = src_rows[j];
  if (kChecks && !index_ok(src_row, T, status)) return;   // checking build: row not copied
  const size_t src = static_cast<size_t>(src_row) * H;
  const size_t dst = static_cast<size_t>(j) * H;
  if ((H & 7) == 0) {
    const uint4* s = reinterpret_cast<const uint4*>(x + src);
    uint4* d = reinterpret_cast<uint4*>(out + dst);
    for (int c = lane; c < (H >> 3); c += 32) d[c] = s[c];
  } else {
    for (int c = lane; c < H; c += 32) out[dst + c] = x[src + c];
  }
}

// Expert-parallel dispatch by peer stores: sorted row j (source row src_rows[j] of x, or j
// itself) belongs to expert e with offsets[e] <= j < offsets[e + 1]; it is written to row
// push_base[e] + (j - offsets[e]) of the receive buffer of rank e / experts_per_rank, whose
// base address (peer-mapped memory) is peer_ptrs[rank].  Plain 16-byte stores over NVLink.
__global__ void __launch_bounds__(256)
push_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src_rows,
                 const int* __restrict__ offsets, const int* __restrict__ push_base, int E,
                 int experts_per_rank, const unsigned long long* __restrict__ peer_ptrs, int T,
                 int H) {
  extern __shared__ int s_off[];   // [E + 1] offsets, [E] push_base
  for (int i = threadIdx.x; i <= E; i += blockDim.x) s_off[i] = offsets[i];
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_off[E + 1 + i] = push_base[i];
  __syncthreads();
  const int j = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (j >= T) return;
  const int lane = threadIdx.x & 31;
  int lo = 0, hi = E;              // largest e with offsets[e] <= j
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (s_off[mid] <= j) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int rank = e / experts_per_rank;
  const long long drow = static_cast<long long>(s_off[E + 1 + e]) + (j - s_off[e]);
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(peer_ptrs[rank]) + drow * H;
  const __nv_bfloat16* src = x + static_cast<size_t>(src_rows ? src_rows[j] : j) * H;
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  for (int c = lane; c < (H >> 3); c += 32) d4[c] = s4[c];
}

// Barrier across the GPUs of an expert-parallel group, between two phases of the exchange by
// peer stores.  flags: this GPU's signal pad, int32 [1 + world]: flags[0] is this GPU's own
// barrier count (advanced here, so the launch arguments never change and the launch can sit
// in a CUDA graph), flags[1 + r] the last count GPU r announced.  Thread r announces this
// GPU's new count in GPU r's pad (a release store at system scope: every store this GPU issued
// before the barrier kernel, peer stores included, is visible to whoever acquires the flag) and
// then waits for GPU r's announcement of the same count.  The wait is bounded: after limit_ns
// the kernel raises the status word and returns, it never spins forever on a GPU that left.
__global__ void __launch_bounds__(64)
peer_barrier_kernel(const unsigned long long* __restrict__ peer_flags, int* flags, int rank,
                    int world, unsigned long long limit_ns, int* status) {
  __shared__ int s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = flags[0] + 1;
    flags[0] = s_epoch;
  }
  __syncthreads();
  const int epoch = s_epoch;
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  int* remote = reinterpret_cast<int*>(peer_flags[r]) + 1 + rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const int* mine = flags + 1 + r;
  unsigned long long t0 = 0;
  unsigned spins = 0;
  while (true) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (seen - epoch >= 0) break;
    if ((++spins & 0xffu) == 0) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        if (status) atomicExch(status, 2);
        break;
      }
    }
  }
}

// One warp per (token, head) over the q and k heads of the fused [T, (hq + 2 hkv) * D]
// buffer: y = rmsnorm(head) * norm_w, then rotate-half RoPE with fp32 cos/sin tables
// [positions, D].  Lane l owns the element pairs (2l', 2l'+1) of the first half together
// with their partners D/2 further, so the rotation needs no shuffles.
//
// Decode-step form (`app.pos_dev` set, one row per sequence): the position of every row is
// read from device memory, and the rotated k head and the v head of the row are also written
// to the KV cache at that position (nothing is written when it is outside the cache).
struct KvAppend {
  const int* pos_dev;          // device scalar: position of the new token (null: use pos0)
  __nv_bfloat16* k_cache;      // [B, hkv, capacity, D] with the strides below (null: no append)
  __nv_bfloat16* v_cache;
  long long stride_b, stride_h, stride_t;
  int capacity;
};

__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(__nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ q_w,
                    const __nv_bfloat16* __restrict__ k_w, const float* __restrict__ cos_t,
                    const float* __restrict__ sin_t, float eps, int T, int S, int pos0, int hq,
                    int hkv, int D, KvAppend app) {
  griddep_wait();               // the previous kernel's writes are visible from here
  griddep_launch_dependents();  // the next kernel may be scheduled
  const int heads = hq + hkv;
  const long long wid = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= static_cast<long long>(T) * heads) return;
  const int lane = threadIdx.x & 31;
  const int t = static_cast<int>(wid / heads);
  const int h = static_cast<int>(wid - static_cast<long long>(t) * heads);
  const int ld = (hq + 2 * hkv) * D;
  __nv_bfloat16* head = qkv + static_cast<size_t>(t) * ld + static_cast<size_t>(h) * D;
  const __nv_bfloat16* nw = (h < hq) ? q_w : k_w;
  const int half = D >> 1;
  if (app.pos_dev) pos0 = __ldg(app.pos_dev);
  const int pos = pos0 + (t % S);
  if (app.pos_dev && (pos < 0 || pos >= app.capacity)) return;
  const float* cs = cos_t + static_cast<size_t>(pos) * D;
  const float* sn = sin_t + static_cast<size_t>(pos) * D;
  __nv_bfloat16* kdst = nullptr;
  if (app.k_cache && h >= hq) {
    const long long off = t * app.stride_b + (h - hq) * app.stride_h + pos * app.stride_t;
    kdst = app.k_cache + off;
    const __nv_bfloat16* vsrc = head + static_cast<size_t>(hkv) * D;   // the v head of this k head
    __nv_bfloat16* vdst = app.v_cache + off;
    for (int j = 2 * lane; j < D; j += 64)
      *reinterpret_cast<uint32_t*>(vdst + j) = *reinterpret_cast<const uint32_t*>(vsrc + j);
  }

  float ss = 0.f;
  for (int j = 2 * lane; j < half; j += 64) {
    const uint32_t a = *reinterpret_cast<const uint32_t*>(head + j);
    const uint32_t b = *reinterpret_cast<const uint32_t*>(head + half + j);
    ss += lo_f(a) * lo_f(a) + hi_f(a) * hi_f(a) + lo_f(b) * lo_f(b) + hi_f(b) * hi_f(b);
  }
  ss = warp_sum(ss);
  const float rstd = nw ? rsqrtf(ss / static_cast<float>(D) + eps) : 1.0f;
  for (int j = 2 * lane; j < half; j += 64) {
    const uint32_t a = *reinterpret_cast<const uint32_t*>(head + j);
    const uint32_t b = *reinterpret_cast<const uint32_t*>(head + half + j);
    float a0 = lo_f(a) * rstd, a1 = hi_f(a) * rstd, b0 = lo_f(b) * rstd, b1 = hi_f(b) * rstd;
    if (nw) {
      const uint32_t wa = *reinterpret_cast<const uint32_t*>(nw + j);
      const uint32_t wb = *reinterpret_cast<const uint32_t*>(nw + half + j);
      a0 *= lo_f(wa); a1 *= hi_f(wa); b0 *= lo_f(wb); b1 *= hi_f(wb);
    }
    // out = x * cos + rotate_half(x) * sin, rotate_half(x) = [-x2, x1]
    const float o_a0 = a0 * cs[j] - b0 * sn[j];
    const float o_a1 = a1 * cs[j + 1] - b1 * sn[j + 1];
    const float o_b0 = b0 * cs[half + j] + a0 * sn[half + j];
    const float o_b1 = b1 * cs[half + j + 1] + a1 * sn[half + j + 1];
    *reinterpret_cast<uint32_t*>(head + j) = pack2(o_a0, o_a1);
    *reinterpret_cast<uint32_t*>(head + half + j) = pack2(o_b0, o_b1);
    if (kdst) {
      *reinterpret_cast<uint32_t*>(kdst + j) = pack2(o_a0, o_a1);
      *reinterpret_cast<uint32_t*>(kdst + half + j) = pack2(o_b0, o_b1);
    }
  }
}

// Vector form for D % 16 == 0 with D/16 a power of two <= 32 (D = 16 ... 512).  One warp per
// token: a head is handled by D/16 adjacent lanes (each owns 8 consecutive columns of the
// first half and the 8 partner columns D/2 further, 16-byte accesses), the warp's 32 / (D/16)
// lane groups take adjacent heads, and every lane walks over heads with the SAME column
// chunk, so the cos/sin values of the token's position are loaded once and reused for all
// its heads.  kAppend: the decode-step form described at KvAppend (same arithmetic).
template <bool kAppend>
__global__ void __launch_bounds__(256, 2)
qk_norm_rope_vec_kernel(__nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ q_w,
                        const __nv_bfloat16* __restrict__ k_w, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, float eps, int T, int S, int pos0, int hq,
                        int hkv, int D, KvAppend app) {
  griddep_wait();               // the previous kernel's writes are visible from here
  griddep_launch_dependents();  // the next kernel may be scheduled
  const int heads = hq + hkv;
  const int half = D >> 1;
  const int lph = half >> 3;        // lanes per head
  const int groups = 32 / lph;      // heads handled side by side by one warp
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;               // whole warps leave together
  const int lane = threadIdx.x & 31;
  const int g = lane / lph;
  const int j = (lane - g * lph) * 8;
  if (kAppend && app.pos_dev) pos0 = __ldg(app.pos_dev);
  const int pos = pos0 + (t % S);
  if (kAppend && (pos < 0 || pos >= app.capacity)) return;   // uniform: one position per call
  float c1[8], s1[8], c2[8], s2[8];
  {
    const float* cs = cos_t + static_cast<size_t>(pos) * D;
    const float* sn = sin_t + static_cast<size_t>(pos) * D;
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(cs + j) + v);
      const float4 b = __ldg(reinterpret_cast<const float4*>(sn + j) + v);
      const float4 c = __ldg(reinterpret_cast<const float4*>(cs + half + j) + v);
      const float4 d = __ldg(reinterpret_cast<const float4*>(sn + half + j) + v);
      c1[4 * v] = a.x; c1[4 * v + 1] = a.y; c1[4 * v + 2] = a.z; c1[4 * v + 3] = a.w;
      s1[4 * v] = b.x; s1[4 * v + 1] = b.y; s1[4 * v + 2] = b.z; s1[4 * v + 3] = b.w;
      c2[4 * v] = c.x; c2[4 * v + 1] = c.y; c2[4 * v + 2] = c.z; c2[4 * v + 3] = c.w;
      s2[4 * v] = d.x; s2[4 * v + 1] = d.y; s2[4 * v + 2] = d.z; s2[4 * v + 3] = d.w;
    }
  }
  // norm weights of this lane's columns, kept packed (q and k heads use different weights)
  uint4 wq1 = make_uint4(0, 0, 0, 0), wq2 = wq1, wk1 = wq1, wk2 = wq1;
  if (q_w) {
    wq1 = *reinterpret_cast<const uint4*>(q_w + j);
    wq2 = *reinterpret_cast<const uint4*>(q_w + half + j);
    wk1 = *reinterpret_cast<const uint4*>(k_w + j);
    wk2 = *reinterpret_cast<const uint4*>(k_w + half + j);
  }
  const int ld = (hq + 2 * hkv) * D;
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * ld;
  // All loads of the token are issued before any arithmetic (up to kMaxIter heads per lane
  // group) so enough bytes are in flight to cover HBM latency.
  constexpr int kMaxIter = 3;
  for (int hb = 0; hb < heads; hb += groups * kMaxIter) {   // uniform trip count across the warp
    uint4 a[kMaxIter], b[kMaxIter];
#pragma unroll
    for (int i = 0; i < kMaxIter; ++i) {
      const int h = hb + i * groups + g;
      a[i] = make_uint4(0, 0, 0, 0);
      b[i] = make_uint4(0, 0, 0, 0);
      if (h < heads) {
        a[i] = *reinterpret_cast<const uint4*>(row + static_cast<size_t>(h) * D + j);
        b[i] = *reinterpret_cast<const uint4*>(row + static_cast<size_t>(h) * D + half + j);
      }
    }
#pragma unroll
    for (int i = 0; i < kMaxIter; ++i) {
      const int h = hb + i * groups + g;
      if (hb + i * groups >= heads) break;                  // uniform
      const bool active = h < heads;
      const uint32_t aw[4] = {a[i].x, a[i].y, a[i].z, a[i].w};
      const uint32_t bw[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
      float x1[8], x2[8];
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x1[2 * e] = lo_f(aw[e]); x1[2 * e + 1] = hi_f(aw[e]);
        x2[2 * e] = lo_f(bw[e]); x2[2 * e + 1] = hi_f(bw[e]);
        ss += x1[2 * e] * x1[2 * e] + x1[2 * e + 1] * x1[2 * e + 1] + x2[2 * e] * x2[2 * e] +
              x2[2 * e + 1] * x2[2 * e + 1];
      }
      for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (!active) continue;
      if (q_w) {
        const float rstd = rsqrtf(ss / static_cast<float>(D) + eps);
        const uint4 w1 = (h < hq) ? wq1 : wk1, w2 = (h < hq) ? wq2 : wk2;
        const uint32_t w1w[4] = {w1.x, w1.y, w1.z, w1.w}, w2w[4] = {w2.x, w2.y, w2.z, w2.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          x1[2 * e] *= rstd * lo_f(w1w[e]); x1[2 * e + 1] *= rstd * hi_f(w1w[e]);
          x2[2 * e] *= rstd * lo_f(w2w[e]); x2[2 * e + 1] *= rstd * hi_f(w2w[e]);
        }
      }
      float o1[8], o2[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o1[e] = x1[e] * c1[e] - x2[e] * s1[e];   // x * cos + rotate_half(x) * sin, first half
        o2[e] = x2[e] * c2[e] + x1[e] * s2[e];   // second half
      }
      uint4 oa, ob;
      oa.x = pack2(o1[0], o1[1]); oa.y = pack2(o1[2], o1[3]); oa.z = pack2(o1[4], o1[5]); oa.w = pack2(o1[6], o1[7]);
      ob.x = pack2(o2[0], o2[1]); ob.y = pack2(o2[2], o2[3]); ob.z = pack2(o2[4], o2[5]); ob.w = pack2(o2[6], o2[7]);
      __nv_bfloat16* head = row + static_cast<size_t>(h) * D;
      *reinterpret_cast<uint4*>(head + j) = oa;
      *reinterpret_cast<uint4*>(head + half + j) = ob;
      if (kAppend && h >= hq) {
        __nv_bfloat16* kdst = app.k_cache + t * app.stride_b + (h - hq) * app.stride_h +
                              pos * app.stride_t;
        *reinterpret_cast<uint4*>(kdst + j) = oa;
        *reinterpret_cast<uint4*>(kdst + half + j) = ob;
      }
    }
  }
  if (kAppend) {   // the row's v heads, 16 bytes per lane and step
    const __nv_bfloat16* vsrc = row + static_cast<size_t>(heads) * D;
    for (int c = lane * 8; c < hkv * D; c += 256) {
      const int vh = c / D;
      __nv_bfloat16* vdst = app.v_cache + t * app.stride_b + vh * app.stride_h +
                            pos * app.stride_t + (c - vh * D);
      *reinterpret_cast<uint4*>(vdst) = *reinterpret_cast<const uint4*>(vsrc + c);
    }
  }
}

}  // namespace

cudaError_t launch_rmsnorm(const void* x, const void* residual, const void* weight, float eps,
                           void* sum_out, void* out, const int* dst_rows, int T, int H,
                           cudaStream_t stream, bool split) {
  if (T == 0) return cudaSuccess;
  auto xb = static_cast<const __nv_bfloat16*>(x);
  auto rb = static_cast<const __nv_bfloat16*>(residual);
  auto wb = static_cast<const __nv_bfloat16*>(weight);
  auto sb = static_cast<__nv_bfloat16*>(sum_out);
  auto ob = static_cast<__nv_bfloat16*>(out);
  int* status = kChecks ? device_status_word() : nullptr;
  if ((H & 255) == 0 && H <= kMaxVec * 256) {
    const int blocks = (T + kNormWarps - 1) / kNormWarps;
    auto go = [&](auto kern) {
      return launch_kernel(kern, dim3(blocks), dim3(kNormWarps * 32), 0, stream, xb, rb, wb, eps, sb,
                           ob, dst_rows, T, H, status);
    };
    switch (H >> 8) {   // hidden sizes 768 / 1024 / 2048 get their own instantiation (fewer registers)
      case 3: return split ? go(rmsnorm_rows_kernel<true, 3>) : go(rmsnorm_rows_kernel<false, 3>);
      case 4: return split ? go(rmsnorm_rows_kernel<true, 4>) : go(rmsnorm_rows_kernel<false, 4>);
      case 8: return split ? go(rmsnorm_rows_kernel<true, 8>) : go(rmsnorm_rows_kernel<false, 8>);
      default: return split ? go(rmsnorm_rows_kernel<true, 0>) : go(rmsnorm_rows_kernel<false, 0>);
    }
  } else {
    return launch_kernel(rmsnorm_generic_kernel, dim3(T), dim3(128), 0, stream, xb, rb, wb, eps, sb,
                         ob, dst_rows, T, H, split ? 1 : 0, status);
  }
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const void* x, const int* src_rows, void* out, int T, int H,
                               cudaStream_t stream) {
  if (T == 0) return cudaSuccess;
  const int wpb = 8;
  return launch_kernel(gather_rows_kernel, dim3((T + wpb - 1) / wpb), dim3(wpb * 32), 0, stream,
                       static_cast<const __nv_bfloat16*>(x), src_rows,
                       static_cast<__nv_bfloat16*>(out), T, H,
                       kChecks ? device_status_word() : nullptr);
}

cudaError_t launch_push_rows(const void* x, const int* src_rows, const int* offsets,
                             const int* push_base, int E, int experts_per_rank,
                             const unsigned long long* peer_ptrs, int T, int H,
                             cudaStream_t stream) {
  if (T == 0) return cudaSuccess;
  const int wpb = 8;
  push_rows_kernel<<<(T + wpb - 1) / wpb, wpb * 32, (2 * E + 1) * sizeof(int), stream>>>(
      static_cast<const __nv_bfloat16*>(x), src_rows, offsets, push_base, E, experts_per_rank,
      peer_ptrs, T, H);
  return cudaGetLastError();
}

cudaError_t launch_peer_barrier(const unsigned long long* peer_flags, int* flags, int rank, int world,
                                unsigned long long limit_ns, int* status, cudaStream_t stream) {
  peer_barrier_kernel<<<1, 64, 0, stream>>>(peer_flags, flags, rank, world, limit_ns, status);
  return cudaGetLastError();
}

cudaError_t launch_qk_norm_rope(void* qkv, const void* q_w, const void* k_w, const float* cos_t,
                                const float* sin_t, float eps, int T, int S, int pos0, int hq,
                                int hkv, int D, cudaStream_t stream, const int* pos_dev,
                                void* k_cache, void* v_cache, long long kv_stride_b,
                                long long kv_stride_h, long long kv_stride_t, int capacity) {
  if (T == 0) return cudaSuccess;
  KvAppend app{pos_dev, static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),
               kv_stride_b, kv_stride_h, kv_stride_t, capacity};
  const bool append = k_cache != nullptr;
  const int lph = D >> 4;
  const bool aligned = (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(cos_t) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(sin_t) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(q_w) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(k_w) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0 &&
                       ((kv_stride_b | kv_stride_h | kv_stride_t) & 7) == 0;
  auto qb = static_cast<__nv_bfloat16*>(qkv);
  auto qw = static_cast<const __nv_bfloat16*>(q_w);
  auto kw = static_cast<const __nv_bfloat16*>(k_w);
  if ((D & 15) == 0 && lph >= 1 && lph <= 32 && (lph & (lph - 1)) == 0 && aligned) {
    const unsigned nblocks = static_cast<unsigned>((T + 7) / 8);  // one warp per token
    return append ? launch_kernel(qk_norm_rope_vec_kernel<true>, dim3(nblocks), dim3(256), 0, stream,
                                  qb, qw, kw, cos_t, sin_t, eps, T, S, pos0, hq, hkv, D, app)
                  : launch_kernel(qk_norm_rope_vec_kernel<false>, dim3(nblocks), dim3(256), 0, stream,
                                  qb, qw, kw, cos_t, sin_t, eps, T, S, pos0, hq, hkv, D, app);
  }
  const long long warps = static_cast<long long>(T) * (hq + hkv);
  const int wpb = 8;
  const long long blocks = (warps + wpb - 1) / wpb;
  return launch_kernel(qk_norm_rope_kernel, dim3(static_cast<unsigned>(blocks)), dim3(wpb * 32), 0,
                       stream, qb, qw, kw, cos_t, sin_t, eps, T, S, pos0, hq, hkv, D, app);
}

}  // namespace cdeep
