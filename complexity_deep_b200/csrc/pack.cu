// One-off weight layout transforms into the layouts the GEMM kernels read (caller-owned
// buffers; run once per weight version, not on the forward path).
//
// The reference stores the routed experts as gate_proj_w / up_proj_w [E, H, I] and down_proj_w
// [E, I, H] and multiplies `x @ W[e]` (complexity_deep/core/token_routed_mlp.py:62-70, :171-174);
// the shared expert is three nn.Linear weights [I, H], [I, H], [H, I] (:75-77).  The tcgen05
// kernels want every B operand K-major (one output feature per row, K contiguous) and the
// gate / up rows interleaved per accumulator tile so that silu(gate) * up is tile-local.
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "kernels.h"

namespace cdeep {

namespace {

// packed[g, t * bn + s * half + j, :] = src_s[g][feature t * half + j][:]   (s = 0 gate, 1 up)
// Features past I are zero rows.  `feature_major` = 1: sources are [G, I, H] (nn.Linear layout,
// rows copied); 0: sources are [G, H, I] (the reference's routed layout, transposed on the way
// through a 32 x 32 shared-memory tile).
__global__ void __launch_bounds__(256)
pack_gate_up_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                    __nv_bfloat16* __restrict__ packed, int I, int H, int half, int rows,
                    int feature_major) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int g = blockIdx.z >> 1;
  const int s = blockIdx.z & 1;
  const __nv_bfloat16* src = (s ? up : gate) + static_cast<size_t>(g) * I * H;
  const int f0 = blockIdx.y * 32;   // feature (output column of the expert) block
  const int h0 = blockIdx.x * 32;   // hidden (K) block
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  const int padded = (rows / (2 * half)) * half;   // features incl. zero padding
  if (feature_major) {
    for (int r = ty; r < 32; r += 8) {
      const int f = f0 + r, h = h0 + tx;
      tile[r][tx] = (f < I && h < H) ? src[static_cast<size_t>(f) * H + h] : __float2bfloat16(0.f);
    }
  } else {
    for (int r = ty; r < 32; r += 8) {
      const int h = h0 + r, f = f0 + tx;
      tile[tx][r] = (f < I && h < H) ? src[static_cast<size_t>(h) * I + f] : __float2bfloat16(0.f);
    }
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int f = f0 + r, h = h0 + tx;
    if (f < padded && h < H) {
      const int t = f / half, j = f - t * half;
      const size_t row = static_cast<size_t>(g) * rows + static_cast<size_t>(t) * 2 * half +
                         static_cast<size_t>(s) * half + j;
      packed[row * H + h] = tile[r][tx];
    }
  }
}

// out[g, c, r] = in[g, r, c]  (in: [G, R, C])
__global__ void __launch_bounds__(256)
transpose_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int R,
                 int C) {
  __shared__ __nv_bfloat16 tile[32][33];
  const size_t base = static_cast<size_t>(blockIdx.z) * R * C;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8)
    if (r0 + r < R && c0 + tx < C) tile[r][tx] = in[base + static_cast<size_t>(r0 + r) * C + c0 + tx];
  __syncthreads();
  for (int c = ty; c < 32; c += 8)
    if (c0 + c < C && r0 + tx < R) out[base + static_cast<size_t>(c0 + c) * R + r0 + tx] = tile[tx][c];
}

}  // namespace

cudaError_t launch_pack_gate_up(const void* gate, const void* up, void* packed, int G, int I, int H,
                                int block_n, int feature_major, cudaStream_t stream) {
  const int half = block_n / 2;
  const int rows = ((I + half - 1) / half) * block_n;
  const int padded = rows / 2;
  dim3 grid((H + 31) / 32, (padded + 31) / 32, 2 * G);
  pack_gate_up_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(gate),
                                                static_cast<const __nv_bfloat16*>(up),
                                                static_cast<__nv_bfloat16*>(packed), I, H, half,
                                                rows, feature_major);
  return cudaGetLastError();
}

cudaError_t launch_transpose(const void* in, void* out, int G, int R, int C, cudaStream_t stream) {
  dim3 grid((C + 31) / 32, (R + 31) / 32, G);
  transpose_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(in),
                                             static_cast<__nv_bfloat16*>(out), R, C);
  return cudaGetLastError();
}

}  // namespace cdeep
