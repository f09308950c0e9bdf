// Exchange plan of the expert-parallel layer in ONE launch (the reference has no distributed
// code; this is the index arithmetic between the dispatch of complexity_deep/core/
// token_routed_mlp.py:166-170 and the grouped expert GEMMs when the experts live on other GPUs).
//
// Input: the count matrix of all ranks, counts[g][e] = rows of expert e among rank g's tokens
// (gathered by peer_put_kernel below and the cross-GPU barrier, or by any all-gather).  Receive buffers are laid out expert-major, source-minor — the order
// the grouped GEMM wants — so for THIS rank the kernel derives
//   push_base[e]    row in the owner's receive buffer where this rank's rows of expert e start
//                   (the owner's segment start of e plus the rows of lower-ranked sources),
//   seg_offsets[.]  segments of this rank's own receive buffer (El + 1 entries),
//   row_ptrs[r]     for every row r of this rank's receive buffer the address of its slot in its
//                   home rank's return buffer: home base + (home's sorted offset of e + k) * bytes,
// the same integers as the host / tensor forms of the plan in expert_parallel.py, bit for bit.
#include <cstdint>
#include <cuda_runtime.h>
#include "kernels.h"

namespace cdeep {

namespace {

constexpr int kPlanThreads = 256;
constexpr int kPlanMaxCounts = 8192;   // ranks x experts
constexpr int kPlanMaxBlocks = 2048;   // ranks x experts per rank

__global__ void __launch_bounds__(kPlanThreads)
ep_plan_kernel(const int* __restrict__ counts, int G, int E, int El, int rank,
               const long long* __restrict__ ret_ptrs, long long row_bytes, int capacity,
               int* __restrict__ push_base, int* __restrict__ seg_offsets,
               long long* __restrict__ row_ptrs) {
  extern __shared__ int sm[];
  int* cnt = sm;                         // [G * E]
  int* block_end = cnt + G * E;          // [El * G] inclusive ends of the (local expert, source) blocks
  int* home_off = block_end + El * G;    // [El * G] source's sorted offset of the block's expert
  const int tid = threadIdx.x;
  for (int i = tid; i < G * E; i += kPlanThreads) cnt[i] = counts[i];
  __syncthreads();
  // rows before local expert le in the source's own sorted order: prefix over the experts
  const int nb = El * G;
  for (int b = tid; b < nb; b += kPlanThreads) {
    const int le = b / G, src = b - le * G;
    const int ge = rank * El + le;
    int acc = 0;
    for (int e = 0; e < ge; ++e) acc += cnt[src * E + e];
    home_off[b] = acc;
  }
  if (tid == 0) {   // a few hundred additions at most
    int acc = 0;
    for (int b = 0; b < nb; ++b) {
      const int le = b / G, src = b - le * G;
      acc += cnt[src * E + rank * El + le];
      block_end[b] = acc;
    }
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e = tid; e < E; e += kPlanThreads) {
      const int owner = e / El;
      int base = 0;
      for (int e2 = owner * El; e2 < e; ++e2)       // the owner's segments before e
        for (int g = 0; g < G; ++g) base += cnt[g * E + e2];
      for (int g = 0; g < rank; ++g) base += cnt[g * E + e];   // lower-ranked sources of e
      push_base[e] = base;
    }
    for (int le = tid; le <= El; le += kPlanThreads)
      seg_offsets[le] = le == 0 ? 0 : block_end[le * G - 1];
  }
  const int received = block_end[nb - 1];
  for (int r = blockIdx.x * kPlanThreads + tid; r < capacity; r += gridDim.x * kPlanThreads) {
    // first block whose end lies past r (entries past the received rows are never used: they
    // get the last block's arithmetic, like the tensor form)
    int lo = 0, hi = nb - 1;
    if (r < received) {
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (block_end[mid] > r) hi = mid; else lo = mid + 1;
      }
    } else {
      lo = nb - 1;
    }
    const int le = lo / G, src = lo - le * G;
    const int start = lo == 0 ? 0 : block_end[lo - 1];
    const long long slot = static_cast<long long>(home_off[lo]) + (r - start);
    (void)le;
    row_ptrs[r] = ret_ptrs[src] + slot * row_bytes;
  }
}

// Copies n int32 from src into every rank's buffer at element offset `offset` (block g writes to
// rank g; the buffers are peer-mapped).  With offset = rank * n every rank ends up holding the
// rows of all ranks: an all-gather of a few hundred bytes by plain peer stores, made visible by the
// cross-GPU barrier that follows it on the stream.
__global__ void __launch_bounds__(128)
peer_put_kernel(const int* __restrict__ src, int n, const unsigned long long* __restrict__ peer_bufs,
                long long offset) {
  int* dst = reinterpret_cast<int*>(peer_bufs[blockIdx.x]) + offset;
  for (int i = threadIdx.x; i < n; i += 128) dst[i] = src[i];
}

}  // namespace

cudaError_t launch_peer_put_i32(const int* src, int n, const unsigned long long* peer_bufs, int world,
                                long long offset, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  peer_put_kernel<<<world, 128, 0, stream>>>(src, n, peer_bufs, offset);
  return cudaGetLastError();
}

bool ep_plan_supported(int G, int E, int El) {
  return G >= 1 && El >= 1 && G * El == E && G * E <= kPlanMaxCounts && El * G <= kPlanMaxBlocks;
}

cudaError_t launch_ep_plan(const int* counts, int G, int E, int El, int rank,
                           const long long* ret_ptrs, long long row_bytes, int capacity,
                           int* push_base, int* seg_offsets, long long* row_ptrs,
                           cudaStream_t stream) {
  const size_t smem = (static_cast<size_t>(G) * E + 2 * static_cast<size_t>(El) * G) * sizeof(int);
  int blocks = (capacity + kPlanThreads * 4 - 1) / (kPlanThreads * 4);
  if (blocks < 1) blocks = 1;
  if (blocks > 148) blocks = 148;
  ep_plan_kernel<<<blocks, kPlanThreads, smem, stream>>>(counts, G, E, El, rank, ret_ptrs, row_bytes,
                                                         capacity, push_base, seg_offsets, row_ptrs);
  return cudaGetLastError();
}

}  // namespace cdeep
