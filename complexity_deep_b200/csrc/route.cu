// Deterministic token dispatch: token id -> expert table lookup, per-expert histogram,
// exclusive prefix sum and the STABLE permutation that groups rows by expert.
//
// Replaces, for all layers at once, what the reference does per layer with a Python loop
// of boolean masks (complexity_deep/core/token_routed_mlp.py:149-150 lookup, :166-170
// mask / gather, :174 scatter).  `x[mask]` keeps rows in ascending row order, so the
// permutation is a stable counting sort of the expert ids; there is no atomic whose order
// could change the result, and two runs give identical bytes.
//
// Two launches:
//   route_lookup_hist : ids -> expert_ids, and one histogram per block of kTokPerBlock tokens
//   route_rank        : totals + offsets from the block histograms, then each warp ranks a
//                       contiguous slice of its block with match/ballot, in row order.
// Scratch: the block histograms, ceil(T / kTokPerBlock) * E int32.
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <cuda_runtime.h>
#include "../../include/cdeep.h"
#include "kernels.h"

namespace cdeep {

constexpr int kRouteThreads = 256;
constexpr int kRouteWarps = kRouteThreads / 32;
constexpr int kTokPerBlock = 2048;
constexpr int kTokPerWarp = kTokPerBlock / kRouteWarps;

__global__ void __launch_bounds__(kRouteThreads)
route_lookup_hist_kernel(const long long* __restrict__ ids, const long long* __restrict__ table,
                         int V, int E, int T, int* __restrict__ expert_ids,
                         int* __restrict__ block_hist) {
  extern __shared__ int s_hist[];  // [E]
  for (int e = threadIdx.x; e < E; e += kRouteThreads) s_hist[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kTokPerBlock;
  for (int k = threadIdx.x; k < kTokPerBlock; k += kRouteThreads) {
    const int i = base + k;
    if (i < T) {
      long long id = ids[i];
      id = id < 0 ? 0 : (id > V - 1 ? V - 1 : id);          // clamp(0, V-1)
      long long e = table[id];
      e = e < 0 ? 0 : (e > E - 1 ? E - 1 : e);              // memory safety only; the host
                                                            // checks the table's range
      expert_ids[i] = static_cast<int>(e);
      atomicAdd(&s_hist[static_cast<int>(e)], 1);           // order-free: only a count
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kRouteThreads)
    block_hist[static_cast<size_t>(blockIdx.x) * E + e] = s_hist[e];
}

__global__ void __launch_bounds__(kRouteThreads)
route_rank_kernel(const int* __restrict__ expert_ids, const int* __restrict__ block_hist, int E,
                  int T, int num_blocks, int* __restrict__ counts, int* __restrict__ offsets,
                  int* __restrict__ perm, int* __restrict__ inv_perm) {
  extern __shared__ int s_mem[];
  int* s_total = s_mem;                 // [E]   tokens of expert e in the whole batch
  int* s_start = s_mem + E;             // [E]   first sorted position for this block
  int* s_whist = s_mem + 2 * E;         // [warps][E]
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // totals and the number of tokens of each expert in earlier blocks
  for (int e = threadIdx.x; e < E; e += kRouteThreads) {
    int total = 0, before = 0;
    for (int b = 0; b < num_blocks; ++b) {
      const int c = block_hist[static_cast<size_t>(b) * E + e];
      total += c;
      if (b < static_cast<int>(blockIdx.x)) before += c;
    }
    s_total[e] = total;
    s_start[e] = before;
  }
  for (int k = threadIdx.x; k < kRouteWarps * E; k += kRouteThreads) s_whist[k] = 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = s_total[e];
      if (blockIdx.x == 0) {
        counts[e] = c;
        offsets[e] = run;
      }
      s_start[e] += run;
      run += c;
    }
    if (blockIdx.x == 0) offsets[E] = run;
  }

  // pass A: histogram of this warp's contiguous slice
  const int wbase = blockIdx.x * kTokPerBlock + warp * kTokPerWarp;
  int* my_hist = s_whist + warp * E;
  for (int k = 0; k < kTokPerWarp; k += 32) {
    const int i = wbase + k + lane;
    const int e = (i < T) ? expert_ids[i] : E;  // E = "no token"
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (e < E && lane == __ffs(peers) - 1) my_hist[e] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  // exclusive scan over the warps of this block, per expert
  for (int e = threadIdx.x; e < E; e += kRouteThreads) {
    int run = s_start[e];
    for (int w = 0; w < kRouteWarps; ++w) {
      const int c = s_whist[w * E + e];
      s_whist[w * E + e] = run;
      run += c;
    }
  }
  __syncthreads();
  // pass B: stable rank inside the warp's slice
  for (int k = 0; k < kTokPerWarp; k += 32) {
    const int i = wbase + k + lane;
    const int e = (i < T) ? expert_ids[i] : E;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const unsigned lower = peers & ((1u << lane) - 1u);
    if (e < E) {
      const int pos = my_hist[e] + __popc(lower);
      perm[pos] = i;
      inv_perm[i] = pos;
    }
    __syncwarp();
    if (e < E && lower == 0) my_hist[e] += __popc(peers);
    __syncwarp();
  }
}

size_t route_workspace_bytes(int T, int E) {
  const size_t nb = (static_cast<size_t>(T) + kTokPerBlock - 1) / kTokPerBlock;
  return (nb > 0 ? nb : 1) * static_cast<size_t>(E) * sizeof(int);
}

cudaError_t launch_route(const long long* ids, const long long* table, int V, int E, int T,
                         int* expert_ids, int* counts, int* offsets, int* perm, int* inv_perm,
                         int* block_hist, cudaStream_t stream) {
  const int nb = (T + kTokPerBlock - 1) / kTokPerBlock;
  const int blocks = nb > 0 ? nb : 1;  // T == 0 still writes zero counts and offsets
  route_lookup_hist_kernel<<<blocks, kRouteThreads, E * sizeof(int), stream>>>(
      ids, table, V, E, T, expert_ids, block_hist);
  route_rank_kernel<<<blocks, kRouteThreads, (2 + kRouteWarps) * E * sizeof(int), stream>>>(
      expert_ids, block_hist, E, T, blocks, counts, offsets, perm, inv_perm);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// Dispatch without any allocation by the caller or the library.
//
// Some hosts of this library cannot allocate device memory at the point where they route a
// batch: a serving loop that runs under a fixed memory budget and must not touch the
// allocator once it is warm, or a plugin that only receives input and output buffers from
// its framework and has no handle to an allocator.  For them the block histograms of the
// dispatch live in a fixed array that is part of the library image; every GPU that loads
// the library holds these 512 KiB until the process exits.
namespace {

constexpr int kStaticScratchInts = 131072;  // 512 KiB: ceil(T / 2048) * E must fit
static __device__ __align__(256) int g_route_scratch[kStaticScratchInts];

constexpr int kStaticMaxDevices = 64;
int* g_scratch_ptr[kStaticMaxDevices] = {nullptr};
std::mutex g_scratch_mu;

// In host code `g_route_scratch` is only a handle for the runtime, not a device address;
// the address on the CURRENT device is looked up once per device and cached.
cudaError_t static_scratch_for_current_device(int** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kStaticMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_route_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace
}  // namespace cdeep

extern "C" int cd_route_static_max_tokens(int E) {
  if (E < 1 || E > 256) return 0;
  const long long blocks = cdeep::kStaticScratchInts / E;
  const long long t = blocks * cdeep::kTokPerBlock;
  return t > 0x7fffffffLL ? 0x7fffffff : static_cast<int>(t);
}

extern "C" int cd_route_static(const int64_t* ids, const int64_t* table, int V, int E, int T,
                               int32_t* expert_ids, int32_t* counts, int32_t* offsets,
                               int32_t* perm, int32_t* inv_perm, void* stream) {
  using namespace cdeep;
  if (T < 0 || V < 1 || E < 1 || E > 256) return CD_ERR_INVALID;
  if (!table || !counts || !offsets) return CD_ERR_INVALID;
  if (T > 0 && (!ids || !expert_ids || !perm || !inv_perm)) return CD_ERR_INVALID;
  const long long blocks = (static_cast<long long>(T) + kTokPerBlock - 1) / kTokPerBlock;
  if ((blocks > 0 ? blocks : 1) * E > kStaticScratchInts) {
    snprintf(g_cuda_err, sizeof(g_cuda_err),
             "cd_route_static: T=%d with E=%d needs %lld scratch ints, the built-in array holds %d "
             "(use cd_route with caller-provided scratch)",
             T, E, (blocks > 0 ? blocks : 1) * E, kStaticScratchInts);
    return CD_ERR_UNSUPPORTED;
  }
  int* scratch = nullptr;
  cudaError_t e = static_scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(route scratch)");
  // Every histogram slot that route_rank reads is written by route_lookup_hist in this same
  // call, so nothing left over from an earlier call has to be cleared.
  e = launch_route(reinterpret_cast<const long long*>(ids),
                   reinterpret_cast<const long long*>(table), V, E, T, expert_ids, counts,
                   offsets, perm, inv_perm, scratch, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "route launch");
}
