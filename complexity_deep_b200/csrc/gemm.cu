// Host side of the tcgen05 GEMM: tensor-map encoding, shape checks, launch.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../../include/cdeep.h"
#include "gemm_sm100.cuh"
#include "kernels.h"

namespace cdeep {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver API is reached through the runtime so that the library links against
// nothing but cudart and still loads on a machine without a driver.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 tensor [rows, cols] with `ld` elements between rows; box = [box_rows, 64 cols],
// 128-byte swizzle (one box row = 128 bytes = one swizzle row), zero fill out of bounds.
bool encode_map(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld,
                int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBoxK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// A tensor map is a pure function of (address, shape, stride, box), and an eager decode step
// asks for the same ~1 000 of them every step (weights always, activations whenever the caller's
// allocator hands the same buffers back), so each thread keeps the ones it has encoded in a small
// direct-mapped table: a hit costs a hash and a 128-byte copy instead of a driver call.
struct MapKey {
  const void* base;
  long long rows, cols, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapSlot {
  MapKey key;
  bool used;
  CUtensorMap map;
};
constexpr int kMapSlots = 2048;   // power of two

bool make_map(CUtensorMap* m, const void* base, long long rows, long long cols, long long ld,
              int box_rows) {
  static thread_local MapSlot* table = nullptr;
  if (!table) table = new MapSlot[kMapSlots]();   // lives as long as the thread
  const MapKey key{base, rows, cols, ld, box_rows};
  unsigned long long h = reinterpret_cast<uintptr_t>(base) >> 4;
  h = (h ^ static_cast<unsigned long long>(rows) * 0x9E3779B97F4A7C15ull) * 0xff51afd7ed558ccdull;
  h ^= static_cast<unsigned long long>(cols) * 0xc4ceb9fe1a85ec53ull + static_cast<unsigned long long>(ld) * 31 +
       static_cast<unsigned long long>(box_rows);
  h ^= h >> 29;
  MapSlot& slot = table[h & (kMapSlots - 1)];
  if (slot.used && slot.key == key) {
    memcpy(m, &slot.map, sizeof(CUtensorMap));
    return true;
  }
  if (!encode_map(m, base, rows, cols, ld, box_rows)) return false;
  slot.key = key;
  slot.used = true;
  memcpy(&slot.map, m, sizeof(CUtensorMap));
  return true;
}

struct DeviceInfo {
  int sm_count = 0;
  bool attr_set[4][4][2] = {};  // [BN 32/64/128/256][epilogue][CTA group 1/2]
  int* status = nullptr;
  void* sk_ws = nullptr;        // split-K workspace registered by the caller (nullptr = split-K off)
  size_t sk_bytes = 0;
};
constexpr int kSkCounterBytes = 1024;   // head of the workspace: one arrival counter per output tile
constexpr int kSkMaxTiles = kSkCounterBytes / 4;
// Measured on B200 (32 rows, 2048 output columns): an unsplit launch costs 4.9 us + 0.21 us per 64
// elements of K, handing the partial tiles over costs about 4.5 us: two ranges pay from about 48
// boxes of 64 (K = 4096: 18.4 -> 16.0 us, K = 5632: 23.4 -> 18.5 us).
constexpr int kSkMinBlocksPerSplit = 16; // 64-element boxes of K per range
constexpr int kSkMinBlocks = 48;         // shortest K loop (in boxes) that is split at all
constexpr int kSkMaxSplits = 8;
// which forms of split-K a launch may take: bit 0 the cluster form, bit 1 the workspace form
int g_splitk_flags = 3;
constexpr int kMaxDevices = 64;
DeviceInfo g_dev[kMaxDevices];
std::mutex g_mu;

__device__ int g_status_word;  // raised by a kernel whose bounded wait ran out

template <int BN, int EPI, int CG>
cudaError_t launch_one(int grid, const CUtensorMap& a0, const CUtensorMap& b0,
                       const CUtensorMap& a1, const CUtensorMap& b1, const GemmParams& p,
                       DeviceInfo& di, cudaStream_t stream) {
  constexpr int bi = (BN == 256) ? 3 : (BN == 128) ? 2 : (BN == 64) ? 1 : 0;
  // CTA pairs are clusters of 2; the cluster form of split-K launches clusters of `splits` CTAs
  const unsigned cluster = (CG == 2) ? 2u : (p.sk_cluster ? static_cast<unsigned>(p.splits) : 1u);
  auto kern = gemm_bf16_sm100_kernel<BN, EPI, CG>;
  constexpr int smem = GemmSmem<BN, CG, gemm_epi_warps<BN, EPI>()>::kDynamic;
  if (!di.attr_set[bi][EPI][CG - 1]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    di.attr_set[bi][EPI][CG - 1] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(gemm_threads<BN, EPI>(), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // the kernel waits for its predecessor itself (griddep_wait) after its set-up
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kern, a0, b0, a1, b1, p);
}

template <int CG>
cudaError_t launch_any(int block_n, int kind, int grid, const CUtensorMap& a0,
                       const CUtensorMap& b0, const CUtensorMap& a1, const CUtensorMap& b1,
                       const GemmParams& p, DeviceInfo& di, cudaStream_t stream) {
  if (block_n == 256) {
    if (kind == kEpiStoreRope) return launch_one<256, kEpiStoreRope, CG>(grid, a0, b0, a1, b1, p, di, stream);
    if (kind == kEpiStoreSplit) return launch_one<256, kEpiStoreSplit, CG>(grid, a0, b0, a1, b1, p, di, stream);
    return kind == kEpiSwiGLU ? launch_one<256, kEpiSwiGLU, CG>(grid, a0, b0, a1, b1, p, di, stream)
                              : launch_one<256, kEpiStore, CG>(grid, a0, b0, a1, b1, p, di, stream);
  }
  if (kind == kEpiStoreRope) return cudaErrorInvalidValue;
  if (kind == kEpiStoreSplit) {
    if (block_n == 128) return launch_one<128, kEpiStoreSplit, CG>(grid, a0, b0, a1, b1, p, di, stream);
    if constexpr (CG == 1) {
      if (block_n == 64) return launch_one<64, kEpiStoreSplit, 1>(grid, a0, b0, a1, b1, p, di, stream);
      if (block_n == 32) return launch_one<32, kEpiStoreSplit, 1>(grid, a0, b0, a1, b1, p, di, stream);
    }
    return cudaErrorInvalidValue;
  }
  if (block_n == 128)
    return kind == kEpiSwiGLU ? launch_one<128, kEpiSwiGLU, CG>(grid, a0, b0, a1, b1, p, di, stream)
                              : launch_one<128, kEpiStore, CG>(grid, a0, b0, a1, b1, p, di, stream);
  // narrow tiles: few rows (decode), single-CTA only
  if constexpr (CG == 1) {
    if (block_n == 64)
      return kind == kEpiSwiGLU ? launch_one<64, kEpiSwiGLU, 1>(grid, a0, b0, a1, b1, p, di, stream)
                                : launch_one<64, kEpiStore, 1>(grid, a0, b0, a1, b1, p, di, stream);
    if (block_n == 32)
      return kind == kEpiSwiGLU ? launch_one<32, kEpiSwiGLU, 1>(grid, a0, b0, a1, b1, p, di, stream)
                                : launch_one<32, kEpiStore, 1>(grid, a0, b0, a1, b1, p, di, stream);
  }
  return cudaErrorInvalidValue;
}

// Accumulator-tile width for the store epilogue.
// Many tiles (prefill): the 256-wide tile whenever it gives (almost) every SM a tile; the GEMM
// is then bound by tensor throughput.  Few tiles (decode): an output tile is one chain of K/16
// MMA instructions issued by one thread, which cost that thread the same whatever their width up
// to 128 columns (measured: 40 .. 64 cycles per instruction plus about 300 per pipeline stage;
// time = 4.9 us + 0.21 us per 64 elements of K with two boxes per stage), so the time
// is set by how many tiles the busiest SM runs one after the other: the narrowest tile that
// still leaves at most one tile per SM; if even 256-wide tiles are more than that, the width
// with the fewest waves.  For grouped calls every non-empty group has at least one row tile.
int store_block_n_impl(int M, int N, int num_groups, int sm_count) {
  long long m_tiles = (M + kBlockM - 1) / kBlockM;
  if (num_groups > m_tiles) m_tiles = num_groups;
  auto tiles = [&](int bn) { return m_tiles * ((N + bn - 1) / bn); };
  if (tiles(256) * 4 >= 3LL * sm_count) return 256;
  for (int bn : {32, 64, 128, 256})
    if (tiles(bn) <= sm_count) return bn;
  int best = 256;
  long long best_cost = -1;
  for (int bn : {256, 128, 64, 32}) {
    const long long waves = (tiles(bn) + sm_count - 1) / sm_count;
    const long long cost = waves * (bn == 256 ? 160 : 140);
    if (best_cost < 0 || cost < best_cost) {
      best = bn;
      best_cost = cost;
    }
  }
  return best;
}

// CTA pairs (256-row tiles) are used whenever the 256-wide tile is: measured on B200 they win
// from 8 192 rows (1B prefill step 16.7 ms against 17.5 ms) to 65 536 rows; below 2 048 rows
// single CTAs keep more SMs busy.  CDEEP_CTA_GROUP=1|2 forces a choice (tuning aid).
int choose_cta_group(int M, int block_n, int sm_count) {
  static const int forced = [] {
    const char* e = getenv("CDEEP_CTA_GROUP");
    return e ? atoi(e) : 0;
  }();
  if (forced == 1 || forced == 2) return forced;
  (void)sm_count;
  if (block_n != 256) return 1;
  return M >= 2048 ? 2 : 1;
}

// Split-K: a dense call whose output tiles leave at least half of the SMs idle is one chain of
// K / 16 dependent MMAs per tile; cutting K into ranges shortens the chain.  Needs a registered
// workspace, single CTAs and a tile of at most 128 columns.  Returns the number of K ranges.
int plan_splits(const DeviceInfo& di, int M, int N, int block_n, int kb_total, int k_boxes) {
  const long long tiles = static_cast<long long>((M + kBlockM - 1) / kBlockM) * ((N + block_n - 1) / block_n);
  if (!(g_splitk_flags & 2) || !di.sk_ws || block_n > 128 || tiles > kSkMaxTiles || tiles * 2 > di.sm_count ||
      kb_total * k_boxes < kSkMinBlocks)
    return 1;
  int splits = static_cast<int>(di.sm_count / tiles);
  if (splits > kb_total * k_boxes / kSkMinBlocksPerSplit) splits = kb_total * k_boxes / kSkMinBlocksPerSplit;
  if (splits > kSkMaxSplits) splits = kSkMaxSplits;
  const size_t need =
      kSkCounterBytes + static_cast<size_t>(tiles) * splits * kBlockM * block_n * sizeof(float);
  return (splits < 2 || need > di.sk_bytes) ? 1 : splits;
}

// Cluster split-K for a dense store-epilogue call of few rows: 128-wide tiles (the widest whose
// MMA costs the issuing thread no more than a narrow one) and 4 or 2 K ranges per tile, when that
// beats the narrowest-tile choice.  Times in ns from the measured model of one launch:
// fixed 4.9 us, 0.21 us (tiles up to 64 wide) or 0.29 us (128 wide) per 64 elements of K on the
// busiest SM, 4.4 us (4 ranges) or 5.1 us (2 ranges) for the exchange of partial tiles inside the
// cluster: writing the partial tile, the barrier across the cluster (which also absorbs the skew
// between its CTAs), the remote reads, the closing cluster barrier.  With that the form pays from
// K = 3072: K = 4096 18.5 -> 14.3 us, K = 5632 23.6 -> 16.0 us (32 rows, 2048 columns).
struct ClusterSplitPlan {
  int splits;   // 1 = keep the unsplit launch
};
ClusterSplitPlan plan_cluster_split(int M, int N, int kb64, int unsplit_bn, int sm_count) {
  // CDEEP_CLUSTER_SPLITK=0 turns the form off, =2 / =4 force that many ranges (tuning aid)
  static const int forced = [] {
    const char* e = getenv("CDEEP_CLUSTER_SPLITK");
    return e ? atoi(e) : -1;
  }();
  ClusterSplitPlan plan{1};
  if (forced == 0 || !(g_splitk_flags & 1)) return plan;
  const long long m_tiles = (M + kBlockM - 1) / kBlockM;
  auto tiles = [&](int bn) { return m_tiles * ((N + bn - 1) / bn); };
  const long long waves = (tiles(unsplit_bn) + sm_count - 1) / sm_count;
  const long long unsplit_ns = 4900 + waves * kb64 * (unsplit_bn <= 64 ? 210 : (unsplit_bn == 128 ? 290 : 330));
  long long best = unsplit_ns;
  for (int s : {4, 2}) {
    if (forced > 0 && s != forced) continue;
    if (tiles(128) * s > sm_count - sm_count / 8) continue;   // one wave, with room to place whole clusters
    if (kb64 / s < 4) continue;
    const long long ns = 4900 + (s == 4 ? 4400 : 5100) + 310LL * ((kb64 + s - 1) / s);
    if (ns + 500 < best) {
      best = ns;
      plan.splits = s;
    }
  }
  return plan;
}

}  // namespace

bool encode_map_2d(void* map_out, const void* base, long long rows, long long cols, long long ld,
                   int box_rows) {
  return make_map(static_cast<CUtensorMap*>(map_out), base, rows, cols, ld, box_rows);
}

static DeviceInfo* device_info(int* status_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *status_out = cuda_fail(e, "cudaGetDevice");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceInfo& di = g_dev[dev];
  if (di.sm_count == 0) {
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
      *status_out = cuda_fail(e, "cudaDeviceGetAttribute");
      return nullptr;
    }
    void* sp = nullptr;
    e = cudaGetSymbolAddress(&sp, g_status_word);
    if (e != cudaSuccess) {
      *status_out = cuda_fail(e, "cudaGetSymbolAddress(status)");
      return nullptr;
    }
    di.status = static_cast<int*>(sp);
    di.sm_count = sms;
  }
  *status_out = CD_OK;
  return &di;
}

int choose_store_block_n(int M, int N, int num_groups, int sm_count) {
  return store_block_n_impl(M, N, num_groups, sm_count);
}

int current_sm_count() {
  int st;
  DeviceInfo* di = device_info(&st);
  return di ? di->sm_count : 148;
}

int* device_status_word() {
  int st;
  DeviceInfo* di = device_info(&st);
  return di ? di->status : nullptr;
}

int splitk_config(int flags) {
  std::lock_guard<std::mutex> lk(g_mu);
  const int old = g_splitk_flags;
  if (flags >= 0) g_splitk_flags = flags & 3;
  return old;
}

size_t splitk_workspace_bytes() {
  // the counters, then one fp32 partial tile (128 x 128 at most) for every CTA of a full grid
  return kSkCounterBytes + static_cast<size_t>(current_sm_count()) * kBlockM * 128 * sizeof(float);
}

int splitk_workspace_set(void* ws, size_t bytes, cudaStream_t stream) {
  if ((ws == nullptr) != (bytes == 0)) return CD_ERR_INVALID;
  if (ws && ((reinterpret_cast<uintptr_t>(ws) & 15) || bytes < static_cast<size_t>(kSkCounterBytes) + 4096))
    return CD_ERR_INVALID;
  int st;
  DeviceInfo* di = device_info(&st);
  if (!di) return st;
  if (ws) {
    cudaError_t e = cudaMemsetAsync(ws, 0, kSkCounterBytes, stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(split-K counters)");
  }
  std::lock_guard<std::mutex> lk(g_mu);
  di->sk_ws = ws;
  di->sk_bytes = bytes;
  return CD_OK;
}

int splitk_ranges_dense(int M, int N, int K) {
  int st;
  DeviceInfo* di = device_info(&st);
  if (!di || M <= 0 || N <= 0 || K <= 0) return 1;
  const int bn = store_block_n_impl(M, N, 1, di->sm_count);
  if (choose_cta_group(M, bn, di->sm_count) != 1) return 1;
  if (bn <= 128 && choose_cta_group(M, 128, di->sm_count) == 1) {
    const int cs = plan_cluster_split(M, N, (K + kBoxK - 1) / kBoxK, bn, di->sm_count).splits;
    if (cs > 1) return cs;
  }
  const int kblock = kBoxK * gemm_k_boxes(bn, 1);
  return plan_splits(*di, M, N, bn, (K + kblock - 1) / kblock, gemm_k_boxes(bn, 1));
}

int launch_gemm(int M, int N, int num_groups, const int* seg_offsets, const GemmOperand& op0,
                const GemmOperand* op1, const GemmEpilogueArgs& epi, int block_n,
                cudaStream_t stream, const GemmSecond* second) {
  if (M < 0 || N <= 0 || num_groups < 1) return CD_ERR_INVALID;
  if (num_groups > kMaxGroups) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "grouped GEMM: %d row groups, at most %d are supported",
             num_groups, kMaxGroups);
    return CD_ERR_UNSUPPORTED;
  }
  if (block_n != 32 && block_n != 64 && block_n != 128 && block_n != 256) return CD_ERR_INVALID;
  if (num_groups > 1 && !seg_offsets) return CD_ERR_INVALID;
  if (op0.K <= 0 || (op0.K & 7) || (op0.lda & 7) || (op0.ldb & 7)) return CD_ERR_INVALID;
  if (op1 && (op1->K <= 0 || (op1->K & 7) || (op1->lda & 7) || (op1->ldb & 7)))
    return CD_ERR_INVALID;
  if ((epi.ldo & 7) || (epi.out_cols & 7) || (epi.residual && (epi.ldr & 7)))
    return CD_ERR_INVALID;
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!op0.a || !op0.b || (!epi.out && !epi.out_row_ptrs) || !aligned16(op0.a) || !aligned16(op0.b) ||
      !aligned16(epi.out) || !aligned16(epi.residual) || !aligned16(epi.residual2) ||
      !aligned16(epi.bias) || (epi.residual2 && (epi.ldr2 & 7)))
    return CD_ERR_INVALID;
  if (op1 && (!op1->a || !op1->b || !aligned16(op1->a) || !aligned16(op1->b)))
    return CD_ERR_INVALID;
  if (epi.rope_cos && (block_n != 256 || epi.kind != kEpiStore || epi.residual || epi.bias ||
                       epi.residual2 || epi.row_map || epi.out_lo))
    return CD_ERR_UNSUPPORTED;
  // split-bf16 output: plain store epilogue into `out`, no per-row addresses
  if ((epi.out_lo || epi.residual_lo) &&
      (epi.kind != kEpiStore || epi.out_row_ptrs || !epi.out || !aligned16(epi.out_lo) ||
       !aligned16(epi.residual_lo) || (epi.residual_lo && !epi.residual)))
    return CD_ERR_INVALID;
  if (second && (epi.kind != kEpiSwiGLU || op1 || !second->b || !second->out || second->n_rows <= 0 ||
                 (second->ldb & 7) || (second->ldo & 7) || (second->out_cols & 7) ||
                 !aligned16(second->b) || !aligned16(second->out)))
    return CD_ERR_INVALID;
  if (M == 0) return CD_OK;

  int st;
  DeviceInfo* di = device_info(&st);
  if (!di) return st;

  // dense store-epilogue calls of few rows may take the cluster form of split-K (128-wide tiles)
  int csk_splits = 1;
  if (num_groups == 1 && !second && epi.kind == kEpiStore && !epi.rope_cos && !epi.selftest_stall &&
      !epi.out_row_ptrs && block_n <= 128 && choose_cta_group(M, 128, di->sm_count) == 1) {
    const int kb64 = (op0.K + kBoxK - 1) / kBoxK + (op1 ? (op1->K + kBoxK - 1) / kBoxK : 0);
    csk_splits = plan_cluster_split(M, N, kb64, block_n, di->sm_count).splits;
    if (csk_splits > 1) block_n = 128;
  }
  const int cg = choose_cta_group(M, block_n, di->sm_count);
  const int b_box = block_n / cg;
  CUtensorMap a0, b0, a1, b1;
  if (!make_map(&a0, op0.a, M, op0.K, op0.lda, kBlockM) ||
      !make_map(&b0, op0.b, op0.b_rows, op0.K, op0.ldb, b_box)) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed (operand 0)");
    return CD_ERR_CUDA;
  }
  if (op1) {
    if (!make_map(&a1, op1->a, M, op1->K, op1->lda, kBlockM) ||
        !make_map(&b1, op1->b, op1->b_rows, op1->K, op1->ldb, b_box)) {
      snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed (operand 1)");
      return CD_ERR_CUDA;
    }
  } else if (second) {
    a1 = a0;
    if (!make_map(&b1, second->b, second->n_rows, op0.K, second->ldb, b_box)) {
      snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed (second problem)");
      return CD_ERR_CUDA;
    }
  } else {
    a1 = a0;
    b1 = b0;
  }

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M;
  p.N = N;
  p.K0 = op0.K;
  p.K1 = op1 ? op1->K : 0;
  p.num_groups = num_groups;
  p.seg_offsets = seg_offsets;
  p.b0_group_rows = op0.b_group_rows;
  p.b1_group_rows = op1 ? op1->b_group_rows : 0;
  static const int forced_band = [] {   // CDEEP_BAND: m-tiles per scheduling band (tuning aid)
    const char* e = getenv("CDEEP_BAND");
    return e ? atoi(e) : 0;
  }();
  p.band = forced_band > 0 ? forced_band : 16;
  p.out = static_cast<__nv_bfloat16*>(epi.out);
  p.ldo = epi.ldo;
  p.out_cols = epi.out_cols;
  p.row_map = epi.row_map;
  p.out_rows = epi.out_rows;
  p.out_row_ptrs = epi.out_row_ptrs;
  p.residual = static_cast<const __nv_bfloat16*>(epi.residual);
  p.ldr = epi.ldr;
  p.residual_lo = static_cast<const __nv_bfloat16*>(epi.residual_lo);
  p.out_lo = static_cast<__nv_bfloat16*>(epi.out_lo);
  if (second) {
    p.N2 = second->n_rows;
    p.out2 = static_cast<__nv_bfloat16*>(second->out);
    p.ldo2 = second->ldo;
    p.out_cols2 = second->out_cols;
  }
  p.residual2 = static_cast<const __nv_bfloat16*>(epi.residual2);
  p.ldr2 = epi.ldr2;
  p.bias = static_cast<const __nv_bfloat16*>(epi.bias);
  p.bias_lo = epi.bias_lo;
  p.bias_hi = epi.bias_hi;
  p.do_clamp = epi.do_clamp;
  p.clamp_lo = epi.clamp_lo;
  p.clamp_hi = epi.clamp_hi;
  p.rope_cos = epi.rope_cos;
  p.rope_sin = epi.rope_sin;
  p.rope_qw = static_cast<const __nv_bfloat16*>(epi.rope_qw);
  p.rope_kw = static_cast<const __nv_bfloat16*>(epi.rope_kw);
  p.rope_eps = epi.rope_eps;
  p.rope_S = epi.rope_S;
  p.rope_pos0 = epi.rope_pos0;
  p.rope_q_cols = epi.rope_q_cols;
  p.rope_cols = epi.rope_cols;
  p.selftest_stall = epi.selftest_stall;
  p.wait_limit_ns = epi.wait_limit_ns;
  p.status = di->status;

  // Upper bound of the tile count without reading the segment sizes (they live on the
  // device): every group adds at most one partial m-tile.
  const int tile_m = kBlockM * cg;
  const long long n_tiles = (N + block_n - 1) / block_n;
  const long long m_tiles_max = (M + tile_m - 1) / tile_m + (num_groups > 1 ? num_groups : 0);
  long long units = m_tiles_max * n_tiles;           // CTAs (cg = 1) or CTA pairs (cg = 2)
  if (second) units += ((M + tile_m - 1) / tile_m) * ((second->n_rows + block_n - 1) / block_n);
  if (units > di->sm_count / cg) units = di->sm_count / cg;
  if (units < 1) units = 1;

  {
    const int kblock = kBoxK * gemm_k_boxes(block_n, cg);
    const int kb_total = (op0.K + kblock - 1) / kblock + (op1 ? (op1->K + kblock - 1) / kblock : 0);
    const bool eligible = cg == 1 && num_groups == 1 && !second && !epi.rope_cos &&
                          !epi.selftest_stall && (epi.kind != kEpiSwiGLU || block_n >= 64);
    const int splits = (eligible && csk_splits == 1)
                           ? plan_splits(*di, M, N, block_n, kb_total, gemm_k_boxes(block_n, cg)) : 1;
    if (csk_splits > 1) {
      p.splits = csk_splits;
      p.sk_cluster = 1;
      units = ((M + kBlockM - 1) / kBlockM) * n_tiles * csk_splits;   // one unit per CTA, clusters of `splits`
    } else if (splits > 1) {
      p.splits = splits;
      p.sk_counters = static_cast<int*>(di->sk_ws);
      p.sk_scratch = reinterpret_cast<float*>(static_cast<char*>(di->sk_ws) + kSkCounterBytes);
      units = ((M + kBlockM - 1) / kBlockM) * n_tiles * splits;
    }
  }
  const int grid = static_cast<int>(units) * cg;

  cudaError_t e;
  std::lock_guard<std::mutex> lk(g_mu);
  const int kind = epi.rope_cos ? static_cast<int>(kEpiStoreRope)
                   : (epi.out_lo || epi.residual_lo) ? static_cast<int>(kEpiStoreSplit) : epi.kind;
  e = (cg == 2) ? launch_any<2>(block_n, kind, grid, a0, b0, a1, b1, p, *di, stream)
                : launch_any<1>(block_n, kind, grid, a0, b0, a1, b1, p, *di, stream);
  if (e != cudaSuccess) return cuda_fail(e, "gemm launch");
  return CD_OK;
}

}  // namespace cdeep
