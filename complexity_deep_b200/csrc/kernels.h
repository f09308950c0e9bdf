// Internal launch functions shared by the translation units of libcdeep.so.
#pragma once
#include <cstddef>
#include <cstdlib>
#include <cuda_runtime.h>

namespace cdeep {

// Programmatic dependent launch is on unless CDEEP_PDL=0 (tuning / debugging aid).
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("CDEEP_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

// <<<grid, block, smem, stream>>> with programmatic stream serialisation allowed (see
// griddep_wait in ptx.cuh: every kernel waits for its predecessor before touching memory).
template <typename... P, typename... A>
inline cudaError_t launch_kernel(void (*kern)(P...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<A&&>(args)...);
}

size_t route_workspace_bytes(int T, int E);
cudaError_t launch_route(const long long* ids, const long long* table, int V, int E, int T,
                         int* expert_ids, int* counts, int* offsets, int* perm, int* inv_perm,
                         int* block_hist, cudaStream_t stream);

// split = false: h = bf16(x + residual) as the reference's bf16 residual add; split = true:
// `residual` is the low part of a split-bf16 value and h = x + residual is kept in fp32.
cudaError_t launch_rmsnorm(const void* x, const void* residual, const void* weight, float eps,
                           void* sum_out, void* out, const int* dst_rows, int T, int H,
                           cudaStream_t stream, bool split);
cudaError_t launch_gather_rows(const void* x, const int* src_rows, void* out, int T, int H,
                               cudaStream_t stream);
cudaError_t launch_push_rows(const void* x, const int* src_rows, const int* offsets,
                             const int* push_base, int E, int experts_per_rank,
                             const unsigned long long* peer_ptrs, int T, int H,
                             cudaStream_t stream);
cudaError_t launch_peer_barrier(const unsigned long long* peer_flags, int* flags, int rank, int world,
                                unsigned long long limit_ns, int* status, cudaStream_t stream);
// pos_dev / k_cache / v_cache: decode-step form (position from device memory, rotated k and v
// also written to the cache at that position); all null for the plain in-place form.
cudaError_t launch_qk_norm_rope(void* qkv, const void* q_w, const void* k_w, const float* cos_t,
                                const float* sin_t, float eps, int T, int S, int pos0, int hq,
                                int hkv, int D, cudaStream_t stream, const int* pos_dev = nullptr,
                                void* k_cache = nullptr, void* v_cache = nullptr,
                                long long kv_stride_b = 0, long long kv_stride_h = 0,
                                long long kv_stride_t = 0, int capacity = 0);

// exchange plan of the expert-parallel layer (ep_plan.cu)
bool ep_plan_supported(int G, int E, int El);
cudaError_t launch_ep_plan(const int* counts, int G, int E, int El, int rank,
                           const long long* ret_ptrs, long long row_bytes, int capacity,
                           int* push_base, int* seg_offsets, long long* row_ptrs,
                           cudaStream_t stream);

cudaError_t launch_peer_put_i32(const int* src, int n, const unsigned long long* peer_bufs, int world,
                                long long offset, cudaStream_t stream);

// split-K workspace of the current device (gemm.cu)
size_t splitk_workspace_bytes();
int splitk_workspace_set(void* ws, size_t bytes, cudaStream_t stream);
int splitk_ranges_dense(int M, int N, int K);
int splitk_config(int flags);   // sets which forms of split-K may be used (negative: query); returns the previous flags   // K ranges a dense store-epilogue call would use now

// Encodes a CUtensorMap (passed as void*) for a 2-D bf16 tensor [rows, cols] with `ld` elements
// between rows, boxes of [box_rows, 64 columns], 128-byte swizzle, zero fill out of bounds.
bool encode_map_2d(void* map_out, const void* base, long long rows, long long cols, long long ld,
                   int box_rows);

// causal prefill attention over the fused projection buffer (attention_prefill.cu)
cudaError_t launch_attention_prefill(const void* qkv, void* out, int B, int S, int hq, int hkv, int D,
                                     float scale, int* status, cudaStream_t stream);

// weight layout transforms (pack.cu)
cudaError_t launch_pack_gate_up(const void* gate, const void* up, void* packed, int G, int I, int H,
                                int block_n, int feature_major, cudaStream_t stream);
cudaError_t launch_transpose(const void* in, void* out, int G, int R, int C, cudaStream_t stream);

size_t decode_attention_workspace_bytes(int B, int hq, int hkv, int L, int D);
cudaError_t launch_decode_attention(const void* q, long long q_stride_b, const void* k,
                                    const void* v, long long kv_stride_b, long long kv_stride_h,
                                    long long kv_stride_t, const void* mask,
                                    long long mask_stride_b, float scale, int B, int hq, int hkv,
                                    int L, int D, void* out, void* ws, cudaStream_t stream,
                                    const int* kv_len_dev = nullptr);

// One operand pair of the GEMM: row-major bf16 matrices with K contiguous.
struct GemmOperand {
  const void* a;   // [M, K], leading dimension lda
  long long lda;
  const void* b;   // [groups * n_rows or n_rows, K], leading dimension ldb
  long long ldb;
  long long b_rows;      // total rows of b (bounds of the tensor map)
  int b_group_rows;      // row offset per group, 0 when every group uses the same rows
  int K;
};

struct GemmEpilogueArgs {
  int kind;                // GemmEpilogue
  void* out;
  int ldo;
  int out_cols;
  const int* row_map;
  int out_rows;            // rows of the destination buffer (checking build: bound of row_map entries; 0 = unknown)
  const long long* out_row_ptrs;  // per sorted row: address of its destination row (may be peer memory)
  const void* residual;
  int ldr;
  const void* residual_lo;  // low part of a split-bf16 residual (same indexing as residual)
  void* out_lo;             // low part of the result (same indexing as out); selects the split epilogue
  const void* residual2;   // indexed by the un-mapped row
  int ldr2;
  const void* bias;
  float bias_lo, bias_hi;
  int do_clamp;
  float clamp_lo, clamp_hi;
  // failure-path self-test (see GemmParams)
  int selftest_stall;
  unsigned long long wait_limit_ns;
  // optional fused Q/K RMSNorm + RoPE (see GemmParams)
  const float* rope_cos;
  const float* rope_sin;
  const void* rope_qw;
  const void* rope_kw;
  float rope_eps;
  int rope_S, rope_pos0, rope_q_cols, rope_cols;
};

// Optional second, dense problem of a SwiGLU launch: h2[M, :cols] from the same A rows against
// its own packed gate/up weights; its tiles run in the same launch after the grouped ones.
struct GemmSecond {
  const void* b;      // [n_rows, K] packed gate/up rows (K = the first operand's K, leading dimension ldb)
  long long ldb;
  int n_rows;         // accumulator columns
  void* out;
  int ldo;
  int out_cols;
};

// Returns a CD_* status code.
int launch_gemm(int M, int N, int num_groups, const int* seg_offsets, const GemmOperand& op0,
                const GemmOperand* op1, const GemmEpilogueArgs& epi, int block_n,
                cudaStream_t stream, const GemmSecond* second = nullptr);

int choose_store_block_n(int M, int N, int num_groups, int sm_count);  // SM count of the current device
int current_sm_count();
int* device_status_word();  // per-device word the kernels raise when a bounded wait ran out

extern thread_local char g_cuda_err[256];        // text behind cd_last_cuda_error()
int cuda_fail(cudaError_t e, const char* what);  // records the text, returns CD_ERR_CUDA

}  // namespace cdeep
