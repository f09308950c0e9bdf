// extern "C" entry points of libcdeep.so (declared in include/cdeep.h).
#include <cstdio>
#include <cuda_runtime.h>
#include "../../include/cdeep.h"
#include "gemm_sm100.cuh"
#include "checks.cuh"
#include "kernels.h"

namespace cdeep {
thread_local char g_cuda_err[256] = "";
int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return CD_ERR_CUDA;
}
}  // namespace cdeep

using namespace cdeep;

static inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" {

int cd_version(void) { return 3; }

const char* cd_error_string(int status) {
  switch (status) {
    case CD_OK: return "ok";
    case CD_ERR_INVALID: return "invalid argument";
    case CD_ERR_CUDA: return "CUDA call failed";
    case CD_ERR_UNSUPPORTED: return "unsupported shape";
    case CD_ERR_TIMEOUT: return "a kernel gave up on a bounded wait";
    case CD_ERR_BOUNDS: return "checking build: a kernel met an index, address or segment table out of range";
    default: return "unknown status";
  }
}

const char* cd_last_cuda_error(void) { return g_cuda_err; }

int cd_max_groups(void) { return kMaxGroups; }

int cd_checks_enabled(void) { return kChecks ? 1 : 0; }

size_t cd_splitk_workspace_bytes(void) { return splitk_workspace_bytes(); }

int cd_splitk_config(int flags) { return splitk_config(flags); }

int cd_splitk_ranges(int T, int K, int N) { return splitk_ranges_dense(T, N, K); }

int cd_splitk_workspace_set(void* workspace, size_t bytes, void* stream) {
  return splitk_workspace_set(workspace, bytes, as_stream(stream));
}

int cd_status_fetch(int* h_status) {
  if (!h_status) return CD_ERR_INVALID;
  int* d = device_status_word();
  if (!d) return CD_ERR_CUDA;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
  e = cudaMemcpy(h_status, d, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
  if (*h_status != 0) {
    e = cudaMemset(d, 0, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(status)");
  }
  return CD_OK;
}

int cd_selftest_wait_timeout(const void* a, const void* b, void* out, int limit_ms, void* stream) {
  if (!a || !b || !out || limit_ms < 1 || limit_ms > 1000) return CD_ERR_INVALID;
  GemmOperand op0{};
  op0.a = a;
  op0.lda = 64;
  op0.b = b;
  op0.ldb = 64;
  op0.b_rows = 128;
  op0.K = 64;
  GemmEpilogueArgs epi{};
  epi.kind = kEpiStore;
  epi.out = out;
  epi.ldo = 128;
  epi.out_cols = 128;
  epi.selftest_stall = 1;
  epi.wait_limit_ns = static_cast<unsigned long long>(limit_ms) * 1000000ull;
  return launch_gemm(128, 128, 1, nullptr, op0, nullptr, epi, 128, as_stream(stream));
}

size_t cd_route_workspace_bytes(int T, int E) {
  if (T < 0 || E < 1) return 0;
  return route_workspace_bytes(T, E);
}

int cd_route(const int64_t* ids, const int64_t* table, int V, int E, int T, int32_t* expert_ids,
             int32_t* counts, int32_t* offsets, int32_t* perm, int32_t* inv_perm, void* ws,
             size_t ws_bytes, void* stream) {
  if (T < 0 || V < 1 || E < 1 || E > 256) return CD_ERR_INVALID;
  if (!table || !counts || !offsets || !ws) return CD_ERR_INVALID;
  if (T > 0 && (!ids || !expert_ids || !perm || !inv_perm)) return CD_ERR_INVALID;
  if (ws_bytes < route_workspace_bytes(T, E)) return CD_ERR_INVALID;
  cudaError_t e = launch_route(reinterpret_cast<const long long*>(ids),
                               reinterpret_cast<const long long*>(table), V, E, T, expert_ids,
                               counts, offsets, perm, inv_perm, static_cast<int*>(ws),
                               as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "route launch");
}

int cd_rmsnorm(const void* x, const void* residual, const void* weight, float eps, void* sum_out,
               void* out, const int32_t* dst_rows, int T, int H, void* stream) {
  if (T < 0 || H < 1 || !weight) return CD_ERR_INVALID;
  if (T > 0 && (!x || !out)) return CD_ERR_INVALID;
  if (sum_out && (!residual || sum_out == x)) return CD_ERR_INVALID;
  if ((H & 7) == 0 && !(aligned16(x) && aligned16(residual) && aligned16(weight) &&
                        aligned16(sum_out) && aligned16(out)))
    return CD_ERR_INVALID;
  cudaError_t e = launch_rmsnorm(x, residual, weight, eps, sum_out, out, dst_rows, T, H,
                                 as_stream(stream), false);
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "rmsnorm launch");
}

int cd_rmsnorm_split(const void* x_hi, const void* x_lo, const void* weight, float eps, void* out,
                     const int32_t* dst_rows, int T, int H, void* stream) {
  if (T < 0 || H < 1 || !weight) return CD_ERR_INVALID;
  if (T > 0 && (!x_hi || !out)) return CD_ERR_INVALID;
  if ((H & 7) == 0 && !(aligned16(x_hi) && aligned16(x_lo) && aligned16(weight) && aligned16(out)))
    return CD_ERR_INVALID;
  cudaError_t e = launch_rmsnorm(x_hi, x_lo, weight, eps, nullptr, out, dst_rows, T, H,
                                 as_stream(stream), true);
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "rmsnorm launch");
}

int cd_gather_rows(const void* x, const int32_t* src_rows, void* out, int T, int H, void* stream) {
  if (T < 0 || H < 1) return CD_ERR_INVALID;
  if (T > 0 && (!x || !src_rows || !out)) return CD_ERR_INVALID;
  if ((H & 7) == 0 && !(aligned16(x) && aligned16(out))) return CD_ERR_INVALID;
  cudaError_t e = launch_gather_rows(x, src_rows, out, T, H, as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "gather launch");
}

int cd_qk_norm_rope(void* qkv, const void* q_w, const void* k_w, const float* cos_t,
                    const float* sin_t, float eps, int T, int S, int pos0, int hq, int hkv, int D,
                    void* stream) {
  if (T < 0 || S < 1 || pos0 < 0 || hq < 1 || hkv < 1 || D < 4 || (D & 3)) return CD_ERR_INVALID;
  if (!cos_t || !sin_t || (T > 0 && !qkv)) return CD_ERR_INVALID;
  if ((q_w == nullptr) != (k_w == nullptr)) return CD_ERR_INVALID;
  cudaError_t e = launch_qk_norm_rope(qkv, q_w, k_w, cos_t, sin_t, eps, T, S, pos0, hq, hkv, D,
                                      as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "qk_norm_rope launch");
}

int cd_decode_rope_append(void* qkv, const void* q_w, const void* k_w, const float* cos_t,
                          const float* sin_t, float eps, int B, int hq, int hkv, int D,
                          void* k_cache, void* v_cache, long long kv_stride_b,
                          long long kv_stride_h, long long kv_stride_t, int capacity,
                          const int32_t* pos_dev, void* stream) {
  if (B < 0 || hq < 1 || hkv < 1 || D < 8 || (D & 7) || capacity < 1) return CD_ERR_INVALID;
  if (!cos_t || !sin_t || !pos_dev || !k_cache || !v_cache || (B > 0 && !qkv))
    return CD_ERR_INVALID;
  if ((q_w == nullptr) != (k_w == nullptr)) return CD_ERR_INVALID;
  if (!aligned16(qkv) || !aligned16(k_cache) || !aligned16(v_cache)) return CD_ERR_INVALID;
  if ((kv_stride_b & 7) || (kv_stride_h & 7) || (kv_stride_t & 7)) return CD_ERR_INVALID;
  cudaError_t e = launch_qk_norm_rope(qkv, q_w, k_w, cos_t, sin_t, eps, B, 1, 0, hq, hkv, D,
                                      as_stream(stream), pos_dev, k_cache, v_cache, kv_stride_b,
                                      kv_stride_h, kv_stride_t, capacity);
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "decode rope/append launch");
}

size_t cd_decode_attention_workspace_bytes(int B, int hq, int hkv, int L, int D) {
  if (B < 1 || hq < 1 || hkv < 1 || L < 1 || D < 1 || hq % hkv) return 0;
  return decode_attention_workspace_bytes(B, hq, hkv, L, D);
}

int cd_decode_attention(const void* q, long long q_stride_b, const void* k, const void* v,
                        long long kv_stride_b, long long kv_stride_h, long long kv_stride_t,
                        const void* mask, long long mask_stride_b, float scale, int B, int hq,
                        int hkv, int L, const int32_t* kv_len_dev, int D, void* out, void* ws,
                        size_t ws_bytes, void* stream) {
  if (B < 1 || hq < 1 || hkv < 1 || L < 1 || hq % hkv) return CD_ERR_INVALID;
  if (D != 64 && D != 128) return CD_ERR_UNSUPPORTED;
  if (hq / hkv > 4) return CD_ERR_UNSUPPORTED;
  if (!q || !k || !v || !out || !ws) return CD_ERR_INVALID;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return CD_ERR_INVALID;
  if ((q_stride_b & 7) || (kv_stride_b & 7) || (kv_stride_h & 7) || (kv_stride_t & 7))
    return CD_ERR_INVALID;
  if (ws_bytes < decode_attention_workspace_bytes(B, hq, hkv, L, D)) return CD_ERR_INVALID;
  cudaError_t e = launch_decode_attention(q, q_stride_b, k, v, kv_stride_b, kv_stride_h,
                                          kv_stride_t, mask, mask_stride_b, scale, B, hq, hkv, L,
                                          D, out, ws, as_stream(stream), kv_len_dev);
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "decode attention launch");
}

int cd_attention_prefill_supported(int B, int S, int hq, int hkv, int D) {
  if (B < 1 || S < 1 || hq < 1 || hkv < 1 || hq % hkv) return 0;
  if (D != 64 && D != 128) return 0;
  if (static_cast<long long>(B) * S > 0x7fffffffLL - 256) return 0;   // token rows are 32-bit TMA coordinates
  return 1;
}

int cd_attention_prefill(const void* qkv, void* out, int B, int S, int hq, int hkv, int D,
                         float scale, void* stream) {
  if (!cd_attention_prefill_supported(B, S, hq, hkv, D)) return CD_ERR_UNSUPPORTED;
  if (!qkv || !out || !aligned16(qkv) || !aligned16(out) || !(scale > 0.f)) return CD_ERR_INVALID;
  int* status = device_status_word();
  if (!status) return CD_ERR_CUDA;
  cudaError_t e = launch_attention_prefill(qkv, out, B, S, hq, hkv, D, scale, status,
                                           as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "prefill attention launch");
}

int cd_gate_up_packed_rows(int I, int block_n) {
  if (I < 1 || (block_n != 32 && block_n != 64 && block_n != 128 && block_n != 256)) return 0;
  const int half = block_n / 2;
  return ((I + half - 1) / half) * block_n;
}

int cd_pack_gate_up(const void* gate, const void* up, void* packed, int G, int I, int H,
                    int block_n, int feature_major, void* stream) {
  if (G < 1 || I < 1 || H < 1 || !gate || !up || !packed) return CD_ERR_INVALID;
  if (cd_gate_up_packed_rows(I, block_n) == 0 || 2 * G > 65535) return CD_ERR_INVALID;
  cudaError_t e = launch_pack_gate_up(gate, up, packed, G, I, H, block_n, feature_major ? 1 : 0,
                                      as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "pack_gate_up launch");
}

int cd_pack_down(const void* down, void* packed, int E, int I, int H, void* stream) {
  if (E < 1 || E > 65535 || I < 1 || H < 1 || !down || !packed) return CD_ERR_INVALID;
  cudaError_t e = launch_transpose(down, packed, E, I, H, as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "pack_down launch");
}

int cd_moe_up(const void* x_sorted, const int32_t* seg_offsets, int num_groups,
              const void* packed_w, void* h, int T, int H, int I, int block_n, void* stream) {
  if (T < 0 || H < 8 || I < 8 || (H & 7) || (I & 7) || num_groups < 1) return CD_ERR_INVALID;
  const int rows = cd_gate_up_packed_rows(I, block_n);
  if (rows == 0) return CD_ERR_INVALID;
  GemmOperand op{};
  op.a = x_sorted;
  op.lda = H;
  op.b = packed_w;
  op.ldb = H;
  op.b_rows = static_cast<long long>(rows) * num_groups;
  op.b_group_rows = rows;
  op.K = H;
  GemmEpilogueArgs epi{};
  epi.kind = kEpiSwiGLU;
  epi.out = h;
  epi.ldo = I;
  epi.out_cols = I;
  return launch_gemm(T, rows, num_groups, seg_offsets, op, nullptr, epi, block_n,
                     as_stream(stream));
}

int cd_moe_up_pair(const void* x_sorted, const int32_t* seg_offsets, int num_groups,
                   const void* packed_w, void* h, int I, const void* packed_shared, void* h_shared,
                   int I_s, int T, int H, int block_n, void* stream) {
  if (T < 0 || H < 8 || I < 8 || I_s < 8 || (H & 7) || (I & 7) || (I_s & 7) || num_groups < 1)
    return CD_ERR_INVALID;
  const int rows = cd_gate_up_packed_rows(I, block_n);
  const int rows_s = cd_gate_up_packed_rows(I_s, block_n);
  if (rows == 0 || rows_s == 0 || !packed_shared || !h_shared) return CD_ERR_INVALID;
  GemmOperand op{};
  op.a = x_sorted;
  op.lda = H;
  op.b = packed_w;
  op.ldb = H;
  op.b_rows = static_cast<long long>(rows) * num_groups;
  op.b_group_rows = rows;
  op.K = H;
  GemmEpilogueArgs epi{};
  epi.kind = kEpiSwiGLU;
  epi.out = h;
  epi.ldo = I;
  epi.out_cols = I;
  GemmSecond sec{};
  sec.b = packed_shared;
  sec.ldb = H;
  sec.n_rows = rows_s;
  sec.out = h_shared;
  sec.ldo = I_s;
  sec.out_cols = I_s;
  return launch_gemm(T, rows, num_groups, seg_offsets, op, nullptr, epi, block_n,
                     as_stream(stream), &sec);
}

int cd_moe_down(const void* h_routed, int I_e, const void* wd_routed, const void* h_shared,
                int I_s, const void* wd_shared, const int32_t* seg_offsets, int E,
                const int32_t* row_map, const void* residual, const void* residual_lo, void* out,
                void* out_lo, int T, int H, void* stream) {
  if (T < 0 || H < 8 || (H & 7) || I_e < 8 || (I_e & 7) || E < 1) return CD_ERR_INVALID;
  if ((h_shared == nullptr) != (wd_shared == nullptr)) return CD_ERR_INVALID;
  if (h_shared && (I_s < 8 || (I_s & 7))) return CD_ERR_INVALID;
  GemmOperand op0{};
  op0.a = h_routed;
  op0.lda = I_e;
  op0.b = wd_routed;
  op0.ldb = I_e;
  op0.b_rows = static_cast<long long>(E) * H;
  op0.b_group_rows = H;
  op0.K = I_e;
  GemmOperand op1{};
  if (h_shared) {
    op1.a = h_shared;
    op1.lda = I_s;
    op1.b = wd_shared;
    op1.ldb = I_s;
    op1.b_rows = H;
    op1.b_group_rows = 0;
    op1.K = I_s;
  }
  GemmEpilogueArgs epi{};
  epi.kind = kEpiStore;
  epi.out = out;
  epi.ldo = H;
  epi.out_cols = H;
  epi.row_map = row_map;
  epi.out_rows = T;
  epi.residual = residual;
  epi.ldr = H;
  epi.residual_lo = residual_lo;
  epi.out_lo = out_lo;
  return launch_gemm(T, H, E, seg_offsets, op0, h_shared ? &op1 : nullptr, epi,
                     choose_store_block_n(T, H, E, current_sm_count()), as_stream(stream));
}

int cd_push_rows(const void* x, const int32_t* src_rows, const int32_t* offsets,
                 const int32_t* push_base, int E, int experts_per_rank, const uint64_t* peer_ptrs,
                 int T, int H, void* stream) {
  if (T < 0 || H < 8 || (H & 7) || E < 1 || E > 256 || experts_per_rank < 1 ||
      E % experts_per_rank)
    return CD_ERR_INVALID;
  if (!offsets || !push_base || !peer_ptrs || (T > 0 && !x) || !aligned16(x)) return CD_ERR_INVALID;
  cudaError_t e = launch_push_rows(x, src_rows, offsets, push_base, E, experts_per_rank,
                                   reinterpret_cast<const unsigned long long*>(peer_ptrs), T, H,
                                   as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "push_rows launch");
}

int cd_ep_plan(const int32_t* counts, int world, int num_experts, int experts_per_rank, int rank,
               const int64_t* ret_ptrs, int64_t row_bytes, int capacity, int32_t* push_base,
               int32_t* seg_offsets, int64_t* row_ptrs, void* stream) {
  if (!counts || !ret_ptrs || !push_base || !seg_offsets || !row_ptrs || capacity < 0 ||
      row_bytes <= 0 || rank < 0 || rank >= world)
    return CD_ERR_INVALID;
  if (!ep_plan_supported(world, num_experts, experts_per_rank)) {
    snprintf(g_cuda_err, sizeof(g_cuda_err),
             "cd_ep_plan: %d ranks x %d experts (%d per rank) is outside what one launch holds",
             world, num_experts, experts_per_rank);
    return CD_ERR_UNSUPPORTED;
  }
  cudaError_t e = launch_ep_plan(counts, world, num_experts, experts_per_rank, rank,
                                 reinterpret_cast<const long long*>(ret_ptrs), row_bytes, capacity,
                                 push_base, seg_offsets, reinterpret_cast<long long*>(row_ptrs),
                                 as_stream(stream));
  if (e != cudaSuccess) return cuda_fail(e, "ep_plan launch");
  return CD_OK;
}

int cd_peer_put_i32(const int32_t* src, int n, const uint64_t* peer_bufs, int world, int64_t offset,
                    void* stream) {
  if (!src || !peer_bufs || n < 0 || world < 1 || world > 64 || offset < 0) return CD_ERR_INVALID;
  cudaError_t e = launch_peer_put_i32(src, n, reinterpret_cast<const unsigned long long*>(peer_bufs),
                                      world, offset, as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "peer_put launch");
}

int cd_peer_barrier(const uint64_t* peer_flags, int32_t* flags, int rank, int world, int limit_ms,
                    void* stream) {
  if (!peer_flags || !flags || world < 1 || world > 64 || rank < 0 || rank >= world ||
      limit_ms < 1 || limit_ms > 60000)
    return CD_ERR_INVALID;
  int* status = device_status_word();
  if (!status) return CD_ERR_CUDA;
  cudaError_t e = launch_peer_barrier(reinterpret_cast<const unsigned long long*>(peer_flags), flags,
                                      rank, world, static_cast<unsigned long long>(limit_ms) * 1000000ull,
                                      status, as_stream(stream));
  return e == cudaSuccess ? CD_OK : cuda_fail(e, "peer_barrier launch");
}

int cd_moe_down_push(const void* h_routed, int I_e, const void* wd_routed,
                     const int32_t* seg_offsets, int E, const int64_t* out_row_ptrs, int T, int H,
                     void* stream) {
  if (T < 0 || H < 8 || (H & 7) || I_e < 8 || (I_e & 7) || E < 1 || !out_row_ptrs)
    return CD_ERR_INVALID;
  GemmOperand op0{};
  op0.a = h_routed;
  op0.lda = I_e;
  op0.b = wd_routed;
  op0.ldb = I_e;
  op0.b_rows = static_cast<long long>(E) * H;
  op0.b_group_rows = H;
  op0.K = I_e;
  GemmEpilogueArgs epi{};
  epi.kind = kEpiStore;
  epi.out = nullptr;
  epi.ldo = H;
  epi.out_cols = H;
  epi.out_row_ptrs = reinterpret_cast<const long long*>(out_row_ptrs);
  return launch_gemm(T, H, E, seg_offsets, op0, nullptr, epi,
                     choose_store_block_n(T, H, E, current_sm_count()), as_stream(stream));
}

int cd_moe_combine(const void* h_shared, int I_s, const void* wd_shared, const void* routed_sorted,
                   const int32_t* row_map, const void* residual, const void* residual_lo, void* out,
                   void* out_lo, int T, int H, void* stream) {
  if (T < 0 || H < 8 || (H & 7) || I_s < 8 || (I_s & 7)) return CD_ERR_INVALID;
  if (!h_shared || !wd_shared) return CD_ERR_INVALID;
  GemmOperand op0{};
  op0.a = h_shared;
  op0.lda = I_s;
  op0.b = wd_shared;
  op0.ldb = I_s;
  op0.b_rows = H;
  op0.K = I_s;
  GemmEpilogueArgs epi{};
  epi.kind = kEpiStore;
  epi.out = out;
  epi.ldo = H;
  epi.out_cols = H;
  epi.row_map = row_map;
  epi.out_rows = T;
  epi.residual = residual;
  epi.ldr = H;
  epi.residual_lo = residual_lo;
  epi.out_lo = out_lo;
  epi.residual2 = routed_sorted;
  epi.ldr2 = H;
  return launch_gemm(T, H, 1, nullptr, op0, nullptr, epi,
                     choose_store_block_n(T, H, 1, current_sm_count()), as_stream(stream));
}

int cd_mu_qkv(const void* x, const void* mu_prev, const void* w, const void* w_mu, void* qkv,
              int T, int H, int N, void* stream) {
  if (T < 0 || H < 8 || (H & 7) || N < 8 || (N & 7)) return CD_ERR_INVALID;
  if ((mu_prev == nullptr) != (w_mu == nullptr)) return CD_ERR_INVALID;
  GemmOperand op0{};
  op0.a = x;
  op0.lda = H;
  op0.b = w;
  op0.ldb = H;
  op0.b_rows = N;
  op0.K = H;
  GemmOperand op1{};
  if (mu_prev) {
    op1.a = mu_prev;
    op1.lda = H;
    op1.b = w_mu;
    op1.ldb = H;
    op1.b_rows = N;
    op1.K = H;
  }
  GemmEpilogueArgs epi{};
  epi.kind = kEpiStore;
  epi.out = qkv;
  epi.ldo = N;
  epi.out_cols = N;
  return launch_gemm(T, N, 1, nullptr, op0, mu_prev ? &op1 : nullptr, epi,
                     choose_store_block_n(T, N, 1, current_sm_count()), as_stream(stream));
}

int cd_mu_qkv_rope_supported(int T, int N, int hq, int hkv, int D) {
  if (T < 1 || N < 8 || hq < 1 || hkv < 1) return 0;
  if (D != 128 || N != (hq + 2 * hkv) * D) return 0;
  if ((hq * D) % 256 || ((hq + hkv) * D) % 256) return 0;     // heads aligned to 256-wide tiles
  return choose_store_block_n(T, N, 1, current_sm_count()) == 256 ? 1 : 0;
}

int cd_mu_qkv_rope(const void* x, const void* mu_prev, const void* w, const void* w_mu, void* qkv,
                   int T, int H, int N, const void* q_w, const void* k_w, const float* cos_t,
                   const float* sin_t, float eps, int S, int pos0, int hq, int hkv, int D,
                   void* stream) {
  if (T < 0 || H < 8 || (H & 7) || N < 8 || (N & 7) || S < 1 || pos0 < 0) return CD_ERR_INVALID;
  if ((mu_prev == nullptr) != (w_mu == nullptr)) return CD_ERR_INVALID;
  if ((q_w == nullptr) != (k_w == nullptr) || !cos_t || !sin_t) return CD_ERR_INVALID;
  if (!aligned16(cos_t) || !aligned16(sin_t) || !aligned16(q_w) || !aligned16(k_w))
    return CD_ERR_INVALID;
  if (T > 0 && !cd_mu_qkv_rope_supported(T, N, hq, hkv, D)) return CD_ERR_UNSUPPORTED;
  GemmOperand op0{};
  op0.a = x;
  op0.lda = H;
  op0.b = w;
  op0.ldb = H;
  op0.b_rows = N;
  op0.K = H;
  GemmOperand op1{};
  if (mu_prev) {
    op1.a = mu_prev;
    op1.lda = H;
    op1.b = w_mu;
    op1.ldb = H;
    op1.b_rows = N;
    op1.K = H;
  }
  GemmEpilogueArgs epi{};
  epi.kind = kEpiStore;
  epi.out = qkv;
  epi.ldo = N;
  epi.out_cols = N;
  epi.rope_cos = cos_t;
  epi.rope_sin = sin_t;
  epi.rope_qw = q_w;
  epi.rope_kw = k_w;
  epi.rope_eps = eps;
  epi.rope_S = S;
  epi.rope_pos0 = pos0;
  epi.rope_q_cols = hq * D;
  epi.rope_cols = (hq + hkv) * D;
  return launch_gemm(T, N, 1, nullptr, op0, mu_prev ? &op1 : nullptr, epi, 256, as_stream(stream));
}

int cd_mu_proj(const void* h, const void* w, const void* mu_param, float mu_min, float mu_max,
               int clamp_out, float out_lo, float out_hi, void* out, int T, int H, void* stream) {
  if (T < 0 || H < 8 || (H & 7) || !mu_param) return CD_ERR_INVALID;
  GemmOperand op0{};
  op0.a = h;
  op0.lda = H;
  op0.b = w;
  op0.ldb = H;
  op0.b_rows = H;
  op0.K = H;
  GemmEpilogueArgs epi{};
  epi.kind = kEpiStore;
  epi.out = out;
  epi.ldo = H;
  epi.out_cols = H;
  epi.bias = mu_param;
  epi.bias_lo = mu_min;
  epi.bias_hi = mu_max;
  epi.do_clamp = clamp_out;
  epi.clamp_lo = out_lo;
  epi.clamp_hi = out_hi;
  return launch_gemm(T, H, 1, nullptr, op0, nullptr, epi,
                     choose_store_block_n(T, H, 1, current_sm_count()), as_stream(stream));
}

int cd_linear(const void* x, const void* w, const void* residual, const void* residual_lo,
              void* out, void* out_lo, int T, int K, int N, void* stream) {
  if (T < 0 || K < 8 || (K & 7) || N < 8 || (N & 7)) return CD_ERR_INVALID;
  GemmOperand op0{};
  op0.a = x;
  op0.lda = K;
  op0.b = w;
  op0.ldb = K;
  op0.b_rows = N;
  op0.K = K;
  GemmEpilogueArgs epi{};
  epi.kind = kEpiStore;
  epi.out = out;
  epi.ldo = N;
  epi.out_cols = N;
  epi.residual = residual;
  epi.ldr = N;
  epi.residual_lo = residual_lo;
  epi.out_lo = out_lo;
  return launch_gemm(T, N, 1, nullptr, op0, nullptr, epi,
                     choose_store_block_n(T, N, 1, current_sm_count()), as_stream(stream));
}

}  // extern "C"
