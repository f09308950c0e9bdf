// Checking build (-DCDEEP_CHECKS, libcdeep_checks.so): indices and addresses that a kernel takes
// from DEVICE memory (row maps, row addresses, segment offsets) are validated before use.  A bad
// entry raises the device status word to kStatusBounds and the access is skipped, so a wrong
// index from the caller shows up as a status from cd_status_fetch instead of a wild store.  In
// the normal build kChecks is false and the checks compile to nothing.
#pragma once

namespace cdeep {

#ifdef CDEEP_CHECKS
constexpr bool kChecks = true;
#else
constexpr bool kChecks = false;
#endif

constexpr int kStatusWaitTimeout = 1;   // a bounded pipeline wait ran out
constexpr int kStatusPeerTimeout = 2;   // the barrier between GPUs ran out
constexpr int kStatusBounds = 4;        // checking build: an index / address / segment table was invalid

// true when 0 <= v < n (always true in the normal build)
__device__ __forceinline__ bool index_ok(int v, int n, int* status) {
  if constexpr (!kChecks) return true;
  if (v >= 0 && v < n) return true;
  if (status) atomicMax(status, kStatusBounds);
  return false;
}

// true when the address is usable for 16-byte stores (always true in the normal build)
__device__ __forceinline__ bool row_address_ok(long long addr, int* status) {
  if constexpr (!kChecks) return true;
  if (addr != 0 && (addr & 15) == 0) return true;
  if (status) atomicMax(status, kStatusBounds);
  return false;
}

}  // namespace cdeep
