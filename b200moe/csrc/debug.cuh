// Checked build (-DB200MOE_DEBUG): data-dependent indices are range-checked before they are used as a row, a
// slot or a peer; the first violation is recorded (code, value, bound, block) in a per-file device record and
// the access is skipped.  In the normal build every check compiles to nothing.  compute-sanitizer style tools
// are not needed to use it: the host reads the record through b2_<file>_debug_read().
#pragma once
#include <cuda_runtime.h>

namespace b2 {

#ifdef B200MOE_DEBUG
static __device__ int g_debug_record[4];

__device__ __forceinline__ bool dbg_in_range(long long value, long long lo, long long hi, int code) {
  if (value >= lo && value < hi) return true;
  if (atomicCAS(&g_debug_record[0], 0, code) == 0) {
    g_debug_record[1] = static_cast<int>(value);
    g_debug_record[2] = static_cast<int>(hi);
    g_debug_record[3] = static_cast<int>(blockIdx.x);
  }
  return false;
}

// Defines ``int NAME(int out[4], int clear)``: copies the record of this file to the host, optionally clearing it.
#define B2_DEFINE_DEBUG_READER(NAME)                                                              \
  extern "C" int NAME(int* out, int clear) {                                                      \
    if (cudaMemcpyFromSymbol(out, b2::g_debug_record, sizeof(int) * 4) != cudaSuccess) return -1; \
    if (clear) {                                                                                  \
      const int zero[4] = {0, 0, 0, 0};                                                           \
      if (cudaMemcpyToSymbol(b2::g_debug_record, zero, sizeof(zero)) != cudaSuccess) return -1;   \
    }                                                                                             \
    return 0;                                                                                     \
  }
#else
__device__ __forceinline__ bool dbg_in_range(long long, long long, long long, int) { return true; }
#define B2_DEFINE_DEBUG_READER(NAME)
#endif

}  // namespace b2
