// Peer-memory primitives shared by the communication kernels: tables of peer pointers, release/acquire
// signal words with monotonically increasing sequence numbers, and bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

constexpr int MAX_RANKS = 8;
constexpr long long COMM_WAIT_CYCLES = 4000000000LL;   // ~2 s

struct Peers {
  void* ptr[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Signal pad layout: int32 [slot][MAX_RANKS]; element [slot][src] of rank r is written by rank src.
__device__ __forceinline__ void signal_all(const Peers& sig, int slot, int me, int n, int seq) {
  for (int p = 0; p < n; ++p) st_release_sys(static_cast<int*>(sig.ptr[p]) + slot * MAX_RANKS + me, seq);
}
__device__ __forceinline__ bool wait_one(const int* my_sig, int slot, int src, int seq) {
  const int* flag = my_sig + slot * MAX_RANKS + src;
  if (ld_acquire_sys(flag) - seq >= 0) return true;
  const long long start = clock64();
  while (ld_acquire_sys(flag) - seq < 0) {
    if (clock64() - start > COMM_WAIT_CYCLES) return false;
    __nanosleep(64);
  }
  return true;
}

}  // namespace b2
