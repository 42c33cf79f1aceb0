// Peer-memory primitives shared by the communication kernels: tables of peer pointers, release/acquire
// signal words with monotonically increasing sequence numbers, and bounded waits.
//
// Wait budget: every cross-GPU wait gives up after ``g_wait_ns`` nanoseconds of the device-wide clock
// (%globaltimer, independent of the SM clock) and reports failure to its caller, which sets the status word and
// skips the work that depended on the peer.  The budget is a per-file device variable with a compile-time
// default; the host sets it at run time through the ``b2_*_set_wait_ns`` function that each file defines with
// B2_DEFINE_WAIT_SETTER (``b2_comm_set_wait_ns`` in comm.cu calls all of them).  A wait also gives up at once
// when the status word is already non-zero, so after a first failure the rest of a step drains quickly.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

constexpr int MAX_RANKS = 8;
constexpr long long COMM_WAIT_NS_DEFAULT = 10000000000LL;   // 10 s

static __device__ long long g_wait_ns = COMM_WAIT_NS_DEFAULT;

#define B2_DEFINE_WAIT_SETTER(NAME)                                                             \
  extern "C" int NAME(long long ns) {                                                            \
    if (ns < 1000) return -1;                                                                    \
    return cudaMemcpyToSymbol(b2::g_wait_ns, &ns, sizeof(ns)) == cudaSuccess ? 0 : -2;           \
  }

struct Peers {
  void* ptr[MAX_RANKS];
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Deadline helper: ``expired()`` is true once the budget that started at construction has run out.
struct Deadline {
  unsigned long long start;
  long long budget;
  __device__ __forceinline__ Deadline() : start(global_ns()), budget(g_wait_ns) {}
  __device__ __forceinline__ bool expired() const { return static_cast<long long>(global_ns() - start) > budget; }
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Signal pad layout: int32 [slot][MAX_RANKS]; element [slot][src] of rank r is written by rank src.
__device__ __forceinline__ void signal_all(const Peers& sig, int slot, int me, int n, int seq) {
  for (int p = 0; p < n; ++p) st_release_sys(static_cast<int*>(sig.ptr[p]) + slot * MAX_RANKS + me, seq);
}
// Wait until flag [slot][src] of my pad reaches ``seq``.  ``status`` (may be null): the status word; a wait that
// finds it non-zero gives up at once.
__device__ __forceinline__ bool wait_one(const int* my_sig, int slot, int src, int seq, const int* status = nullptr) {
  const int* flag = my_sig + slot * MAX_RANKS + src;
  if (ld_acquire_sys(flag) - seq >= 0) return true;
  const Deadline deadline;
  while (ld_acquire_sys(flag) - seq < 0) {
    if (deadline.expired()) return false;
    if (status && ld_relaxed_sys(status) != 0) return false;
    __nanosleep(64);
  }
  return true;
}

}  // namespace b2
