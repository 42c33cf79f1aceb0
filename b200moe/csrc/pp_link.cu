// Stage-to-stage transfers of the pipeline over peer memory (NVLink), three small kernels on the compute stream.
//
// Every stage owns, in symmetric memory, a ring of landing slots for the activations of its upstream neighbour and
// a ring for the gradients of its downstream neighbour, plus three kinds of int32 words:
//   full[slot]  written by the sender after the payload: the number of the message the slot now holds;
//   ack         written by the receiver: how many of the sender's messages it has finished with.
// Messages of one direction are numbered 1, 2, 3, ... for the life of the link; message n uses slot (n-1) mod R.
//
//   pp_send_kernel   waits until message n-R has been acknowledged (no wait while n <= R), copies the payload into
//                    the peer's slot with 16-byte peer stores from the whole grid, and the last block to finish
//                    publishes ``full[slot] = n`` with a system-scope release store.  The sender never waits for the
//                    receiver to arrive at a matching call: it only waits when the ring is full.
//   pp_wait_kernel   one thread spins (bounded) until ``full[slot] >= n``; the kernels that follow on the stream
//                    read the slot in place, there is no second copy.
//   pp_ack_kernel    after the backward pass of a microbatch: tells both neighbours that its slots are free.
//
// Takes the place of the blocking ``batch_isend_irecv(...).wait()`` exchange of the reference scheduler
// (pipeline/pipelined_train_overlap.py:40-75), in which a stage's send completes only when its neighbour has
// reached the matching receive.
//
// Every wait is bounded by a budget passed with the launch (the pipeline's waits span whole stage steps, so they
// have their own, longer budget); a wait that runs out, or that finds the status word already set, records a code
// in the status word (321 ring full, 322 message never arrived), skips the copy and never publishes the flag.
#include "peer.cuh"

namespace b2 {

__device__ __forceinline__ bool pp_wait_flag(const int* flag, int seq, long long budget_ns, const int* status) {
  if (ld_acquire_sys(flag) - seq >= 0) return true;
  const unsigned long long start = global_ns();
  while (ld_acquire_sys(flag) - seq < 0) {
    if (static_cast<long long>(global_ns() - start) > budget_ns) return false;
    if (status && ld_relaxed_sys(status) != 0) return false;
    __nanosleep(128);
  }
  return true;
}

struct PpSend {
  const uint4* src;
  uint4* dst;             // the receiver's slot (peer memory)
  long long units;        // 16-byte units
  int* full_flag;         // the receiver's word for this slot (peer memory)
  const int* ack;         // local word: messages of this direction the receiver has finished with
  int seq, need_ack;
  long long wait_ns;
  unsigned int* ticket;   // local, zero between launches
  int* status;
};

constexpr int PP_THREADS = 512;

__global__ void __launch_bounds__(PP_THREADS) pp_send_kernel(const PpSend a) {
  __shared__ int ring_has_room;
  if (threadIdx.x == 0)
    ring_has_room = a.need_ack <= 0 || pp_wait_flag(a.ack, a.need_ack, a.wait_ns, a.status) ? 1 : 0;
  __syncthreads();
  if (ring_has_room) {
    const long long stride = static_cast<long long>(gridDim.x) * PP_THREADS;
    long long i = static_cast<long long>(blockIdx.x) * PP_THREADS + threadIdx.x;
    for (; i + 3 * stride < a.units; i += 4 * stride) {      // four loads in flight per thread
      const uint4 v0 = __ldcs(a.src + i), v1 = __ldcs(a.src + i + stride), v2 = __ldcs(a.src + i + 2 * stride),
                  v3 = __ldcs(a.src + i + 3 * stride);
      a.dst[i] = v0;
      a.dst[i + stride] = v1;
      a.dst[i + 2 * stride] = v2;
      a.dst[i + 3 * stride] = v3;
    }
    for (; i < a.units; i += stride) a.dst[i] = __ldcs(a.src + i);
  } else if (threadIdx.x == 0) {
    atomicCAS(a.status, 0, 321);
  }
  __threadfence_system();          // this thread's peer stores before the block's ticket
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(a.ticket, 1u);
    if (t == gridDim.x - 1) {
      __threadfence();             // the other blocks' tickets (and what they fenced) before the flag
      *a.ticket = 0;
      if (ld_relaxed_sys(a.status) == 0) st_release_sys(a.full_flag, a.seq);
    }
  }
}

__global__ void pp_wait_kernel(const int* flag, int seq, long long wait_ns, int* status) {
  if (threadIdx.x == 0 && !pp_wait_flag(flag, seq, wait_ns, status)) atomicCAS(status, 0, 322);
}

__global__ void pp_ack_kernel(int* upstream, int* downstream, int value) {
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (upstream) st_release_sys(upstream, value);
    if (downstream) st_release_sys(downstream, value);
  }
}

static int pp_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

}  // namespace b2

// Copy ``bytes`` (a multiple of 16, both addresses 16-byte aligned) into the receiver's slot and publish message
// ``seq``; waits first until the receiver has acknowledged message ``need_ack`` when that is positive.
extern "C" int b2_pp_send(const void* src, void* dst_peer, long long bytes, void* full_flag_peer, const void* ack_local,
                          int seq, int need_ack, long long wait_ns, void* ticket, void* status, cudaStream_t stream) {
  if (!src || !dst_peer || !full_flag_peer || !ack_local || !ticket || !status) return -1;
  if (bytes <= 0 || (bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(dst_peer) & 15))
    return -8;
  b2::PpSend a;
  a.src = static_cast<const uint4*>(src);
  a.dst = static_cast<uint4*>(dst_peer);
  a.units = bytes / 16;
  a.full_flag = static_cast<int*>(full_flag_peer);
  a.ack = static_cast<const int*>(ack_local);
  a.seq = seq;
  a.need_ack = need_ack;
  a.wait_ns = wait_ns;
  a.ticket = static_cast<unsigned int*>(ticket);
  a.status = static_cast<int*>(status);
  const long long want = (a.units + b2::PP_THREADS * 4 - 1) / (b2::PP_THREADS * 4);
  const int grid = static_cast<int>(want < 1 ? 1 : (want > 2LL * b2::pp_sms() ? 2LL * b2::pp_sms() : want));
  b2::pp_send_kernel<<<grid, b2::PP_THREADS, 0, stream>>>(a);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -2;
}

// Make the stream wait (bounded) until message ``seq`` has landed in the slot that ``full_flag_local`` guards.
extern "C" int b2_pp_wait(const void* full_flag_local, int seq, long long wait_ns, void* status, cudaStream_t stream) {
  if (!full_flag_local || !status) return -1;
  b2::pp_wait_kernel<<<1, 32, 0, stream>>>(static_cast<const int*>(full_flag_local), seq, wait_ns,
                                           static_cast<int*>(status));
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -2;
}

// Tell the upstream neighbour (activations) and the downstream neighbour (gradients) that this stage has finished
// with ``value`` of their messages; either pointer may be null.
extern "C" int b2_pp_ack(void* ack_upstream_peer, void* ack_downstream_peer, int value, cudaStream_t stream) {
  b2::pp_ack_kernel<<<1, 32, 0, stream>>>(static_cast<int*>(ack_upstream_peer), static_cast<int*>(ack_downstream_peer),
                                          value);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -2;
}
