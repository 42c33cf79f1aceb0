// Peer-memory communication kernels (NVLink 5 / NVSwitch).  Every buffer named
// "peers" is a table of device pointers to the same symmetric allocation on each
// rank of a group; kernels load and store through those pointers directly.
//
//   * FSDP end of step: reduce-scatter of the fp32 gradients by peer loads,
//     fused with the AdamW update of the owned shard and the all-gather of the
//     new bf16 weights by peer stores — one kernel;
//   * replica all-reduce: one-shot, two-shot and NVLS (multimem) variants.
//
// Synchronisation is by monotonically increasing sequence numbers written with
// st.release.sys into the receiver's signal pad and read with ld.acquire.sys.
// Every wait is bounded (a cycle budget); on expiry the kernel sets the status
// word and carries on to its end, so a missing peer can never hang the GPU.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "debug.cuh"
#include "peer.cuh"

namespace b2 {

// Block-wide: threads 0..n-1 each wait for one source, then everyone proceeds.  Returns (to every thread of the
// block) whether all sources arrived; on failure ``code`` is in the status word and the caller skips whatever
// depended on the peers.
__device__ __forceinline__ bool block_wait_all(const int* my_sig, int slot, int n, int seq, int* status, int code) {
  int ok = 1;
  if (threadIdx.x < n) {
    if (!wait_one(my_sig, slot, threadIdx.x, seq, status)) {
      atomicCAS(status, 0, code);
      ok = 0;
    }
  }
  return __syncthreads_and(ok) != 0;
}

struct alignas(16) vec16 {
  uint32_t v[4];
};

// ------------------------------------------------------------------ replica all-reduce
struct ArArgs {
  Peers buf;        // symmetric fp32 buffer on each rank
  Peers sig;
  float* mc;        // multicast address of the buffer (NVLS) or null
  int rank, n, seq, sig_slot;
  long long count;  // floats, multiple of 4
  float scale;      // 1/n for averaging
  unsigned int* counter;
  int* status;
};

// Grid barrier across GPUs: block 0 announces arrival; every block waits for all ranks.  Returns false (to the
// whole block) when a rank did not arrive in time: the caller must then touch neither its own state nor a peer's.
__device__ __forceinline__ bool gpu_barrier_enter(const ArArgs& a, int slot) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    signal_all(a.sig, slot, a.rank, a.n, a.seq);
  }
  return block_wait_all(static_cast<const int*>(a.sig.ptr[a.rank]), slot, a.n, a.seq, a.status, 105);
}
// Leave: the last block to finish tells the peers and waits until every peer has finished too.  With ``entered``
// false (the enter barrier failed) only the block counter is restored: the peers are not told that this rank is
// done, because it has not done its part, and they run into their own budget.
__device__ __forceinline__ void gpu_barrier_leave(const ArArgs& a, int slot, bool entered = true) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int old = atomicInc(a.counter, gridDim.x - 1);
    if (old == gridDim.x - 1 && entered) {
      signal_all(a.sig, slot, a.rank, a.n, a.seq);
      const int* my_sig = static_cast<const int*>(a.sig.ptr[a.rank]);
      for (int src = 0; src < a.n; ++src)
        if (!wait_one(my_sig, slot, src, a.seq, a.status)) atomicCAS(a.status, 0, 106);
    }
  }
}

// One-shot: every rank reads all copies and writes the sum to a private output.
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const ArArgs a, float* out) {
  if (!gpu_barrier_enter(a, a.sig_slot)) {
    gpu_barrier_leave(a, a.sig_slot + 1, false);
    return;
  }
  const long long vecs = a.count / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < a.n; ++p) {
      const float4 v = reinterpret_cast<const float4*>(a.buf.ptr[p])[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= a.scale; acc.y *= a.scale; acc.z *= a.scale; acc.w *= a.scale;
    reinterpret_cast<float4*>(out)[i] = acc;
  }
  gpu_barrier_leave(a, a.sig_slot + 1);
}

// Two-shot, in place: rank r reduces chunk r from all copies and stores the result into every copy.
__global__ void __launch_bounds__(512) allreduce_twoshot_kernel(const ArArgs a) {
  if (!gpu_barrier_enter(a, a.sig_slot)) {
    gpu_barrier_leave(a, a.sig_slot + 1, false);
    return;
  }
  const long long vecs = a.count / 4;
  const long long chunk = (vecs + a.n - 1) / a.n;
  const long long lo = chunk * a.rank, hi = min(vecs, lo + chunk);
  for (long long i = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < hi;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < a.n; ++p) {
      const float4 v = reinterpret_cast<const float4*>(a.buf.ptr[p])[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= a.scale; acc.y *= a.scale; acc.z *= a.scale; acc.w *= a.scale;
    for (int p = 0; p < a.n; ++p) reinterpret_cast<float4*>(a.buf.ptr[p])[i] = acc;
  }
  gpu_barrier_leave(a, a.sig_slot + 1);
}

// NVLS, in place: the switch sums the copies (multimem.ld_reduce) and broadcasts the result (multimem.st).
__global__ void __launch_bounds__(512) allreduce_nvls_kernel(const ArArgs a) {
  if (!gpu_barrier_enter(a, a.sig_slot)) {
    gpu_barrier_leave(a, a.sig_slot + 1, false);
    return;
  }
  const long long vecs = a.count / 4;
  const long long chunk = (vecs + a.n - 1) / a.n;
  const long long lo = chunk * a.rank, hi = min(vecs, lo + chunk);
  for (long long i = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < hi;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 v;
    float* addr = a.mc + i * 4;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(addr)
                 : "memory");
    v.x *= a.scale; v.y *= a.scale; v.z *= a.scale; v.w *= a.scale;
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y),
                 "f"(v.z), "f"(v.w)
                 : "memory");
  }
  gpu_barrier_leave(a, a.sig_slot + 1);
}

// ------------------------------------------------------------------ FSDP: reduce-scatter + AdamW + all-gather
struct FsdpEntry {
  long long full_off;    // offset of the full tensor in the flat full buffers (elements)
  long long shard_off;   // offset of the shard in the flat shard buffers
  long long shard_numel;
  long long local_only;  // 1: the new bf16 rows are written to my own copy only (a later kernel gathers them)
};

struct FsdpArgs {
  Peers full_g;          // fp32 full gradients on each rank
  Peers full_w;          // bf16 full compute weights on each rank
  Peers sig;
  const FsdpEntry* entries;
  int num_entries, rank, n, seq, sig_slot;
  float* master;         // fp32 shards
  float* m;
  float* v;
  float* shard_grad;     // fp32 reduced shard gradient (kept for inspection / replica all-reduce)
  float lr, beta1, beta2, eps, wd, a_t;
  int do_update;         // 0: only reduce-scatter into shard_grad; 1: also AdamW + weight push
  int do_reduce;         // 0: shard_grad already holds the gradient (after a replica all-reduce)
  int push_all;          // 1: ignore FsdpEntry::local_only (initial materialisation)
  unsigned int* counter;
  int* status;
};

// One AdamW step on a value and its moments (the reference's rule, implementation/optimizer.py:29-39).
__device__ __forceinline__ float adamw_one(const FsdpArgs& a, float p, float g, float& m, float& v) {
  p *= 1.f - a.lr * a.wd;
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  return p - a.a_t * m / (sqrtf(v) + a.eps);
}

// One entry of the flat buffers, 16 bytes at a time.  Unit of work: one float4.  Consecutive lanes take
// consecutive units, so every warp-wide load is 512 contiguous bytes (whole sectors over NVLink) and every bf16 store
// 256.  A thread handles UNITS units per iteration, a grid apart, and issues all their loads (NR ranks' gradients,
// master, both moments) before the first use: remote loads take several times as long as local ones, and the bytes
// in flight per SM are what bounds the kernel.  NR: ranks the registers are laid out for (>= a.n).
template <int NR, int UNITS>
__device__ __forceinline__ void fsdp_vector_entry(const FsdpArgs& a, const FsdpEntry& ent, long long full_base,
                                                  bool everyone, float inv, long long tid, long long nthreads) {
  const long long units = ent.shard_numel / 4;
  for (long long u0 = tid; u0 < units; u0 += UNITS * nthreads) {
    float4 gr[UNITS][NR], pv[UNITS], mv[UNITS], vv[UNITS];
#pragma unroll
    for (int k = 0; k < UNITS; ++k) {
      const long long u = u0 + k * nthreads;
      if (u < units) {
        const long long i = u * 4;
        if (a.do_reduce) {
#pragma unroll
          for (int p = 0; p < NR; ++p)
            if (p < a.n)
              gr[k][p] = __ldcg(reinterpret_cast<const float4*>(static_cast<const float*>(a.full_g.ptr[p]) + full_base + i));
        } else {
          gr[k][0] = *reinterpret_cast<const float4*>(a.shard_grad + ent.shard_off + i);
        }
        if (a.do_update) {
          pv[k] = *reinterpret_cast<const float4*>(a.master + ent.shard_off + i);
          mv[k] = *reinterpret_cast<const float4*>(a.m + ent.shard_off + i);
          vv[k] = *reinterpret_cast<const float4*>(a.v + ent.shard_off + i);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < UNITS; ++k) {
      const long long u = u0 + k * nthreads;
      if (u >= units) continue;
      const long long i = u * 4;
      const long long si = ent.shard_off + i;
      float4 g = gr[k][0];
      if (a.do_reduce) {
#pragma unroll
        for (int p = 1; p < NR; ++p)
          if (p < a.n) {
            g.x += gr[k][p].x; g.y += gr[k][p].y; g.z += gr[k][p].z; g.w += gr[k][p].w;
          }
        g.x *= inv; g.y *= inv; g.z *= inv; g.w *= inv;
        *reinterpret_cast<float4*>(a.shard_grad + si) = g;
      }
      if (a.do_update) {
        float4 pn;
        pn.x = adamw_one(a, pv[k].x, g.x, mv[k].x, vv[k].x);
        pn.y = adamw_one(a, pv[k].y, g.y, mv[k].y, vv[k].y);
        pn.z = adamw_one(a, pv[k].z, g.z, mv[k].z, vv[k].z);
        pn.w = adamw_one(a, pv[k].w, g.w, mv[k].w, vv[k].w);
        *reinterpret_cast<float4*>(a.master + si) = pn;
        *reinterpret_cast<float4*>(a.m + si) = mv[k];
        *reinterpret_cast<float4*>(a.v + si) = vv[k];
        const __nv_bfloat162 lo = __floats2bfloat162_rn(pn.x, pn.y), hi = __floats2bfloat162_rn(pn.z, pn.w);
        const uint2 w = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        if (everyone) {
          for (int p = 0; p < a.n; ++p)
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.full_w.ptr[p]) + full_base + i) = w;
        } else {
          *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.full_w.ptr[a.rank]) + full_base + i) = w;
        }
      }
    }
  }
}

// Gradients cross NVLink as 16-byte fp32 vectors (peer loads), new weights as 8-byte vectors of four bf16 (peer
// stores), both lane-contiguous; entries whose offsets or sizes are not multiples of eight elements take the scalar
// loop.
// NR: ranks the registers are laid out for (2, 4 or MAX_RANKS, >= a.n).  With two ranks the state of two units fits
// 64 registers, so two CTAs share an SM and twice as many loads are in flight.
template <int NR>
__global__ void __launch_bounds__(512, NR <= 2 ? 2 : 1) fsdp_step_kernel(const FsdpArgs a) {
  ArArgs bar{};
  bar.sig = a.sig; bar.rank = a.rank; bar.n = a.n; bar.seq = a.seq; bar.counter = a.counter; bar.status = a.status;
  // every rank has finished accumulating its gradients; if one never says so, this rank neither reduces nor
  // updates (master weights and moments stay as they were) and does not report completion to the others
  if (!gpu_barrier_enter(bar, a.sig_slot)) {
    gpu_barrier_leave(bar, a.sig_slot + 1, false);
    return;
  }
  const float inv = 1.f / a.n;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int e = 0; e < a.num_entries; ++e) {
    const FsdpEntry ent = a.entries[e];
    const long long full_base = ent.full_off + ent.shard_numel * a.rank;
    const bool everyone = !(ent.local_only && !a.push_all);
    if (((full_base | ent.shard_off | ent.shard_numel) & 7) == 0) {
      fsdp_vector_entry<NR, 2>(a, ent, full_base, everyone, inv, tid, nthreads);
      continue;
    }
    for (long long i = tid; i < ent.shard_numel; i += nthreads) {
      const long long si = ent.shard_off + i;
      float g;
      if (a.do_reduce) {
        g = 0.f;
        for (int p = 0; p < a.n; ++p) g += static_cast<const float*>(a.full_g.ptr[p])[full_base + i];
        g *= inv;
        a.shard_grad[si] = g;
      } else {
        g = a.shard_grad[si];
      }
      if (a.do_update) {
        float mv = a.m[si], vv = a.v[si];
        const float pv = adamw_one(a, a.master[si], g, mv, vv);
        a.master[si] = pv;
        a.m[si] = mv;
        a.v[si] = vv;
        const __nv_bfloat16 wb = __float2bfloat16_rn(pv);
        if (everyone) {
          for (int p = 0; p < a.n; ++p) static_cast<__nv_bfloat16*>(a.full_w.ptr[p])[full_base + i] = wb;
        } else {
          static_cast<__nv_bfloat16*>(a.full_w.ptr[a.rank])[full_base + i] = wb;
        }
      }
    }
  }
  gpu_barrier_leave(bar, a.sig_slot + 1);  // every rank has read my gradients and written my weights
}

// All-gather only (initial materialisation / after a checkpoint load): push my bf16 shard to every rank.
__global__ void __launch_bounds__(512) fsdp_allgather_kernel(const FsdpArgs a) {
  ArArgs bar{};
  bar.sig = a.sig; bar.rank = a.rank; bar.n = a.n; bar.seq = a.seq; bar.counter = a.counter; bar.status = a.status;
  if (!gpu_barrier_enter(bar, a.sig_slot)) {
    gpu_barrier_leave(bar, a.sig_slot + 1, false);
    return;
  }
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int e = 0; e < a.num_entries; ++e) {
    const FsdpEntry ent = a.entries[e];
    const long long full_base = ent.full_off + ent.shard_numel * a.rank;
    const bool everyone = !(ent.local_only && !a.push_all);
    if (((full_base | ent.shard_off | ent.shard_numel) & 7) == 0) {
      for (long long i = tid * 8; i < ent.shard_numel; i += nthreads * 8) {
        const float4* pm = reinterpret_cast<const float4*>(a.master + ent.shard_off + i);
        const float4 lo = pm[0], hi = pm[1];
        const __nv_bfloat162 b0 = __floats2bfloat162_rn(lo.x, lo.y), b1 = __floats2bfloat162_rn(lo.z, lo.w);
        const __nv_bfloat162 b2v = __floats2bfloat162_rn(hi.x, hi.y), b3 = __floats2bfloat162_rn(hi.z, hi.w);
        vec16 w;
        w.v[0] = *reinterpret_cast<const uint32_t*>(&b0); w.v[1] = *reinterpret_cast<const uint32_t*>(&b1);
        w.v[2] = *reinterpret_cast<const uint32_t*>(&b2v); w.v[3] = *reinterpret_cast<const uint32_t*>(&b3);
        if (everyone) {
          for (int p = 0; p < a.n; ++p)
            *reinterpret_cast<vec16*>(static_cast<__nv_bfloat16*>(a.full_w.ptr[p]) + full_base + i) = w;
        } else {
          *reinterpret_cast<vec16*>(static_cast<__nv_bfloat16*>(a.full_w.ptr[a.rank]) + full_base + i) = w;
        }
      }
      continue;
    }
    for (long long i = tid; i < ent.shard_numel; i += nthreads) {
      const __nv_bfloat16 wb = __float2bfloat16_rn(a.master[ent.shard_off + i]);
      if (everyone) {
        for (int p = 0; p < a.n; ++p) static_cast<__nv_bfloat16*>(a.full_w.ptr[p])[full_base + i] = wb;
      } else {
        static_cast<__nv_bfloat16*>(a.full_w.ptr[a.rank])[full_base + i] = wb;
      }
    }
  }
  gpu_barrier_leave(bar, a.sig_slot + 1);
}

static int device_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

static inline int launched() { return cudaGetLastError() == cudaSuccess ? 0 : -1; }

}  // namespace b2

using namespace b2;

extern "C" {

int b2_ag_gemm_file_set_wait_ns(long long ns);
int b2_comm_file_set_wait_ns(long long ns);
int b2_moe_ep_file_set_wait_ns(long long ns);

// Budget, in nanoseconds of the device-wide clock, of every cross-GPU wait in this library's kernels on the
// current device (default 10 s).  Returns non-zero if a file's copy of the setting could not be written.
int b2_comm_set_wait_ns(long long ns) {
  int rc = b2_comm_file_set_wait_ns(ns);
  if (!rc) rc = b2_ag_gemm_file_set_wait_ns(ns);
  if (!rc) rc = b2_moe_ep_file_set_wait_ns(ns);
  return rc;
}

int b2_comm_max_ranks() { return MAX_RANKS; }

// Pointer tables are passed as arrays of MAX_RANKS device addresses (unused entries 0).
static Peers table(const unsigned long long* p) {
  Peers t{};
  for (int i = 0; i < MAX_RANKS; ++i) t.ptr[i] = p ? reinterpret_cast<void*>(p[i]) : nullptr;
  return t;
}

// kind: 0 one-shot (result in ``out``), 1 two-shot in place, 2 NVLS in place (needs ``mc``).
int b2_comm_allreduce(const unsigned long long* buf, const unsigned long long* sig, void* mc, float* out, int kind,
                      int rank, int n, int seq, int sig_slot, long long count, float scale, unsigned int* counter,
                      int* status, cudaStream_t s) {
  if (count % 4 || n > MAX_RANKS) return -10;
  ArArgs a{};
  a.buf = table(buf); a.sig = table(sig); a.mc = static_cast<float*>(mc); a.rank = rank; a.n = n; a.seq = seq;
  a.sig_slot = sig_slot; a.count = count; a.scale = scale; a.counter = counter; a.status = status;
  const long long vecs = count / 4;
  int blocks = static_cast<int>((vecs + 511) / 512);
  blocks = blocks < 1 ? 1 : (blocks > device_sms() * 2 ? device_sms() * 2 : blocks);
  if (kind == 0) allreduce_oneshot_kernel<<<blocks, 512, 0, s>>>(a, out);
  else if (kind == 1) allreduce_twoshot_kernel<<<blocks, 512, 0, s>>>(a);
  else if (kind == 2 && mc) allreduce_nvls_kernel<<<blocks, 512, 0, s>>>(a);
  else return -11;
  return launched();
}

// mode: 0 reduce-scatter only, 1 reduce-scatter + AdamW + weight all-gather, 2 AdamW + all-gather on shard_grad,
//       3 all-gather of the current master weights only.
int b2_fsdp_step(const unsigned long long* full_g, const unsigned long long* full_w, const unsigned long long* sig,
                 const void* entries, int num_entries, int rank, int n, int seq, int sig_slot, float* master, float* m,
                 float* v, float* shard_grad, float lr, float beta1, float beta2, float eps, float wd, float a_t,
                 int mode, int push_all, unsigned int* counter, int* status, cudaStream_t s) {
  FsdpArgs a{};
  a.full_g = table(full_g); a.full_w = table(full_w); a.sig = table(sig);
  a.entries = static_cast<const FsdpEntry*>(entries); a.num_entries = num_entries; a.rank = rank; a.n = n;
  a.seq = seq; a.sig_slot = sig_slot; a.master = master; a.m = m; a.v = v; a.shard_grad = shard_grad; a.lr = lr;
  a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd; a.a_t = a_t; a.counter = counter; a.status = status;
  a.do_reduce = mode == 0 || mode == 1;
  a.do_update = mode == 1 || mode == 2;
  a.push_all = push_all;
  if (mode == 3) fsdp_allgather_kernel<<<device_sms() * 2, 512, 0, s>>>(a);
  else if (n <= 2) fsdp_step_kernel<2><<<device_sms() * 2, 512, 0, s>>>(a);
  else if (n <= 4) fsdp_step_kernel<4><<<device_sms() * 2, 512, 0, s>>>(a);
  else fsdp_step_kernel<MAX_RANKS><<<device_sms() * 2, 512, 0, s>>>(a);
  return launched();
}

}  // extern "C"

B2_DEFINE_DEBUG_READER(b2_comm_debug_read)
B2_DEFINE_WAIT_SETTER(b2_comm_file_set_wait_ns)
