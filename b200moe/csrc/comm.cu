// Peer-memory communication kernels (NVLink 5 / NVSwitch).  Every buffer named
// "peers" is a table of device pointers to the same symmetric allocation on each
// rank of a group; kernels load and store through those pointers directly.
//
//   * expert-parallel dispatch/return: a one-CTA plan kernel that exchanges the
//     per-expert counts through peer stores (no size all-to-all, no host sync),
//     a push kernel that writes token rows straight into the destination rank's
//     landing buffer, and consume kernels that wait for the senders' flags and
//     finish the local part (zero padding, scaling, routing-weight gradients);
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

// ------------------------------------------------------------------ EP plan with count exchange
constexpr int PLAN_THREADS = 1024;
constexpr int ALIGN_ROWS = 256;   // segment padding; tile tables are per 128-row unit
constexpr int TILE_ROWS = 128;
constexpr int MAX_EXPERTS = 32;

struct EpPlanArgs {
  const long long* idx;   // [slots] global expert of each slot
  int slots, experts_total, ep, rank, seq, capacity_rows;
  Peers counts_all;       // int32 [MAX_RANKS][MAX_EXPERTS] on each rank: [src][expert]
  Peers sig;
  int sig_slot;
  int* slot_row;          // [slots] landing row at the destination rank
  int* slot_dest;         // [slots] destination rank
  int* offs;              // [E_local] padded cumulative segment ends (this rank as expert owner)
  int* seg_live_end;      // [E_local] first padding row of each segment
  int* tile_expert;       // [capacity_rows / 128]
  int* meta;              // {live tiles, live rows, overflow, rows needed}
  int* status;
};

__global__ void __launch_bounds__(PLAN_THREADS) ep_plan_kernel(const EpPlanArgs a) {
  extern __shared__ uint8_t plan_smem[];
  uint32_t* local = reinterpret_cast<uint32_t*>(plan_smem);   // [E][PLAN_THREADS]
  __shared__ int warp_tot[32];
  __shared__ int my_count[MAX_EXPERTS];
  __shared__ int all_counts[MAX_RANKS][MAX_EXPERTS];
  __shared__ int base_row[MAX_EXPERTS];                        // landing row of my first slot of expert e
  const int E = a.experts_total, e_local = E / a.ep;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (a.slots + PLAN_THREADS - 1) / PLAN_THREADS;
  const int s0 = min(a.slots, tid * per), s1 = min(a.slots, s0 + per);
  for (int e = 0; e < E; ++e) local[e * PLAN_THREADS + tid] = 0;
  for (int s = s0; s < s1; ++s) local[min(max(static_cast<int>(a.idx[s]), 0), E - 1) * PLAN_THREADS + tid] += 1;
  __syncthreads();
  for (int e = 0; e < E; ++e) {
    const int mine = local[e * PLAN_THREADS + tid];
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += up;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      const int t = warp_tot[lane];
      int winc = t;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += up;
      }
      warp_tot[lane] = winc - t;
      if (lane == 31) my_count[e] = winc;
    }
    __syncthreads();
    local[e * PLAN_THREADS + tid] = static_cast<uint32_t>(inc - mine + warp_tot[warp]);
    __syncthreads();
  }
  // publish my counts in every rank's table, then the flag
  if (tid < E) {
    for (int p = 0; p < a.ep; ++p)
      static_cast<int*>(a.counts_all.ptr[p])[a.rank * MAX_EXPERTS + tid] = my_count[tid];
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) signal_all(a.sig, a.sig_slot, a.rank, a.ep, a.seq);
  const int* my_sig = static_cast<const int*>(a.sig.ptr[a.rank]);
  if (!block_wait_all(my_sig, a.sig_slot, a.ep, a.seq, a.status, 101)) {
    // a peer's counts never came: plan nothing (no tiles, no rows, every slot unsent) instead of using stale counts
    if (tid == 0) {
      a.meta[0] = 0; a.meta[1] = 0; a.meta[2] = 1; a.meta[3] = 0;
    }
    if (tid < e_local) {
      a.offs[tid] = 0;
      a.seg_live_end[tid] = 0;
    }
    for (int s = s0; s < s1; ++s) {
      a.slot_row[s] = -1;
      a.slot_dest[s] = -1;
    }
    return;
  }
  if (tid < a.ep * E) {
    const int src = tid / E, e = tid - src * E;
    all_counts[src][e] = ld_acquire_sys(static_cast<const int*>(a.counts_all.ptr[a.rank]) + src * MAX_EXPERTS + e);
  }
  __syncthreads();
  if (tid == 0) {
    for (int d = 0; d < a.ep; ++d) {
      int row = 0, tile = 0;
      for (int j = 0; j < e_local; ++j) {
        const int e = d * e_local + j;
        int total = 0, before_me = 0;
        for (int src = 0; src < a.ep; ++src) {
          if (src < a.rank) before_me += all_counts[src][e];
          total += all_counts[src][e];
        }
        base_row[e] = row + before_me;
        const int padded = (total + ALIGN_ROWS - 1) / ALIGN_ROWS * ALIGN_ROWS;
        if (d == a.rank) {
          a.seg_live_end[j] = row + total;
          if (row + padded <= a.capacity_rows)
            for (int t = 0; t < padded / TILE_ROWS; ++t) a.tile_expert[tile++] = j;
          a.offs[j] = row + padded;
        }
        row += padded;
      }
      if (d == a.rank) {
        const bool overflow = row > a.capacity_rows;
        a.meta[0] = overflow ? 0 : tile;
        a.meta[1] = overflow ? 0 : row;
        a.meta[2] = overflow ? 1 : 0;
        a.meta[3] = row;                       // rows this call needed (capacity hint for the host)
        if (overflow) atomicExch(a.status, 102);
      }
    }
  }
  __syncthreads();
  for (int s = s0; s < s1; ++s) {
    const int e = min(max(static_cast<int>(a.idx[s]), 0), E - 1);
    const int pos = local[e * PLAN_THREADS + tid];
    local[e * PLAN_THREADS + tid] = static_cast<uint32_t>(pos + 1);
    a.slot_row[s] = base_row[e] + pos;
    a.slot_dest[s] = e / e_local;
  }
}

// ------------------------------------------------------------------ push rows to their destination
struct EpPushArgs {
  const __nv_bfloat16* src;   // [rows_src, D]
  const int* row_of;          // [items] landing row at the destination
  const int* dest_of;         // [items] destination rank
  const int* tag_of;          // [items] int tag stored beside the row (source slot), or null
  const float* scalar_of;     // [items] float stored beside the row (routing weight), or null
  const int* live_items;      // device scalar: number of items (null = items)
  int items, D, src_shift;    // source row of item i = i >> src_shift (1: slots -> tokens, 0: rows)
  int dest_capacity, rank, n, seq, sig_slot;
  Peers land, land_tag, land_src, land_scalar, sig;
  unsigned int* counter;      // self-resetting block counter
};

__global__ void __launch_bounds__(256) ep_push_kernel(const EpPushArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int items = a.live_items ? min(a.items, *a.live_items) : a.items;
  for (int i = blockIdx.x * 8 + warp; i < items; i += gridDim.x * 8) {
    const int dest = a.dest_of[i];
    const int row = a.row_of[i];
    if (dest < 0 || row < 0 || row >= a.dest_capacity) continue;   // padding rows / overflow are not sent
    if (!dbg_in_range(dest, 0, a.n, 401)) continue;
    const __nv_bfloat16* src = a.src + static_cast<size_t>(i >> a.src_shift) * a.D;
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.land.ptr[dest]) + static_cast<size_t>(row) * a.D;
    // four 16-byte loads in flight per lane before the (possibly remote) stores
    int c = lane * 8;
    for (; c + 768 < a.D; c += 1024) {
      const vec16 v0 = *reinterpret_cast<const vec16*>(src + c);
      const vec16 v1 = *reinterpret_cast<const vec16*>(src + c + 256);
      const vec16 v2 = *reinterpret_cast<const vec16*>(src + c + 512);
      const vec16 v3 = *reinterpret_cast<const vec16*>(src + c + 768);
      *reinterpret_cast<vec16*>(dst + c) = v0;
      *reinterpret_cast<vec16*>(dst + c + 256) = v1;
      *reinterpret_cast<vec16*>(dst + c + 512) = v2;
      *reinterpret_cast<vec16*>(dst + c + 768) = v3;
    }
    for (; c < a.D; c += 256) *reinterpret_cast<vec16*>(dst + c) = *reinterpret_cast<const vec16*>(src + c);
    if (lane == 0) {
      if (a.tag_of) static_cast<int*>(a.land_tag.ptr[dest])[row] = a.tag_of[i];
      if (a.land_src.ptr[0]) static_cast<int*>(a.land_src.ptr[dest])[row] = a.rank;
      if (a.scalar_of) static_cast<float*>(a.land_scalar.ptr[dest])[row] = a.scalar_of[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int old = atomicInc(a.counter, gridDim.x - 1);
    if (old == gridDim.x - 1) {
      __threadfence_system();
      signal_all(a.sig, a.sig_slot, a.rank, a.n, a.seq);
    }
  }
}

// ------------------------------------------------------------------ expert side: take landed rows
struct EpConsumeArgs {
  const __nv_bfloat16* land;   // [capacity, D] local landing buffer
  const int* land_tag;
  const int* land_src;
  const float* land_scalar;    // null in forward
  const int* tile_expert;
  const int* seg_live_end;
  const int* meta;
  const __nv_bfloat16* y_perm; // backward: saved expert outputs for the routing-weight gradient
  Peers ret_scalar;            // backward: float [slots] at each source rank
  __nv_bfloat16* out;          // [capacity, D] owned buffer
  int* row_tag;                // forward: saved source slot per row (-1 padding)
  int* row_src;                // forward: saved source rank per row (-1 padding)
  const int* my_sig;
  int D, capacity, n, seq, sig_slot;
  int* status;
};

__global__ void __launch_bounds__(256) ep_consume_kernel(const EpConsumeArgs a) {
  if (!block_wait_all(a.my_sig, a.sig_slot, a.n, a.seq, a.status, 103)) return;   // rows of a peer are missing
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int live_rows = min(a.meta[1], a.capacity);
  for (int r = blockIdx.x * 8 + warp; r < live_rows; r += gridDim.x * 8) {
    const int expert = a.tile_expert[r / TILE_ROWS];
    if (!dbg_in_range(expert, 0, MAX_EXPERTS, 403)) continue;
    const bool live = r < a.seg_live_end[expert];
    __nv_bfloat16* dst = a.out + static_cast<size_t>(r) * a.D;
    if (!live) {
      for (int c = lane * 8; c < a.D; c += 256) *reinterpret_cast<vec16*>(dst + c) = vec16{{0, 0, 0, 0}};
      if (lane == 0 && a.row_tag) {
        a.row_tag[r] = -1;
        a.row_src[r] = -1;
      }
      continue;
    }
    const __nv_bfloat16* src = a.land + static_cast<size_t>(r) * a.D;
    if (!a.land_scalar) {
      for (int c = lane * 8; c < a.D; c += 256) *reinterpret_cast<vec16*>(dst + c) = *reinterpret_cast<const vec16*>(src + c);
      if (lane == 0) {
        a.row_tag[r] = a.land_tag[r];
        a.row_src[r] = a.land_src[r];
      }
      continue;
    }
    if (!dbg_in_range(a.land_src[r], 0, a.n, 402) || !dbg_in_range(a.land_tag[r], 0, 1 << 30, 404)) continue;
    const float w = a.land_scalar[r];
    float dot = 0.f;
    for (int c = lane * 8; c < a.D; c += 256) {
      const vec16 in = *reinterpret_cast<const vec16*>(src + c);
      const vec16 yv = *reinterpret_cast<const vec16*>(a.y_perm + static_cast<size_t>(r) * a.D + c);
      vec16 o;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in.v[i]));
        const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yv.v[i]));
        dot += f.x * g.x + f.y * g.y;
        const __nv_bfloat162 s = __floats2bfloat162_rn(f.x * w, f.y * w);
        o.v[i] = *reinterpret_cast<const uint32_t*>(&s);
      }
      *reinterpret_cast<vec16*>(dst + c) = o;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) static_cast<float*>(a.ret_scalar.ptr[a.land_src[r]])[a.land_tag[r]] = dot;
  }
}

// One block: wait for every peer's flag in ``sig_slot`` (placed before a kernel that reads landed data).
__global__ void ep_wait_kernel(const int* my_sig, int sig_slot, int n, int seq, int* status) {
  block_wait_all(my_sig, sig_slot, n, seq, status, 104);   // on failure the status word tells the host
}

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

// Gradients cross NVLink as 16-byte fp32 vectors (peer loads), new weights as 16-byte vectors of eight bf16
// (peer stores); entries whose offsets or sizes are not multiples of eight elements take the scalar loop.
__global__ void __launch_bounds__(512) fsdp_step_kernel(const FsdpArgs a) {
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
      for (long long i = tid * 8; i < ent.shard_numel; i += nthreads * 8) {
        const long long si = ent.shard_off + i;
        float g[8];
        if (a.do_reduce) {
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] = 0.f;
          for (int p = 0; p < a.n; ++p) {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(a.full_g.ptr[p]) + full_base + i);
            const float4 lo = src[0], hi = src[1];
            g[0] += lo.x; g[1] += lo.y; g[2] += lo.z; g[3] += lo.w;
            g[4] += hi.x; g[5] += hi.y; g[6] += hi.z; g[7] += hi.w;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] *= inv;
          float4* sg = reinterpret_cast<float4*>(a.shard_grad + si);
          sg[0] = make_float4(g[0], g[1], g[2], g[3]);
          sg[1] = make_float4(g[4], g[5], g[6], g[7]);
        } else {
          const float4* sg = reinterpret_cast<const float4*>(a.shard_grad + si);
          const float4 lo = sg[0], hi = sg[1];
          g[0] = lo.x; g[1] = lo.y; g[2] = lo.z; g[3] = lo.w; g[4] = hi.x; g[5] = hi.y; g[6] = hi.z; g[7] = hi.w;
        }
        if (a.do_update) {
          float4* pm = reinterpret_cast<float4*>(a.master + si);
          float4* mm = reinterpret_cast<float4*>(a.m + si);
          float4* vm = reinterpret_cast<float4*>(a.v + si);
          float pv[8], mv[8], vv[8];
          *reinterpret_cast<float4*>(pv) = pm[0]; *reinterpret_cast<float4*>(pv + 4) = pm[1];
          *reinterpret_cast<float4*>(mv) = mm[0]; *reinterpret_cast<float4*>(mv + 4) = mm[1];
          *reinterpret_cast<float4*>(vv) = vm[0]; *reinterpret_cast<float4*>(vv + 4) = vm[1];
#pragma unroll
          for (int j = 0; j < 8; ++j) pv[j] = adamw_one(a, pv[j], g[j], mv[j], vv[j]);
          pm[0] = *reinterpret_cast<float4*>(pv); pm[1] = *reinterpret_cast<float4*>(pv + 4);
          mm[0] = *reinterpret_cast<float4*>(mv); mm[1] = *reinterpret_cast<float4*>(mv + 4);
          vm[0] = *reinterpret_cast<float4*>(vv); vm[1] = *reinterpret_cast<float4*>(vv + 4);
          vec16 w;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(pv[2 * j], pv[2 * j + 1]);
            w.v[j] = *reinterpret_cast<const uint32_t*>(&b);
          }
          if (everyone) {
            for (int p = 0; p < a.n; ++p)
              *reinterpret_cast<vec16*>(static_cast<__nv_bfloat16*>(a.full_w.ptr[p]) + full_base + i) = w;
          } else {
            *reinterpret_cast<vec16*>(static_cast<__nv_bfloat16*>(a.full_w.ptr[a.rank]) + full_base + i) = w;
          }
        }
      }
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
int b2_comm_max_experts() { return MAX_EXPERTS; }

// Pointer tables are passed as arrays of MAX_RANKS device addresses (unused entries 0).
static Peers table(const unsigned long long* p) {
  Peers t{};
  for (int i = 0; i < MAX_RANKS; ++i) t.ptr[i] = p ? reinterpret_cast<void*>(p[i]) : nullptr;
  return t;
}

int b2_ep_plan(const long long* idx, int slots, int experts_total, int ep, int rank, int seq, int capacity_rows,
               const unsigned long long* counts_all, const unsigned long long* sig, int sig_slot, int* slot_row,
               int* slot_dest, int* offs, int* seg_live_end, int* tile_expert, int* meta, int* status,
               cudaStream_t s) {
  if (experts_total > MAX_EXPERTS || ep > MAX_RANKS || experts_total % ep || ep * experts_total > PLAN_THREADS)
    return -10;
  EpPlanArgs a{};
  a.idx = idx; a.slots = slots; a.experts_total = experts_total; a.ep = ep; a.rank = rank; a.seq = seq;
  a.capacity_rows = capacity_rows; a.counts_all = table(counts_all); a.sig = table(sig); a.sig_slot = sig_slot;
  a.slot_row = slot_row; a.slot_dest = slot_dest; a.offs = offs; a.seg_live_end = seg_live_end;
  a.tile_expert = tile_expert; a.meta = meta; a.status = status;
  const size_t smem = static_cast<size_t>(experts_total) * PLAN_THREADS * 4;
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(ep_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    set = true;
  }
  ep_plan_kernel<<<1, PLAN_THREADS, smem, s>>>(a);
  return launched();
}

int b2_ep_push(const void* src, const int* row_of, const int* dest_of, const int* tag_of, const float* scalar_of,
               const int* live_items, int items, int D, int src_shift, int dest_capacity, int rank, int n, int seq,
               int sig_slot, const unsigned long long* land, const unsigned long long* land_tag,
               const unsigned long long* land_src, const unsigned long long* land_scalar,
               const unsigned long long* sig, unsigned int* counter, cudaStream_t s) {
  if (D % 8) return -10;
  EpPushArgs a{};
  a.src = static_cast<const __nv_bfloat16*>(src); a.row_of = row_of; a.dest_of = dest_of; a.tag_of = tag_of;
  a.scalar_of = scalar_of; a.live_items = live_items; a.items = items; a.D = D; a.src_shift = src_shift;
  a.dest_capacity = dest_capacity; a.rank = rank; a.n = n; a.seq = seq; a.sig_slot = sig_slot;
  a.land = table(land); a.land_tag = table(land_tag); a.land_src = table(land_src);
  a.land_scalar = table(land_scalar); a.sig = table(sig); a.counter = counter;
  ep_push_kernel<<<device_sms() * 8, 256, 0, s>>>(a);
  return launched();
}

int b2_ep_consume(const void* land, const int* land_tag, const int* land_src, const float* land_scalar,
                  const int* tile_expert, const int* seg_live_end, const int* meta, const void* y_perm,
                  const unsigned long long* ret_scalar, void* out, int* row_tag, int* row_src, const int* my_sig,
                  int D, int capacity, int n, int seq, int sig_slot, int* status, cudaStream_t s) {
  if (D % 8) return -10;
  EpConsumeArgs a{};
  a.land = static_cast<const __nv_bfloat16*>(land); a.land_tag = land_tag; a.land_src = land_src;
  a.land_scalar = land_scalar; a.tile_expert = tile_expert; a.seg_live_end = seg_live_end; a.meta = meta;
  a.y_perm = static_cast<const __nv_bfloat16*>(y_perm); a.ret_scalar = table(ret_scalar);
  a.out = static_cast<__nv_bfloat16*>(out); a.row_tag = row_tag; a.row_src = row_src; a.my_sig = my_sig; a.D = D;
  a.capacity = capacity; a.n = n; a.seq = seq; a.sig_slot = sig_slot; a.status = status;
  ep_consume_kernel<<<device_sms() * 4, 256, 0, s>>>(a);
  return launched();
}

int b2_ep_wait(const int* my_sig, int sig_slot, int n, int seq, int* status, cudaStream_t s) {
  ep_wait_kernel<<<1, 32, 0, s>>>(my_sig, sig_slot, n, seq, status);
  return launched();
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
  else fsdp_step_kernel<<<device_sms() * 2, 512, 0, s>>>(a);
  return launched();
}

}  // extern "C"

B2_DEFINE_DEBUG_READER(b2_comm_debug_read)
B2_DEFINE_WAIT_SETTER(b2_comm_file_set_wait_ns)
