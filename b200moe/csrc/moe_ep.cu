// Expert-parallel MoE: the row exchange fused with the expert GEMMs.
//
// The expert owner PULLS.  After the plan kernel (ep_plan2_kernel: counts exchanged through peer stores, then the
// source slot, source rank and routing weight of every row written straight into the owner's row tables) the
// owner's grouped GEMM itself fetches the rows it multiplies:
//
//   ep_gather_gemm_kernel   one persistent cooperative kernel per rank.  Each CTA (one per SM) has
//       warp 0      TMA producer          warp 1      MMA issuer (tcgen05, accumulators double-buffered in TMEM)
//       warps 2..5  epilogue              warps 6..9  copiers
//     The copier warps of all CTAs together walk the expert-major rows in order; for each row they read the token's
//     activation row from the source rank's buffer with plain 16-byte loads (NVLink for a peer, HBM for this rank),
//     store it into this rank's expert-major operand buffer, and bump the counter of the row's 128-row tile.  The
//     TMA producer of a tile waits (bounded) for that counter and then loads the tile from LOCAL memory, so every
//     TMA load reads this GPU's own memory, a remote row crosses NVLink once, and the exchange runs under the
//     tensor-core work of the tiles already in place.  Two instances:
//       gate/up   y = x_perm W1^T, x_perm W3^T with the SwiGLU epilogue (forward, and the rebuild of the
//                 pre-activations in the backward pass);  x rows come from the peers' token buffers
//       dh        dh = dy_perm W2 (W2 read MN-major);  dy rows come from the peers' output-gradient buffers
//   The return path is the epilogue of the following GEMM (csrc/gemm.cu, EPI_PUSH): every finished output row is
//   scaled by its routing weight and stored into the SOURCE rank's slot-indexed return buffer, and the last CTA
//   raises a flag; ep_combine_kernel on the source rank waits for the flags and adds the two slots of a token.
//
// Replaces the reference's _dispatch_tokens / TensorExchange / grouped_mm / _combine_tokens sequence
// (implementation/layers.py:14-52, 139-246): no size all-to-all, no host read, no landing copy.
//
// Ordering between calls needs no extra handshakes: every call starts with an all-to-all dependency (the plan's
// counts, or the staged gradient rows) and ends with one (the return flags), and the ranks of a group issue the
// same sequence of calls, so when a rank overwrites a buffer its peers read, they have finished the call that
// read it.
#include <cuda_bf16.h>

#include "debug.cuh"
#include "peer.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace b2 {
namespace ep {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 320;
constexpr int COPY_WARPS = 4;
constexpr int GROUP_M = 8;
constexpr int TILE_ROWS = 128;
constexpr int ALIGN_ROWS = 256;
constexpr int MAX_EXPERTS = 32;

enum Epi : int { EPI_STORE = 0, EPI_SWIGLU = 1 };

struct Params {
  CUtensorMap map_a;        // the local expert-major operand buffer [cap, K]
  CUtensorMap map_b;        // weights: K-major [E*rows, K] (gate rows for SwiGLU) or MN-major [E*K, N]
  CUtensorMap map_b2;       // SwiGLU: up-projection rows
  int N, K;                 // output columns (2F for SwiGLU), reduction length
  int b_expert_rows;        // rows of one expert in the weight map
  const int* tile_expert;   // [cap/128] local expert of each 128-row tile
  const int* meta;          // {live 128-row tiles, live rows, overflow, rows needed}
  const int* seg_live_end;  // [E_local] first padding row of each expert segment
  int gemm_tile_begin;      // first 128-row tile the tensor cores compute (the copiers always fill every live tile)
  int cap_rows;             // rows of the operand buffer
  // ---- gather
  Peers src;                // every rank's source buffer [src_rows, K] bf16
  int src_shift;            // source row = tag >> src_shift (1: slot -> token)
  const int* row_src;       // [cap] source rank of each row      (forward: the landing tables the peers wrote)
  const int* row_tag;       // [cap] slot id at the source rank
  const float* row_w;       // [cap] routing weight of the slot
  int* save_src;            // optional copies for the backward pass (padding rows get -1)
  int* save_tag;
  float* save_w;
  __nv_bfloat16* a_buf;     // gather destination = base of map_a
  int* tile_ready;          // [cap/128] zero on entry; the last CTA zeroes it again on exit
  unsigned int* ticket;     // self-resetting CTA counter
  Peers sig;
  int n, rank, sig_slot, seq;
  int handshake;            // 0: sources are ready; 1: wait for every rank's flag; 2: raise mine first, then wait
  // ---- epilogue
  void* d;                  // EPI_STORE: [cap, N] bf16;  EPI_SWIGLU: h [cap, N/2] bf16 or null
  long long ldd;
  void* gate_lo;            // SwiGLU pre-activations of rows < split_row (null: not stored)
  void* up_lo;
  void* gate_hi;            // ... of rows >= split_row, indexed by absolute row (null: not stored)
  void* up_hi;
  int split_row;
  int* status;
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void copier_sync() { asm volatile("bar.sync 1, %0;" ::"n"(COPY_WARPS * 32) : "memory"); }

struct Tile {
  int m_tile, n_tile;
};
// Grouped raster over (m, n): eight row tiles share their column blocks; row tiles come in increasing order, which
// is also the order in which the copiers complete them.
__device__ __forceinline__ Tile decode(long long tile, int m_first, int m_tiles, int n_tiles) {
  const int group = static_cast<int>(tile / (GROUP_M * n_tiles));
  const int first_m = group * GROUP_M;
  const int rows_in_group = min(GROUP_M, m_tiles - first_m);
  const int in_group = static_cast<int>(tile - static_cast<long long>(group) * GROUP_M * n_tiles);
  Tile t;
  t.m_tile = m_first + first_m + in_group % rows_in_group;
  t.n_tile = in_group / rows_in_group;
  return t;
}

struct alignas(16) vec16 {
  uint32_t v[4];
};

template <int B_MN, int EPI>
__global__ void __launch_bounds__(THREADS, 1) ep_gather_gemm_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* copy_ok = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cap_tiles = p.cap_rows / TILE_ROWS;
  const int live_tiles = min(max(p.meta[0], 0), cap_tiles);
  const int m_tiles = max(live_tiles - p.gemm_tile_begin, 0);
  const int n_tiles = (p.N + BN - 1) / BN;
  const long long total_tiles = static_cast<long long>(m_tiles) * n_tiles;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    *copy_ok = 1;
    mbar_fence_init();
    tma_prefetch_desc(&p.map_a);
    tma_prefetch_desc(&p.map_b);
    if (EPI == EPI_SWIGLU) tma_prefetch_desc(&p.map_b2);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (long long tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        const Tile t = decode(tile, p.gemm_tile_begin, m_tiles, n_tiles);
        {
          // the rows of this tile are being (or have been) brought in by the copier warps of all CTAs
          const int* flag = p.tile_ready + t.m_tile;
          bool ok = ld_acquire_gpu(flag) >= TILE_ROWS;
          if (!ok) {
            const Deadline deadline;
            while (!(ok = ld_acquire_gpu(flag) >= TILE_ROWS)) {
              if (deadline.expired() || *abort_flag) break;
              __nanosleep(100);
            }
          }
          if (!ok) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, 311);
            break;
          }
          fence_proxy_async_all();   // the copiers' generic-proxy stores before my async-proxy (TMA) reads
        }
        const int expert = p.tile_expert[t.m_tile];
        const int m0 = t.m_tile * BM;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, 312);
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          uint64_t* full = &full_bar[stage];
          mbar_expect_tx(full, STAGE_BYTES);
          const int k0 = kb * BK;
          tma_load_2d(sa, &p.map_a, full, k0, m0);
          if (EPI == EPI_SWIGLU) {
            const int row = expert * p.b_expert_rows + t.n_tile * 128;      // gate rows, then up rows
            tma_load_2d(sb, &p.map_b, full, k0, row);
            tma_load_2d(sb + 16384, &p.map_b2, full, k0, row);
          } else if (B_MN) {
            const int krow = expert * p.b_expert_rows + k0;
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &p.map_b, full, t.n_tile * BN + c * 64, krow);
          } else {
            tma_load_2d(sb, &p.map_b, full, k0, expert * p.b_expert_rows + t.n_tile * BN);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, B_MN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (long long tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, 313);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool failed = false;
        for (int kb = 0; kb < k_blocks; ++kb) {
          // the producer may itself be waiting for rows from a peer (bounded by the cross-GPU budget)
          bool got = false;
          const Deadline deadline;
          while (!got && !*abort_flag) {
            got = mbar_wait(&full_bar[stage], phase);
            if (!got && deadline.expired()) break;
          }
          if (!got) {
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = umma_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(sb + k * 2048, 8192, 1024) : umma_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (failed) {
          if (!*abort_flag) atomicCAS(p.status, 0, 314);
          *abort_flag = 1;
          break;
        }
        umma_commit(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (long long tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
      const Tile t = decode(tile, p.gemm_tile_begin, m_tiles, n_tiles);
      bool got = false;
      const Deadline deadline;
      while (!got && !*abort_flag) {
        got = mbar_wait(&tmem_full[acc], acc_phase);
        if (!got && deadline.expired()) break;
      }
      if (!got) {
        if (!*abort_flag) atomicCAS(p.status, 0, 315);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      const long long row = static_cast<long long>(t.m_tile) * BM + row_in_tile;
      const bool row_ok = row < p.cap_rows;
      if (EPI == EPI_SWIGLU) {
        const long long half_n = p.N / 2;
        const long long col0 = static_cast<long long>(t.n_tile) * 128;
        __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(p.d);
        const bool low = row < p.split_row;
        __nv_bfloat16* gdst = reinterpret_cast<__nv_bfloat16*>(low ? p.gate_lo : p.gate_hi);
        __nv_bfloat16* udst = reinterpret_cast<__nv_bfloat16*>(low ? p.up_lo : p.up_hi);
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + c, g);
          tmem_ld_32x32(taddr + 128 + c, u);
          tmem_ld_wait();
          if (!row_ok || col0 + c >= half_n) continue;
          uint32_t out[16], og[16], ou[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
            const float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
            out[i] = pack_bf16(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
            og[i] = pack_bf16(g0, g1);
            ou[i] = pack_bf16(u0, u1);
          }
          const long long off = row * half_n + col0 + c;
          if (h) {
            uint4* dst = reinterpret_cast<uint4*>(h + off);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
          }
          if (gdst) {
            uint4* dg = reinterpret_cast<uint4*>(gdst + off);
            uint4* du = reinterpret_cast<uint4*>(udst + off);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              dg[i] = make_uint4(og[4 * i], og[4 * i + 1], og[4 * i + 2], og[4 * i + 3]);
              du[i] = make_uint4(ou[4 * i], ou[4 * i + 1], ou[4 * i + 2], ou[4 * i + 3]);
            }
          }
        }
      } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.d);
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + c, v);
          tmem_ld_wait();
          const long long col = static_cast<long long>(t.n_tile) * BN + c;
          if (!row_ok || col >= p.N) continue;      // N is a multiple of 32 (checked on the host)
          uint4* dst = reinterpret_cast<uint4*>(out + row * p.ldd + col);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[i] = make_uint4(pack_bf16(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])),
                                pack_bf16(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])),
                                pack_bf16(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])),
                                pack_bf16(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7])));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ copiers (warps 6..9)
    const int cw = warp - 6;
    if (cw == 0 && lane == 0) {
      if (p.handshake == 2 && blockIdx.x == 0) {
        // my source rows were written by earlier work on this stream: the peers may read them
        __threadfence_system();
        signal_all(p.sig, p.sig_slot, p.rank, p.n, p.seq);
      }
      if (p.handshake) {
        const int* my_sig = static_cast<const int*>(p.sig.ptr[p.rank]);
        for (int src = 0; src < p.n; ++src) {
          if (!wait_one(my_sig, p.sig_slot, src, p.seq, p.status)) {
            atomicCAS(p.status, 0, 316);
            *copy_ok = 0;
          }
        }
      }
    }
    copier_sync();
    if (*copy_ok) {
      const int live_rows = min(max(p.meta[1], 0), p.cap_rows);
      const int vecs = p.K / 8;                                  // 16-byte vectors per row
      const int stride = static_cast<int>(gridDim.x) * COPY_WARPS;
      for (int r = static_cast<int>(blockIdx.x) * COPY_WARPS + cw; r < live_rows; r += stride) {
        const int tile = r / TILE_ROWS;
        const int expert = p.tile_expert[tile];
        bool live = dbg_in_range(expert, 0, MAX_EXPERTS, 411) && r < p.seg_live_end[expert];
        int src = -1, tag = -1;
        float w = 0.f;
        if (live) {
          src = p.row_src[r];
          tag = p.row_tag[r];
          w = p.row_w ? p.row_w[r] : 0.f;
          if (src < 0 || src >= p.n || tag < 0) live = false;    // never follow a row table entry out of range
          dbg_in_range(src, 0, p.n, 412);
        }
        vec16* dst = reinterpret_cast<vec16*>(p.a_buf + static_cast<size_t>(r) * p.K);
        if (live) {
          const vec16* from = reinterpret_cast<const vec16*>(static_cast<const __nv_bfloat16*>(p.src.ptr[src]) +
                                                             static_cast<size_t>(tag >> p.src_shift) * p.K);
          int c = lane;
          for (; c + 7 * 32 < vecs; c += 8 * 32) {
            vec16 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = from[c + u * 32];
#pragma unroll
            for (int u = 0; u < 8; ++u) dst[c + u * 32] = v[u];
          }
          for (; c < vecs; c += 32) dst[c] = from[c];
        } else {
          for (int c = lane; c < vecs; c += 32) dst[c] = vec16{{0, 0, 0, 0}};
        }
        if (lane == 0 && p.save_tag) {
          p.save_src[r] = live ? src : -1;
          p.save_tag[r] = live ? tag : -1;
          p.save_w[r] = live ? w : 0.f;
        }
        __threadfence();
        fence_proxy_async_all();
        __syncwarp();
        if (lane == 0) red_release_gpu_add(p.tile_ready + tile, 1);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0) {
    // the last CTA out puts the tile counters back to zero for the next launch
    __threadfence();
    const unsigned int old = atomicInc(p.ticket, gridDim.x - 1);
    if (old == gridDim.x - 1)
      for (int t = 0; t < cap_tiles; ++t) p.tile_ready[t] = 0;
  }
}

// ------------------------------------------------------------------ plan: counts exchange + row tables at the owner
constexpr int PLAN_THREADS = 1024;

struct PlanArgs {
  const long long* idx;     // [slots] global expert of each slot
  const float* weights;     // [slots] routing weight of each slot
  int slots, experts_total, ep, rank, seq, capacity_rows;
  Peers counts_all;         // int32 [MAX_RANKS][MAX_EXPERTS] on each rank: [src][expert]
  Peers land_src, land_tag, land_w;   // row tables [capacity] on each rank, written by the sources
  Peers sig;
  int counts_slot, meta_slot;
  int* offs;                // [E_local] padded cumulative segment ends (this rank as expert owner)
  int* seg_live_end;        // [E_local] first padding row of each segment
  int* tile_expert;         // [capacity_rows / 128]
  int* meta;                // {live tiles, live rows, overflow, rows needed}
  int* status;
};

// One CTA.  Stable counting sort of my slots by expert; my per-expert counts go to every rank; with everybody's counts
// each rank knows the expert-major layout at every owner, so the row of each of my slots at its owner is known here
// and (source rank, slot, routing weight) are written into the owner's row tables directly.  Two flags: counts
// published, row tables written.
__global__ void __launch_bounds__(PLAN_THREADS) ep_plan2_kernel(const PlanArgs a) {
  extern __shared__ uint8_t plan_smem[];
  uint32_t* local = reinterpret_cast<uint32_t*>(plan_smem);   // [E][PLAN_THREADS]
  __shared__ int warp_tot[32];
  __shared__ int my_count[MAX_EXPERTS];
  __shared__ int all_counts[MAX_RANKS][MAX_EXPERTS];
  __shared__ int base_row[MAX_EXPERTS];                        // row at the owner of my first slot of expert e
  __shared__ int owner_rows[MAX_RANKS];                        // padded rows each owner needs
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
  if (tid < E) {
    for (int p = 0; p < a.ep; ++p)
      static_cast<int*>(a.counts_all.ptr[p])[a.rank * MAX_EXPERTS + tid] = my_count[tid];
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) signal_all(a.sig, a.counts_slot, a.rank, a.ep, a.seq);
  const int* my_sig = static_cast<const int*>(a.sig.ptr[a.rank]);
  int ok = 1;
  if (tid < a.ep && !wait_one(my_sig, a.counts_slot, tid, a.seq, a.status)) {
    atomicCAS(a.status, 0, 101);
    ok = 0;
  }
  if (!__syncthreads_and(ok)) {
    // a peer's counts never came: plan nothing instead of using stale counts, and do not raise the second flag
    if (tid == 0) {
      a.meta[0] = 0; a.meta[1] = 0; a.meta[2] = 1; a.meta[3] = 0;
    }
    if (tid < e_local) {
      a.offs[tid] = 0;
      a.seg_live_end[tid] = 0;
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
      owner_rows[d] = row;
      if (d == a.rank) {
        const bool overflow = row > a.capacity_rows;
        a.meta[0] = overflow ? 0 : tile;
        a.meta[1] = overflow ? 0 : row;
        a.meta[2] = overflow ? 1 : 0;
        a.meta[3] = row;                       // rows this call needed (read back asynchronously by the host)
        if (overflow) {
          for (int j = 0; j < e_local; ++j) {
            a.offs[j] = 0;
            a.seg_live_end[j] = 0;
          }
          atomicCAS(a.status, 0, 102);
        }
      }
    }
  }
  __syncthreads();
  for (int s = s0; s < s1; ++s) {
    const int e = min(max(static_cast<int>(a.idx[s]), 0), E - 1);
    const int pos = local[e * PLAN_THREADS + tid];
    local[e * PLAN_THREADS + tid] = static_cast<uint32_t>(pos + 1);
    const int dest = e / e_local;
    const int row = base_row[e] + pos;
    if (owner_rows[dest] > a.capacity_rows || row >= a.capacity_rows) continue;   // that owner overflowed: it plans nothing
    static_cast<int*>(a.land_src.ptr[dest])[row] = a.rank;
    static_cast<int*>(a.land_tag.ptr[dest])[row] = s;
    static_cast<float*>(a.land_w.ptr[dest])[row] = a.weights[s];
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) signal_all(a.sig, a.meta_slot, a.rank, a.ep, a.seq);
}

// ------------------------------------------------------------------ SwiGLU backward on expert-major rows
// One warp per row.  dh holds dy W2 for the UNSCALED output gradient; w is the row's routing weight.
//   dgu[r, 0:F]  = w dh u silu'(g)      dgu[r, F:2F] = w dh silu(g)      dh[r, :] <- w silu(g) u   (in place)
//   d(routing weight of the row's slot) = sum_f dh silu(g) u, stored at the slot's source rank.
// gate/up of rows < split_row are read from (gate_lo, up_lo), the others from (gate_hi, up_hi).
struct SwigluBwdArgs {
  __nv_bfloat16* dh;
  const __nv_bfloat16 *gate_lo, *up_lo, *gate_hi, *up_hi;
  int split_row;
  __nv_bfloat16* dgu;
  const int* meta;
  const int *row_tag, *row_src;
  const float* row_w;
  Peers dw_ret;             // float [slots] on each rank
  int cap_rows, F, n;
};

__device__ __forceinline__ void unpack8(const vec16& in, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in.v[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ vec16 pack8(const float (&f)[8]) {
  vec16 o;
#pragma unroll
  for (int i = 0; i < 4; ++i) o.v[i] = pack_bf16(f[2 * i], f[2 * i + 1]);
  return o;
}

__global__ void __launch_bounds__(256) ep_swiglu_bwd_kernel(const SwigluBwdArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int live_rows = min(max(a.meta[1], 0), a.cap_rows);
  const int vecs = a.F / 8;
  for (int r = blockIdx.x * 8 + warp; r < live_rows; r += gridDim.x * 8) {
    const bool low = r < a.split_row;
    const vec16* g = reinterpret_cast<const vec16*>((low ? a.gate_lo : a.gate_hi) + static_cast<size_t>(r) * a.F);
    const vec16* u = reinterpret_cast<const vec16*>((low ? a.up_lo : a.up_hi) + static_cast<size_t>(r) * a.F);
    vec16* d = reinterpret_cast<vec16*>(a.dh + static_cast<size_t>(r) * a.F);
    vec16* dg = reinterpret_cast<vec16*>(a.dgu + static_cast<size_t>(r) * 2 * a.F);
    vec16* du = dg + vecs;
    const float w = a.row_w[r];
    float dot = 0.f;
#pragma unroll 2
    for (int c = lane; c < vecs; c += 32) {
      float dv[8], gv[8], uv[8], og[8], ou[8], oh[8];
      unpack8(d[c], dv);
      unpack8(g[c], gv);
      unpack8(u[c], uv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sig = 1.f / (1.f + __expf(-gv[j]));
        const float sl = gv[j] * sig;
        const float hh = sl * uv[j];
        dot += dv[j] * hh;
        og[j] = w * dv[j] * uv[j] * sig * (1.f + gv[j] * (1.f - sig));
        ou[j] = w * dv[j] * sl;
        oh[j] = w * hh;
      }
      dg[c] = pack8(og);
      du[c] = pack8(ou);
      d[c] = pack8(oh);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) {
      const int tag = a.row_tag[r], src = a.row_src[r];
      if (tag >= 0 && src >= 0 && src < a.n) static_cast<float*>(a.dw_ret.ptr[src])[tag] = dot;
    }
  }
}

// ------------------------------------------------------------------ source side: wait for the owners, add the slots
// out[t, :] = ret[2t, :] + ret[2t+1, :] (the owners already applied the routing weights); optionally the per-slot
// scalars the owners returned (routing-weight gradients) are copied out as well.
__global__ void __launch_bounds__(256) ep_combine_kernel(const __nv_bfloat16* __restrict__ ret,
                                                         const float* __restrict__ ret_scalar,
                                                         __nv_bfloat16* __restrict__ out, float* __restrict__ scalars,
                                                         int tokens, int D, const int* my_sig, int sig_slot, int n,
                                                         int seq, int* status) {
  int ok = 1;
  if (threadIdx.x < n && !wait_one(my_sig, sig_slot, threadIdx.x, seq, status)) {
    atomicCAS(status, 0, 104);
    ok = 0;
  }
  if (!__syncthreads_and(ok)) return;      // an owner never delivered: leave the output alone, the status word tells
  const int vecs = D / 8;
  const size_t total = static_cast<size_t>(tokens) * vecs;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / vecs, c = i - t * vecs;
    float x[8], y[8];
    unpack8(reinterpret_cast<const vec16*>(ret + (2 * t) * D)[c], x);
    unpack8(reinterpret_cast<const vec16*>(ret + (2 * t + 1) * D)[c], y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    reinterpret_cast<vec16*>(out + t * D)[c] = pack8(x);
  }
  if (scalars) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < static_cast<size_t>(tokens) * 2;
         i += static_cast<size_t>(gridDim.x) * blockDim.x)
      scalars[i] = ret_scalar[i];
  }
}

}  // namespace ep
}  // namespace b2

using namespace b2;

namespace {

Peers table(const unsigned long long* p) {
  Peers t{};
  for (int i = 0; i < MAX_RANKS; ++i) t.ptr[i] = p ? reinterpret_cast<void*>(p[i]) : nullptr;
  return t;
}

int sms_and_coop(bool* coop_ok) {
  static int sms = 0;
  static bool coop = false;
  if (!sms) {
    int dev = 0, flag = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&flag, cudaDevAttrCooperativeLaunch, dev);
    coop = flag != 0;
  }
  *coop_ok = coop;
  return sms;
}

template <int B_MN, int EPI>
int launch_gather(ep::Params& p, cudaStream_t stream) {
  auto kernel = ep::ep_gather_gemm_kernel<B_MN, EPI>;
  static int usable = -1;
  bool coop = false;
  const int sms = sms_and_coop(&coop);
  if (usable < 0) {
    int per_sm = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ep::SMEM) != cudaSuccess) return -3;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, ep::THREADS, ep::SMEM);
    usable = coop && per_sm >= 1 ? 1 : 0;
  }
  if (!usable) return -20;
  void* args[] = {&p};
  // cooperative: the producer of one CTA waits for rows that the copier warps of all the others bring in, so every
  // CTA has to be resident
  if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(sms), dim3(ep::THREADS), args, ep::SMEM,
                                  stream) != cudaSuccess) {
    cudaGetLastError();
    return -4;
  }
  return 0;
}

}  // namespace

extern "C" {

// Plan of one dispatch (see ep_plan2_kernel).  Pointer tables: MAX_RANKS device addresses each.
int b2_ep_plan2(const long long* idx, const float* weights, int slots, int experts_total, int ep, int rank, int seq,
                int capacity_rows, const unsigned long long* counts_all, const unsigned long long* land_src,
                const unsigned long long* land_tag, const unsigned long long* land_w, const unsigned long long* sig,
                int counts_slot, int meta_slot, int* offs, int* seg_live_end, int* tile_expert, int* meta, int* status,
                cudaStream_t s) {
  if (experts_total > ep::MAX_EXPERTS || ep > MAX_RANKS || ep < 1 || experts_total % ep ||
      ep * experts_total > ep::PLAN_THREADS || capacity_rows % ep::ALIGN_ROWS)
    return -10;
  ep::PlanArgs a{};
  a.idx = idx; a.weights = weights; a.slots = slots; a.experts_total = experts_total; a.ep = ep; a.rank = rank;
  a.seq = seq; a.capacity_rows = capacity_rows; a.counts_all = table(counts_all); a.land_src = table(land_src);
  a.land_tag = table(land_tag); a.land_w = table(land_w); a.sig = table(sig); a.counts_slot = counts_slot;
  a.meta_slot = meta_slot; a.offs = offs; a.seg_live_end = seg_live_end; a.tile_expert = tile_expert; a.meta = meta;
  a.status = status;
  const size_t smem = static_cast<size_t>(experts_total) * ep::PLAN_THREADS * 4;
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(ep::ep_plan2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    set = true;
  }
  ep::ep_plan2_kernel<<<1, ep::PLAN_THREADS, smem, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// Gather + grouped GEMM in one kernel.
//   mode 0  gate/up with SwiGLU: a_buf[cap, K] <- rows of ``src`` (token = tag >> src_shift);
//           h[cap, F] = silu(a W1^T) * (a W3^T) (h may be null); the pre-activations of rows < split_row go to
//           (gate_lo, up_lo), the others to (gate_hi, up_hi); either pair may be null.  w: W1 [E, F, K], w_b: W3.
//   mode 1  dh[cap, N] = a W2 with W2 [E, K, N] read MN-major; a_buf <- rows of ``src``.
// ``gemm_tile_begin``: first 128-row tile the tensor cores compute (the gather always covers every live tile).
// ``handshake``: 0 none, 1 wait for flag ``seq`` in ``sig_slot`` from every rank, 2 raise mine first.
// ``tile_ready`` [cap/128] and ``ticket`` [1]: zero-initialised device words the kernel leaves at zero.
// Returns -20 when the device cannot keep one CTA per SM resident.
int b2_ep_gather_gemm(int mode, void* a_buf, const void* w, const void* w_b, int cap_rows, int N, int K,
                      int num_experts, const int* tile_expert, const int* meta, const int* seg_live_end,
                      int gemm_tile_begin, const unsigned long long* src, int src_shift, const int* row_src,
                      const int* row_tag, const float* row_w, int* save_src, int* save_tag, float* save_w,
                      int* tile_ready, unsigned int* ticket, const unsigned long long* sig, int n, int rank,
                      int sig_slot, int seq, int handshake, void* d, void* gate_lo, void* up_lo, void* gate_hi,
                      void* up_hi, int split_row, int* status, cudaStream_t stream) {
  if (cap_rows % ep::ALIGN_ROWS || K % 64 || n < 1 || n > MAX_RANKS) return -10;
  ep::Params p{};
  p.N = N; p.K = K; p.tile_expert = tile_expert; p.meta = meta; p.seg_live_end = seg_live_end;
  p.gemm_tile_begin = gemm_tile_begin; p.cap_rows = cap_rows; p.src = table(src); p.src_shift = src_shift;
  p.row_src = row_src; p.row_tag = row_tag; p.row_w = row_w; p.save_src = save_src; p.save_tag = save_tag;
  p.save_w = save_w; p.a_buf = static_cast<__nv_bfloat16*>(a_buf); p.tile_ready = tile_ready; p.ticket = ticket;
  p.sig = table(sig); p.n = n; p.rank = rank; p.sig_slot = sig_slot; p.seq = seq; p.handshake = handshake;
  p.d = d; p.gate_lo = gate_lo; p.up_lo = up_lo; p.gate_hi = gate_hi; p.up_hi = up_hi; p.split_row = split_row;
  p.status = status;
  if (make_map(&p.map_a, a_buf, K, cap_rows, K, ep::BM)) return -11;
  if (mode == 0) {
    if (N % 256) return -10;                       // N = 2F, F a multiple of 128
    const int F = N / 2;
    p.b_expert_rows = F; p.ldd = F;
    if (make_map(&p.map_b, w, K, static_cast<long long>(num_experts) * F, K, 128)) return -12;
    if (make_map(&p.map_b2, w_b, K, static_cast<long long>(num_experts) * F, K, 128)) return -12;
    return launch_gather<0, ep::EPI_SWIGLU>(p, stream);
  }
  if (mode == 1) {
    if (N % 32) return -10;
    p.b_expert_rows = K; p.ldd = N;
    if (make_map(&p.map_b, w, N, static_cast<long long>(num_experts) * K, N, 64)) return -12;
    return launch_gather<1, ep::EPI_STORE>(p, stream);
  }
  return -13;
}

int b2_ep_swiglu_bwd(void* dh, const void* gate_lo, const void* up_lo, const void* gate_hi, const void* up_hi,
                     int split_row, void* dgu, const int* meta, const int* row_tag, const int* row_src,
                     const float* row_w, const unsigned long long* dw_ret, int cap_rows, int F, int n,
                     cudaStream_t s) {
  if (F % 8) return -10;
  ep::SwigluBwdArgs a{};
  a.dh = static_cast<__nv_bfloat16*>(dh);
  a.gate_lo = static_cast<const __nv_bfloat16*>(gate_lo); a.up_lo = static_cast<const __nv_bfloat16*>(up_lo);
  a.gate_hi = static_cast<const __nv_bfloat16*>(gate_hi); a.up_hi = static_cast<const __nv_bfloat16*>(up_hi);
  a.split_row = split_row; a.dgu = static_cast<__nv_bfloat16*>(dgu); a.meta = meta; a.row_tag = row_tag;
  a.row_src = row_src; a.row_w = row_w; a.dw_ret = table(dw_ret); a.cap_rows = cap_rows; a.F = F; a.n = n;
  bool coop;
  ep::ep_swiglu_bwd_kernel<<<sms_and_coop(&coop) * 8, 256, 0, s>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int b2_ep_combine(const void* ret, const float* ret_scalar, void* out, float* scalars, int tokens, int D,
                  const int* my_sig, int sig_slot, int n, int seq, int* status, cudaStream_t s) {
  if (D % 8) return -10;
  bool coop;
  ep::ep_combine_kernel<<<sms_and_coop(&coop) * 4, 256, 0, s>>>(
      static_cast<const __nv_bfloat16*>(ret), ret_scalar, static_cast<__nv_bfloat16*>(out), scalars, tokens, D, my_sig,
      sig_slot, n, seq, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"

B2_DEFINE_DEBUG_READER(b2_moe_ep_debug_read)
B2_DEFINE_WAIT_SETTER(b2_moe_ep_file_set_wait_ns)
