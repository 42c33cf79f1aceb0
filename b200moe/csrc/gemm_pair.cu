// bf16 GEMM on CTA pairs (tcgen05 cta_group::2):  y[M,N] = x[M,K] * W[N,K]^T.
//
// Two CTAs of a cluster (two SMs) share one 256 x 256 output tile.  Each CTA stages only its own half of the
// operands by TMA — 128 rows of x and 128 rows of W per 64-wide k-block, 32 KiB per stage instead of the 48 KiB a
// single CTA needs for 128 x 256 — the even CTA (the leader) issues one tcgen05.mma.cta_group::2 per 16-wide
// k-step that reads both CTAs' shared memory, and every CTA's tensor memory receives its 128 rows x 256 columns of
// the accumulator.  So a pair moves a third fewer operand bytes per FLOP than two independent 128 x 256 CTAs (as
// a single-CTA 256 x 256 tile would) while each CTA still has room for two accumulators in its 512 TMEM columns:
// the epilogue of tile i runs under the main loop of tile i + 1.
//
// Synchronisation inside a pair (all mbarrier waits are bounded and end in a status code):
//   full[stage]   on the leader: one arrive.expect_tx by the leader's producer for the bytes of BOTH CTAs; each
//                 CTA's own tile loads complete on it (the loads carry the leader's barrier address);
//   empty[stage]  on each CTA: signalled by a tcgen05.commit of the leader's MMA thread per CTA;
//   acc_full[b]   on each CTA: commit after the last k-block of a tile;
//   acc_empty[b]  on the leader: the four epilogue warps of both CTAs arrive (remote arrive from the peer).
// A cluster barrier after the barrier initialisation and before the TMEM release brackets the kernel.
#include "ptx.cuh"
#include "tensormap.cuh"

namespace b2 {
namespace pair {

constexpr int TILE_M = 256, TILE_N = 256, BK = 64;
constexpr int HALF = 128;                          // rows of A / rows of B staged by one CTA
constexpr int A_BYTES = HALF * BK * 2;             // 16 KiB
constexpr int B_BYTES = HALF * BK * 2;             // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;     // per CTA
constexpr int STAGES = 6;
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 192;
constexpr int GROUP_M = 8;

struct Params {
  CUtensorMap map_a;     // x [M, K], box 128 x 64
  CUtensorMap map_b;     // W [N, K], box 128 x 64
  int M, N, K;
  int acc_bufs;          // 1 or 2 accumulators of 256 columns
  void* d;               // y [M, N] bf16
  long long ldd;
  int* status;
  int* probe;            // optional int[4]: {leader TMEM base, peer TMEM base, 0, 0} of pair 0
};

struct Tile {
  int m_tile, n_tile;
};

__device__ __forceinline__ Tile decode(long long tile, int m_tiles, int n_tiles) {
  const int group = static_cast<int>(tile / (GROUP_M * n_tiles));
  const int first_m = group * GROUP_M;
  const int rows_in_group = min(GROUP_M, m_tiles - first_m);
  const int in_group = static_cast<int>(tile - static_cast<long long>(group) * GROUP_M * n_tiles);
  Tile t;
  t.m_tile = first_m + in_group % rows_in_group;
  t.n_tile = in_group / rows_in_group;
  return t;
}

__global__ void __launch_bounds__(THREADS, 1) gemm_pair_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();            // 0: leader, 1: peer
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int m_tiles = (p.M + TILE_M - 1) / TILE_M;
  const int n_tiles = (p.N + TILE_N - 1) / TILE_N;
  const long long total_tiles = static_cast<long long>(m_tiles) * n_tiles;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int nacc = p.acc_bufs;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);       // four epilogue warps of each CTA
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.map_a);
    tma_prefetch_desc(&p.map_b);
  }
  __syncthreads();
  cluster_sync_all();                     // both CTAs' barriers exist before anything remote touches them
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 256 * nacc);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (p.probe && pair_id == 0 && threadIdx.x == 0) p.probe[cta] = static_cast<int>(tmem_base);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (long long tile = pair_id; tile < total_tiles && !*abort_flag; tile += num_pairs) {
        const Tile t = decode(tile, m_tiles, n_tiles);
        const int m0 = t.m_tile * TILE_M + static_cast<int>(cta) * HALF;
        const int n0 = t.n_tile * TILE_N + static_cast<int>(cta) * HALF;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            *abort_flag = 1;
            atomicExch(p.status, 501);
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          const uint32_t full_on_leader = mapa_u32(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &p.map_a, full_on_leader, kb * BK, m0);
          tma_load_2d_pair(sa + A_BYTES, &p.map_b, full_on_leader, kb * BK, n0);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (cta == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, TILE_N, 0, 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (long long tile = pair_id; tile < total_tiles && !*abort_flag; tile += num_pairs) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1)) {
          *abort_flag = 1;
          atomicExch(p.status, 502);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TILE_N;
        bool failed = false;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_ss_pair(d_tmem, umma_smem_desc(sa + k * 32, 16, 1024), umma_smem_desc(sb + k * 32, 16, 1024),
                              idesc, (kb | k) != 0);
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(mapa_u32(smem_u32(&empty_bar[stage]), 0));
          umma_commit_pair(mapa_u32(smem_u32(&empty_bar[stage]), 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (failed) {
          *abort_flag = 1;
          atomicExch(p.status, 503);
          break;
        }
        umma_commit_pair(mapa_u32(smem_u32(&acc_full[acc]), 0));
        umma_commit_pair(mapa_u32(smem_u32(&acc_full[acc]), 1));
        if (++acc == nacc) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quad = warp & 3;
    const int row_in_half = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.d);
    for (long long tile = pair_id; tile < total_tiles && !*abort_flag; tile += num_pairs) {
      const Tile t = decode(tile, m_tiles, n_tiles);
      bool got = false;
      for (int tries = 0; tries < 4 && !got && !*abort_flag; ++tries) got = mbar_wait(&acc_full[acc], acc_phase);
      if (!got) {
        if (!*abort_flag) atomicExch(p.status, 504);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * TILE_N + (static_cast<uint32_t>(quad * 32) << 16);
      const long long row = static_cast<long long>(t.m_tile) * TILE_M + static_cast<int>(cta) * HALF + row_in_half;
#pragma unroll 1
      for (int c = 0; c < TILE_N; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c, v);
        tmem_ld_wait();
        const long long col = static_cast<long long>(t.n_tile) * TILE_N + c;
        if (row >= p.M || col >= p.N) continue;   // N is a multiple of 32 (checked on the host)
        uint4* dst = reinterpret_cast<uint4*>(out + row * p.ldd + col);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          dst[i] = make_uint4(pack_bf16(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])),
                              pack_bf16(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])),
                              pack_bf16(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])),
                              pack_bf16(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7])));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[acc]), 0));
      if (++acc == nacc) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                     // the peer's tensor memory and barriers are idle as well
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 256 * nacc);
  }
}

}  // namespace pair
}  // namespace b2

using namespace b2;

static int g_max_pairs = -1;

extern "C" {

// y[M,N] (bf16) = x[M,K] * w[N,K]^T on CTA pairs.  ``acc_bufs``: 2 (epilogue overlapped) or 1.  ``probe``: optional
// device int[4] receiving the TMEM base address seen by the two CTAs of pair 0.  Returns -20 if the device cannot
// run clusters of two CTAs with this kernel's shared memory.
int b2_gemm_pair_nt(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw,
                    long long ldy, int acc_bufs, int* probe, int* status, cudaStream_t stream) {
  if (N % 32 || K % 8 || (acc_bufs != 1 && acc_bufs != 2)) return -10;
  pair::Params p{};
  if (make_map(&p.map_a, x, K, M, ldx, pair::HALF)) return -11;
  if (make_map(&p.map_b, w, K, N, ldw, pair::HALF)) return -12;
  p.M = M; p.N = N; p.K = K; p.acc_bufs = acc_bufs; p.d = y; p.ldd = ldy; p.status = status; p.probe = probe;
  int& max_pairs = g_max_pairs;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.blockDim = dim3(pair::THREADS);
  cfg.dynamicSmemBytes = pair::SMEM;
  cfg.stream = stream;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (max_pairs < 0) {
    if (cudaFuncSetAttribute(pair::gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM) !=
        cudaSuccess)
      return -3;
    int dev = 0, sms = 0, clusters = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(sms / 2 * 2);
    if (cudaOccupancyMaxActiveClusters(&clusters, pair::gemm_pair_kernel, &cfg) != cudaSuccess) {
      cudaGetLastError();
      clusters = 0;
    }
    max_pairs = clusters;
  }
  if (max_pairs < 1) return -20;
  const long long tiles = static_cast<long long>((M + pair::TILE_M - 1) / pair::TILE_M) *
                          ((N + pair::TILE_N - 1) / pair::TILE_N);
  const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
  cfg.gridDim = dim3(2 * pairs);
  if (cudaLaunchKernelEx(&cfg, pair::gemm_pair_kernel, p) != cudaSuccess) {
    cudaGetLastError();
    return -4;
  }
  return 0;
}

// Pairs of CTAs the device keeps resident for this kernel (0: unsupported, -1: not asked yet).
int b2_gemm_pair_max_pairs() { return g_max_pairs; }

}  // extern "C"
