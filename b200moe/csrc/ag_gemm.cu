// All-gather fused with the GEMM that consumes the gathered weight:  y[M,N] = x[M,K] * W[N,K]^T  where the rows
// of W are sharded over the ranks of a group and every rank holds a full-size copy of W in symmetric memory in
// which only its own rows are current.  W is a stack of up to four row segments, each sharded evenly (inside a
// segment of S rows rank r owns rows [r S/n, (r + 1) S/n)); one segment is a plain linear layer, three are the
// fused q/k/v projection whose parts are sharded one by one.
//
// One kernel per rank does both jobs.  Each CTA (one per SM, launched cooperatively so that all of them are
// resident) has
//   warp 0       TMA producer      warp 1   MMA issuer (tcgen05, accumulators double-buffered in TMEM)
//   warps 2..5   epilogue          warps 6..9   copiers
// The copier warps of all CTAs together pull the peers' rows over NVLink with plain 16-byte peer loads into
// this rank's own copy of W, one 256-row block of W (= one column of output tiles) after another, and bump a
// per-block counter when their slice of the block is in place.  The output tiles are scheduled so that the
// columns whose weight rows are local come first; the TMA producer of a tile whose weight rows came from a peer
// waits (bounded) for that block's counter, then loads it from LOCAL memory like any other tile.  The remote
// rows therefore cross NVLink exactly once, the copy runs under the tensor-core work of the local columns, and
// after the kernel the whole of W is local (later microbatches and the backward pass use it as it is).
// Every TMA load of this kernel reads this GPU's own memory; peers are read with ordinary loads only.
//
// Replaces, for one linear layer, the reference's per-module weight all-gather followed by the einsum
// (implementation/distributed/ddp_modules.py:24-49, implementation/layers.py:69).
#include "peer.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace b2 {

namespace ag {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int THREADS = 320;
constexpr int COPY_THREADS = 128;
constexpr int COPY_UNROLL = 8;      // 16-byte peer loads in flight per copier thread
constexpr int GROUP_M = 8;
constexpr int MAX_SEG = 4;
constexpr int MAX_BLOCKS = 192;     // column blocks of 256 rows of W: N <= 49152

struct Params {
  CUtensorMap map_a;      // x [M, K]
  CUtensorMap map_b;      // this rank's full copy of W [N, K]
  int M, N, K;
  int n, rank;            // group size, my index
  int num_seg;            // row segments of W
  int seg_begin[MAX_SEG + 1];   // first row of each segment; seg_begin[num_seg] = N
  int seg_shard[MAX_SEG];       // rows per rank inside the segment
  int n_local;            // column blocks whose rows are all mine: order[0 .. n_local)
  unsigned char order[MAX_BLOCKS];   // column blocks in the order they are computed (mine first) and copied
  Peers w;                // every rank's copy of W (same layout); ptr[rank] is map_b's base
  Peers sig;              // signal pads
  int sig_slot, seq;
  int* block_flags;       // [ceil(N/256)] counters in local memory, monotonically increasing over launches
  int flag_epoch;         // launches so far with these counters, this one included
  void* d;                // y [M, N] bf16
  long long ldd;
  int* status;
};

struct Tile {
  int m_tile, n_tile;
};

__host__ __device__ __forceinline__ int owner_of_row(const Params& p, int row) {
  int s = 0;
  while (s + 1 < p.num_seg && row >= p.seg_begin[s + 1]) ++s;
  return (row - p.seg_begin[s]) / p.seg_shard[s];
}

// Tiles come in two phases: first the column blocks whose weight rows are all local, then the others; inside a
// phase the usual grouped raster (8 row tiles share their column blocks) keeps operands in L2.
__device__ __forceinline__ Tile decode(const Params& p, long long tile, int m_tiles, int n_tiles, bool* local) {
  const long long first = static_cast<long long>(m_tiles) * p.n_local;
  const bool ph = tile >= first;
  const int rest = static_cast<int>(ph ? tile - first : tile);
  const int len = ph ? n_tiles - p.n_local : p.n_local;
  const int group = rest / (GROUP_M * len);
  const int first_m = group * GROUP_M;
  const int rows_in_group = min(GROUP_M, m_tiles - first_m);
  const int in_group = rest - group * GROUP_M * len;
  Tile t;
  t.m_tile = first_m + in_group % rows_in_group;
  t.n_tile = p.order[(ph ? p.n_local : 0) + in_group / rows_in_group];
  *local = !ph;
  return t;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void copier_sync() { asm volatile("bar.sync 1, %0;" ::"n"(COPY_THREADS) : "memory"); }

__global__ void __launch_bounds__(THREADS, 1) ag_gemm_kernel(const __grid_constant__ Params p) {
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
  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const long long total_tiles = static_cast<long long>(m_tiles) * n_tiles;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int flag_target = p.flag_epoch * static_cast<int>(gridDim.x);

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
        bool local;
        const Tile t = decode(p, tile, m_tiles, n_tiles, &local);
        if (!local) {
          // rows of this block came (or are coming) from a peer: wait until every CTA has stored its slice
          const int* flag = p.block_flags + t.n_tile;
          bool ok = ld_acquire_gpu(flag) - flag_target >= 0;
          if (!ok) {
            const Deadline deadline;
            while (!(ok = ld_acquire_gpu(flag) - flag_target >= 0)) {
              if (deadline.expired()) break;
              __nanosleep(200);
            }
          }
          if (!ok) {
            *abort_flag = 1;
            atomicExch(p.status, 301);
            break;
          }
          fence_proxy_async_all();   // the copiers' generic-proxy stores before my async-proxy (TMA) reads
        }
        const int m0 = t.m_tile * BM, n0 = t.n_tile * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            *abort_flag = 1;
            atomicExch(p.status, 302);
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, &p.map_a, &full_bar[stage], kb * BK, m0);
          tma_load_2d(sa + A_BYTES, &p.map_b, &full_bar[stage], kb * BK, n0);
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
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0, 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      for (long long tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          *abort_flag = 1;
          atomicExch(p.status, 303);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool failed = false;
        for (int kb = 0; kb < k_blocks; ++kb) {
          // the producer may be waiting for a peer copy (bounded by the cross-GPU wait budget): keep waiting in
          // mbarrier-budget slices until that budget, plus a slice, is over
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
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_ss(d_tmem, umma_smem_desc(sa + k * 32, 16, 1024), umma_smem_desc(sb + k * 32, 16, 1024), idesc,
                         (kb | k) != 0);
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (failed) {
          if (!*abort_flag) atomicExch(p.status, 304);
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
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.d);
    for (long long tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
      bool local;
      const Tile t = decode(p, tile, m_tiles, n_tiles, &local);
      bool got = false;
      const Deadline deadline;
      while (!got && !*abort_flag) {
        got = mbar_wait(&tmem_full[acc], acc_phase);
        if (!got && deadline.expired()) break;
      }
      if (!got) {
        if (!*abort_flag) atomicExch(p.status, 305);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      const long long row = static_cast<long long>(t.m_tile) * BM + row_in_tile;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c, v);
        tmem_ld_wait();
        const long long col = static_cast<long long>(t.n_tile) * BN + c;
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
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------ copiers (warps 6..9)
    const int ct = threadIdx.x - 6 * 32;                     // 0..127
    if (ct == 0) {
      // my own rows were written by earlier work on this stream: tell the peers they may read them
      if (blockIdx.x == 0) {
        __threadfence_system();
        signal_all(p.sig, p.sig_slot, p.rank, p.n, p.seq);
      }
      const int* my_sig = static_cast<const int*>(p.sig.ptr[p.rank]);
      for (int src = 0; src < p.n; ++src) {
        if (src != p.rank && !wait_one(my_sig, p.sig_slot, src, p.seq, p.status)) {
          atomicExch(p.status, 306);
          *copy_ok = 0;
        }
      }
    }
    copier_sync();
    if (*copy_ok) {
      const long long vec_per_row = p.K / 8;                    // 16-byte vectors per row of W
      uint4* mine = static_cast<uint4*>(p.w.ptr[p.rank]);
      for (int i = p.n_local; i < n_tiles; ++i) {
        const int nb = p.order[i];
        const int row0 = nb * BN;
        const long long vecs = static_cast<long long>(min(BN, p.N - row0)) * vec_per_row;
        const long long lo = vecs * blockIdx.x / gridDim.x, hi = vecs * (blockIdx.x + 1) / gridDim.x;
        const long long base = static_cast<long long>(row0) * vec_per_row;
        for (long long v0 = lo + ct; v0 < hi; v0 += static_cast<long long>(COPY_THREADS) * COPY_UNROLL) {
          uint4 r[COPY_UNROLL];
          bool live[COPY_UNROLL];
#pragma unroll
          for (int u = 0; u < COPY_UNROLL; ++u) {
            const long long v = v0 + static_cast<long long>(u) * COPY_THREADS;
            live[u] = false;
            if (v < hi) {
              const int owner = owner_of_row(p, row0 + static_cast<int>(v / vec_per_row));
              if (owner != p.rank) {
                live[u] = true;
                r[u] = __ldcg(static_cast<const uint4*>(p.w.ptr[owner]) + base + v);
              }
            }
          }
#pragma unroll
          for (int u = 0; u < COPY_UNROLL; ++u)
            if (live[u]) __stcg(mine + base + v0 + static_cast<long long>(u) * COPY_THREADS, r[u]);
        }
        __threadfence();
        fence_proxy_async_all();
        copier_sync();
        if (ct == 0) red_release_gpu_add(p.block_flags + nb, 1);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ag
}  // namespace b2

using namespace b2;

// Host side of the schedule: row ownership from the segment sizes, then the order in which column blocks are
// computed and copied — blocks whose rows are all mine first, then the others starting after my last own block, so
// that the ranks do not all read the same peer rows at the same time.  Returns non-zero for an invalid layout.
static int plan_blocks(ag::Params& p, const int* seg_rows, int num_seg, int n, int rank, int N) {
  if (n < 1 || n > MAX_RANKS || rank < 0 || rank >= n || num_seg < 1 || num_seg > ag::MAX_SEG || N < 1 ||
      (N + ag::BN - 1) / ag::BN > ag::MAX_BLOCKS)
    return -1;
  p.N = N; p.n = n; p.rank = rank; p.num_seg = num_seg; p.n_local = 0;
  int row = 0;
  for (int s = 0; s < num_seg; ++s) {
    if (seg_rows[s] <= 0 || seg_rows[s] % n) return -1;
    p.seg_begin[s] = row;
    p.seg_shard[s] = seg_rows[s] / n;
    row += seg_rows[s];
  }
  if (row != N) return -1;
  p.seg_begin[num_seg] = N;
  const int n_tiles = (N + ag::BN - 1) / ag::BN;
  int others[ag::MAX_BLOCKS], n_others = 0, last_local = -1;
  for (int b = 0; b < n_tiles; ++b) {
    const int lo = b * ag::BN, hi = (lo + ag::BN < N ? lo + ag::BN : N) - 1;
    bool mine = true;
    // ownership changes only at shard boundaries: checking every row of a 256-row block is cheap on the host
    for (int r = lo; r <= hi && mine; ++r) mine = ag::owner_of_row(p, r) == rank;
    if (mine) {
      p.order[p.n_local++] = static_cast<unsigned char>(b);
      last_local = b;
    } else {
      others[n_others++] = b;
    }
  }
  int start = 0;
  while (start < n_others && others[start] < last_local) ++start;
  for (int i = 0; i < n_others; ++i) p.order[p.n_local + i] = static_cast<unsigned char>(others[(start + i) % n_others]);
  return 0;
}

extern "C" {

// The schedule of ``b2_ag_gemm_nt`` for one rank, computed on the host without touching a device (for tests and
// tools): ``order_out`` [ceil(N/256)] column blocks in launch order, ``n_local_out`` how many of them need no peer
// rows, ``owner_out`` (optional) [N] the rank that owns each row.  Returns non-zero for an invalid layout.
int b2_ag_gemm_plan(const int* seg_rows, int num_seg, int n, int rank, int N, int* order_out, int* n_local_out,
                    int* owner_out) {
  ag::Params p{};
  if (plan_blocks(p, seg_rows, num_seg, n, rank, N)) return -10;
  const int n_tiles = (N + ag::BN - 1) / ag::BN;
  for (int i = 0; i < n_tiles; ++i) order_out[i] = p.order[i];
  *n_local_out = p.n_local;
  if (owner_out)
    for (int r = 0; r < N; ++r) owner_out[r] = ag::owner_of_row(p, r);
  return 0;
}

// y[M,N] = x[M,K] * W[N,K]^T with W row-sharded over ``n`` ranks.  ``seg_rows``: rows of each of the ``num_seg``
// stacked segments of W (their sum is N; each a multiple of n).  ``w_peers``/``sig``: MAX_RANKS device addresses
// (each rank's copy of W, each rank's signal pad).  ``block_flags``: int32 [ceil(N/256)] in local memory, zeroed
// once at allocation; ``flag_epoch`` counts the launches that used it (1 for the first).  Every launch with the
// same counters must use the same grid, which is the SM count.  Returns -20 when the device cannot co-schedule
// one CTA per SM (the caller then gathers and multiplies separately).
int b2_ag_gemm_nt(const void* x, const unsigned long long* w_peers, void* y, int M, int N, int K, long long ldx,
                  long long ldy, const int* seg_rows, int num_seg, int n, int rank, const unsigned long long* sig,
                  int sig_slot, int seq, int* block_flags, int flag_epoch, int* status, cudaStream_t stream) {
  if (N % 32 || K % 8) return -10;
  ag::Params p{};
  p.M = M; p.K = K;
  if (plan_blocks(p, seg_rows, num_seg, n, rank, N)) return -10;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.w.ptr[i] = i < n ? reinterpret_cast<void*>(w_peers[i]) : nullptr;
    p.sig.ptr[i] = i < n ? reinterpret_cast<void*>(sig[i]) : nullptr;
  }
  if (make_map(&p.map_a, x, K, M, ldx, ag::BM)) return -11;
  if (make_map(&p.map_b, p.w.ptr[rank], K, N, K, ag::BN)) return -12;
  p.sig_slot = sig_slot; p.seq = seq;
  p.block_flags = block_flags; p.flag_epoch = flag_epoch; p.d = y; p.ldd = ldy; p.status = status;
  static int sms = 0;
  static bool usable = false;
  if (!sms) {
    int dev = 0, coop = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (cudaFuncSetAttribute(ag::ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ag::SMEM) != cudaSuccess)
      return -3;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ag::ag_gemm_kernel, ag::THREADS, ag::SMEM);
    usable = coop && per_sm >= 1;
  }
  if (!usable) return -20;
  void* args[] = {&p};
  if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ag::ag_gemm_kernel), dim3(sms), dim3(ag::THREADS), args,
                                  ag::SMEM, stream) != cudaSuccess) {
    cudaGetLastError();
    return -20;
  }
  return 0;
}

// Grid size every launch of ``b2_ag_gemm_nt`` uses (the counters advance by this much per launch).
int b2_ag_gemm_grid() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // extern "C"

B2_DEFINE_WAIT_SETTER(b2_ag_gemm_file_set_wait_ns)
