// bf16 GEMM family on 5th-generation tensor cores (tcgen05), fp32 accumulation in
// tensor memory, operands staged by TMA (one plain tile load per CTA and tile).
//
// One persistent kernel template covers every contraction of the training step:
//   NT  y = x W^T            (forward linears, grouped expert forward)
//   NN  dx = dy W            (data gradients; W is read MN-major, no transpose copy)
//   TN  dW (+)= dy^T x       (weight gradients, accumulated in fp32 or bf16 in place)
// with a device-side tile table for grouped (per-expert) problems, a fused
// SwiGLU epilogue for the gate/up projection and a K-concatenated form for
// dx = dgate W1 + dup W3.
//
// Layout of one CTA (192 threads, one CTA per SM):
//   warp 0       TMA producer (one elected lane)
//   warp 1       tensor-memory allocation, MMA issue (one elected lane)
//   warps 2..5   epilogue: tcgen05.ld the 128 x BN fp32 tile, convert, store
// The accumulator is double-buffered in TMEM (2 x 256 columns), so the epilogue
// of tile i overlaps the main loop of tile i+1.  Shared memory holds a 4-stage
// ring of {A 128x64, B 256x64} bf16 tiles in the 128-byte-swizzled layout that
// both TMA and the MMA descriptors understand.
#include "peer.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace b2 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int A_SUB_BYTES = BM * BK * 2;   // 16 KiB per 128-row sub-tile of A
constexpr int B_BYTES = BN * BK * 2;       // 32 KiB
constexpr int GEMM_THREADS = 192;
// MT = 128-row sub-tiles of A per CTA tile.  MT=1: 128x256 tile, 4 stages, accumulator double-buffered in
// TMEM (epilogue overlaps the next main loop).  MT=2: 256x256 tile (two MMAs per k-step share the B tile in
// shared memory, a third fewer operand bytes per FLOP), 3 stages, both accumulators fill TMEM.
// PAIR = 1 (with MT = 1): two CTAs of a cluster share a 256x256 tile (tcgen05 cta_group::2).  Each CTA stages its
// own 128 rows of A and 128 rows/columns of B (32 KiB per stage, 6 stages), the even CTA issues the MMAs for both,
// and each CTA's tensor memory holds its 128 rows x 256 columns, double-buffered: the operand traffic of a 256x256
// tile with the epilogue overlap of a 128x256 one.
template <int MT, int PAIR = 0> struct Cfg {
  static constexpr int STAGES = PAIR ? 6 : (MT == 2 ? 3 : 4);
  static constexpr int A_BYTES = MT * A_SUB_BYTES;
  static constexpr int B_STAGE_BYTES = PAIR ? B_BYTES / 2 : B_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_STAGE_BYTES;
  static constexpr int NACC = MT == 2 ? 1 : 2;
  static constexpr int TM = PAIR ? 2 : MT;     // 128-row units per output tile
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int PUSH_STAGING = 4 * 32 * 256;   // EPI_PUSH: 32 rows x 128 bf16 columns per epilogue warp
};
template <int EPI, int MT, int PAIR = 0> constexpr int smem_bytes() {
  return Cfg<MT, PAIR>::SMEM + (EPI == 5 /*EPI_PUSH*/ ? Cfg<MT, PAIR>::PUSH_STAGING : 0);
}
constexpr int GROUP_M = 8;

enum Epilogue : int {
  EPI_STORE_BF16 = 0,   // D[M,N] bf16 = acc
  EPI_ACC_F32 = 1,      // D[M,N] fp32 += acc   (beta selects += or =)
  EPI_ACC_BF16 = 2,     // D[M,N] bf16 += acc
  EPI_SWIGLU = 3,       // H[M,N/2] = silu(acc[:, :128]) * acc[:, 128:]; optional gate/up stores
  EPI_STORE_F32 = 4,    // D[M,N] fp32 = acc
  EPI_ROPE = 6,         // D[M,N] bf16 = acc with the rotary embedding applied to the leading rope_cols columns
                        // (adjacent pairs, heads of 128 columns, position = row mod rope_seq): the fused q/k/v projection
  EPI_PUSH = 5,         // expert-parallel return: row r, scaled by push_w[r], is stored as bf16 into row push_tag[r]
                        // of rank push_src[r]'s buffer through its peer pointer; the last CTA raises a flag
};

enum Schedule : int {
  SCHED_FLAT = 0,       // tiles over (M, N); optional per-m-tile expert for B
  SCHED_WGRAD = 1,      // tiles over (expert, M, N); K range = rows of the expert
};

struct GemmParams {
  CUtensorMap map_a;
  CUtensorMap map_b;
  CUtensorMap map_b2;          // second B: up-projection (SwiGLU) or K-continuation (k >= k_split)
  int M, N, K;                 // problem per expert for SCHED_WGRAD (K unused there)
  int num_experts;             // >= 1
  int b_expert_rows;           // rows of one expert in the B map (outer TMA coordinate pitch)
  int k_split;                 // K index where map_b2 takes over (0 = unused)
  const int* tile_expert;      // [m_tiles] expert of each m-tile, or null
  const int* num_m_tiles;      // device scalar: live 128-row tiles, or null (= ceil(M/128))
  int group_align256;          // grouped problems: every expert segment is a multiple of 256 rows
  const int* expert_offsets;   // [E] cumulative row ends (SCHED_WGRAD)
  void* d;                     // output
  void* d_gate;                // optional gate pre-activation (SwiGLU)
  void* d_up;                  // optional up pre-activation (SwiGLU)
  long long ldd;               // leading dimension of d (elements)
  long long d_expert_stride;   // elements between experts in d (SCHED_WGRAD)
  float beta;                  // 1 accumulate, 0 overwrite (EPI_ACC_*)
  int* status;                 // device word; non-zero = a wait ran out
  // EPI_ROPE only
  const float* rope_cos;       // [rope_seq, 64] fp32
  const float* rope_sin;
  int rope_cols, rope_seq;
  // EPI_PUSH only
  Peers push_dst;              // every rank's return buffer [slots, ldd] bf16
  const int* push_tag;         // [M] destination row (slot id) of each row, -1 for padding rows
  const int* push_src;         // [M] destination rank
  const float* push_w;         // [M] scale (routing weight), or null for 1
  Peers push_sig;              // signal pads
  int push_slot, push_seq, push_rank, push_n;
  unsigned int* push_ticket;   // self-resetting CTA counter
};

struct TileCoord {
  int m_tile, n_tile, expert, k_begin, k_blocks;
  bool valid;
};

template <int SCHED, int MT>
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, long long tile, int m_tiles, int n_tiles) {
  TileCoord t;
  t.valid = true;
  if (SCHED == SCHED_WGRAD) {
    const long long per_expert = static_cast<long long>(m_tiles) * n_tiles;
    t.expert = static_cast<int>(tile / per_expert);
    const int rest = static_cast<int>(tile - t.expert * per_expert);
    const int group = rest / (GROUP_M * n_tiles);
    const int first_m = group * GROUP_M;
    const int rows_in_group = min(GROUP_M, m_tiles - first_m);
    const int in_group = rest - group * GROUP_M * n_tiles;
    t.m_tile = first_m + in_group % rows_in_group;
    t.n_tile = in_group / rows_in_group;
    const int begin = t.expert == 0 ? 0 : p.expert_offsets[t.expert - 1];
    const int end = p.expert_offsets[t.expert];
    t.k_begin = begin;
    t.k_blocks = (end - begin + BK - 1) / BK;
  } else {
    const int group = static_cast<int>(tile / (GROUP_M * n_tiles));
    const int first_m = group * GROUP_M;
    const int rows_in_group = min(GROUP_M, m_tiles - first_m);
    const int in_group = static_cast<int>(tile - static_cast<long long>(group) * GROUP_M * n_tiles);
    t.m_tile = first_m + in_group % rows_in_group;
    t.n_tile = in_group / rows_in_group;
    t.expert = p.tile_expert ? p.tile_expert[t.m_tile * MT] : 0;
    t.k_begin = 0;
    t.k_blocks = (p.K + BK - 1) / BK;
  }
  return t;
}

template <int A_MN, int B_MN, int EPI, int SCHED, int MT, int PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
  static_assert(!PAIR || MT == 1, "a CTA of a pair holds one 128-row sub-tile");
  constexpr int STAGES = Cfg<MT, PAIR>::STAGES;
  constexpr int A_BYTES = Cfg<MT, PAIR>::A_BYTES;
  constexpr int STAGE_BYTES = Cfg<MT, PAIR>::STAGE_BYTES;
  constexpr int NACC = Cfg<MT, PAIR>::NACC;
  constexpr int TM = Cfg<MT, PAIR>::TM;
  constexpr int TILE_M = BM * TM;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // pair mode: ``cta`` is this CTA's half of the tile (0 = leader), a "worker" is a CTA pair
  const uint32_t cta = PAIR ? cluster_ctarank() : 0;
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int num_workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int m_tiles = p.num_m_tiles ? (*p.num_m_tiles + TM - 1) / TM : (p.M + TILE_M - 1) / TILE_M;
  const int n_tiles = (p.N + BN - 1) / BN;
  const long long total_tiles = static_cast<long long>(m_tiles) * n_tiles * (SCHED == SCHED_WGRAD ? p.num_experts : 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], PAIR ? 8 : 4);   // epilogue warps (of both CTAs of a pair)
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.map_a);
    tma_prefetch_desc(&p.map_b);
    if (EPI == EPI_SWIGLU || p.k_split > 0) tma_prefetch_desc(&p.map_b2);
  }
  if (PAIR) {
    __syncthreads();
    cluster_sync_all();      // both CTAs' barriers exist before a remote arrive or a remote completion can reach them
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, 512);     // one collective allocation by one warp of each CTA
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (every CTA)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (long long tile = worker; tile < total_tiles && !*abort_flag; tile += num_workers) {
        const TileCoord t = decode_tile<SCHED, TM>(p, tile, m_tiles, n_tiles);
        const int m0 = t.m_tile * TILE_M + (PAIR ? static_cast<int>(cta) * BM : 0);
        const int n0 = t.n_tile * BN + (PAIR ? static_cast<int>(cta) * (BN / 2) : 0);
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            *abort_flag = 1;
            atomicExch(p.status, 1);
            break;
          }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          // pair: the leader's barrier counts the bytes of both CTAs; every load names that barrier
          uint64_t* const full = &full_bar[stage];
          const uint32_t full_on_leader = PAIR ? mapa_u32(smem_u32(full), 0) : 0;
          if (!PAIR) mbar_expect_tx(full, STAGE_BYTES);
          else if (cta == 0) mbar_expect_tx(full, 2 * STAGE_BYTES);
          auto load = [&](void* dst, const CUtensorMap* map, int c0, int c1) {
            if (PAIR) tma_load_2d_pair(dst, map, full_on_leader, c0, c1);
            else tma_load_2d(dst, map, full, c0, c1);
          };
          const int k0 = t.k_begin + kb * BK;
          // ---- A
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            if (A_MN) {
              // MN-major: two boxes of [64 (m) x 64 (k)]; inner coordinate = m, outer = k row
              load(sa + i * A_SUB_BYTES, &p.map_a, m0 + i * BM, k0);
              load(sa + i * A_SUB_BYTES + 8192, &p.map_a, m0 + i * BM + 64, k0);
            } else {
              load(sa + i * A_SUB_BYTES, &p.map_a, k0, m0 + i * BM);
            }
          }
          // ---- B
          if (EPI == EPI_SWIGLU) {
            // gate rows then up rows of the same 128 output features (K-major)
            const int row = t.expert * p.b_expert_rows + t.n_tile * 128;
            if (PAIR) {
              load(sb, cta == 0 ? &p.map_b : &p.map_b2, k0, row);      // leader: gate rows, peer: up rows
            } else {
              load(sb, &p.map_b, k0, row);
              load(sb + 16384, &p.map_b2, k0, row);
            }
          } else if (B_MN) {
            const bool second = p.k_split > 0 && k0 >= p.k_split;
            const CUtensorMap* map = second ? &p.map_b2 : &p.map_b;
            const int krow = (SCHED == SCHED_WGRAD ? 0 : t.expert * p.b_expert_rows) + (second ? k0 - p.k_split : k0);
#pragma unroll
            for (int c = 0; c < (PAIR ? BN / 128 : BN / 64); ++c) load(sb + c * 8192, map, n0 + c * 64, krow);
          } else {
            load(sb, &p.map_b, k0, t.expert * p.b_expert_rows + n0);     // box of 256 rows (128 in pair mode)
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (the leader of a pair)
    if (cta == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(PAIR ? 2 * BM : BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      // arrive on the same barrier of every CTA of the pair once the MMAs issued so far have retired
      auto commit = [&](uint64_t* bar) {
        if (PAIR) {
          umma_commit_pair(mapa_u32(smem_u32(bar), 0));
          umma_commit_pair(mapa_u32(smem_u32(bar), 1));
        } else {
          umma_commit(bar);
        }
      };
      for (long long tile = worker; tile < total_tiles && !*abort_flag; tile += num_workers) {
        const TileCoord t = decode_tile<SCHED, TM>(p, tile, m_tiles, n_tiles);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) {
          *abort_flag = 1;
          atomicExch(p.status, 2);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (MT == 2 ? 0 : acc * BN);
        bool failed = false;
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t db = B_MN ? umma_smem_desc(sb + k * 2048, 8192, 1024) : umma_smem_desc(sb + k * 32, 16, 1024);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
              const uint32_t sai = sa + i * A_SUB_BYTES;
              const uint64_t da = A_MN ? umma_smem_desc(sai + k * 2048, 8192, 1024) : umma_smem_desc(sai + k * 32, 16, 1024);
              if (PAIR) umma_bf16_ss_pair(d_tmem + i * BN, da, db, idesc, (kb | k) != 0);
              else umma_bf16_ss(d_tmem + i * BN, da, db, idesc, (kb | k) != 0);
            }
          }
          commit(&empty_bar[stage]);   // frees the stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (failed) {
          *abort_flag = 1;
          atomicExch(p.status, 3);
          break;
        }
        commit(&tmem_full[acc]);
        if (++acc == NACC) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;                 // TMEM lane group this warp may read
    const int row_in_tile = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (long long tile = worker; tile < total_tiles && !*abort_flag; tile += num_workers) {
      const TileCoord t = decode_tile<SCHED, TM>(p, tile, m_tiles, n_tiles);
      if (!mbar_wait(&tmem_full[acc], acc_phase)) {
        *abort_flag = 1;
        atomicExch(p.status, 4);
        break;
      }
      tc_fence_after();
      const bool empty_k = t.k_blocks == 0;   // an expert without rows contributes nothing
#pragma unroll 1
      for (int sub = 0; sub < MT; ++sub) {
      const uint32_t taddr = tmem_base + (MT == 2 ? sub * BN : acc * BN) + (static_cast<uint32_t>(quad * 32) << 16);
      const long long row = static_cast<long long>(t.m_tile) * TILE_M + (PAIR ? static_cast<int>(cta) : sub) * BM + row_in_tile;
      const bool row_ok = row < p.M;
      if (EPI == EPI_SWIGLU) {
        __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(p.d);
        const long long half_n = p.N / 2;
        const long long col0 = static_cast<long long>(t.n_tile) * 128;
#pragma unroll 1
        for (int c = 0; c < 128; c += 32) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + c, g);
          tmem_ld_32x32(taddr + 128 + c, u);
          tmem_ld_wait();
          if (row_ok && col0 + c < half_n) {
            uint32_t out[16], og[16], ou[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
              const float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
              const float h0 = g0 / (1.f + __expf(-g0)) * u0;
              const float h1 = g1 / (1.f + __expf(-g1)) * u1;
              out[i] = pack_bf16(h0, h1);
              og[i] = pack_bf16(g0, g1);
              ou[i] = pack_bf16(u0, u1);
            }
            const long long off = row * half_n + col0 + c;
            uint4* dst = reinterpret_cast<uint4*>(h + off);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
            if (p.d_gate) {
              uint4* dg = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.d_gate) + off);
              uint4* du = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.d_up) + off);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                dg[i] = make_uint4(og[4 * i], og[4 * i + 1], og[4 * i + 2], og[4 * i + 3]);
                du[i] = make_uint4(ou[4 * i], ou[4 * i + 1], ou[4 * i + 2], ou[4 * i + 3]);
              }
            }
          }
        }
      } else if (EPI == EPI_PUSH) {
        // Rows leave for other GPUs.  A thread owns one row of the accumulator, so storing straight from registers
        // would put 16 bytes per lane at 32 different rows in every store instruction.  Instead each warp stages
        // 128 columns of its 32 rows in shared memory (16-byte units XOR-swizzled by row: conflict-free both ways) and
        // writes them out two rows per instruction, 256 contiguous bytes per row.
        const long long col_base = static_cast<long long>(t.n_tile) * BN;
        uint4* stage = reinterpret_cast<uint4*>(smem + STAGES * STAGE_BYTES + 256) + (warp - 2) * (32 * 16);
        int tag = -1, dest = -1;
        float w = 1.f;
        if (row_ok) {
          tag = p.push_tag[row];
          dest = p.push_src[row];
          if (p.push_w) w = p.push_w[row];
          if (dest < 0 || dest >= p.push_n) tag = -1;          // padding row: nobody waits for it
        }
#pragma unroll 1
        for (int half = 0; half < BN / 128; ++half) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + half * 128 + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i)
              stage[lane * 16 + ((c * 4 + i) ^ (lane & 15))] =
                  make_uint4(pack_bf16(w * __uint_as_float(v[8 * i]), w * __uint_as_float(v[8 * i + 1])),
                             pack_bf16(w * __uint_as_float(v[8 * i + 2]), w * __uint_as_float(v[8 * i + 3])),
                             pack_bf16(w * __uint_as_float(v[8 * i + 4]), w * __uint_as_float(v[8 * i + 5])),
                             pack_bf16(w * __uint_as_float(v[8 * i + 6]), w * __uint_as_float(v[8 * i + 7])));
          }
          __syncwarp();
          const int unit = lane & 15;
          const long long col = col_base + half * 128 + unit * 8;
#pragma unroll 4
          for (int pair = 0; pair < 16; ++pair) {
            const int r = pair * 2 + (lane >> 4);
            const int tag_r = __shfl_sync(0xffffffffu, tag, r);
            const int dest_r = __shfl_sync(0xffffffffu, dest, r);
            if (tag_r >= 0 && col < p.N) {
              const uint4 data = stage[r * 16 + (unit ^ (r & 15))];
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.push_dst.ptr[dest_r]) +
                                        static_cast<long long>(tag_r) * p.ldd + col) = data;
            }
          }
          __syncwarp();
        }
      } else {
        const long long col_base = static_cast<long long>(t.n_tile) * BN;
        const long long expert_off = SCHED == SCHED_WGRAD ? t.expert * p.d_expert_stride : 0;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          if (!empty_k) {
            tmem_ld_32x32(taddr + c, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0;
          }
          const long long col = col_base + c;
          if (!row_ok || col >= p.N) continue;   // N is a multiple of 32 (checked on the host)
          const long long off = expert_off + row * p.ldd + col;
          if (EPI == EPI_ROPE) {
            if (col < p.rope_cols) {
              // 32 consecutive columns of one head: pairs (2j, 2j+1), table entries [pos][(col mod 128)/2 + j]
              const size_t tab = static_cast<size_t>(row % p.rope_seq) * 64 + ((col & 127) >> 1);
              const float4* c4 = reinterpret_cast<const float4*>(p.rope_cos + tab);
              const float4* s4 = reinterpret_cast<const float4*>(p.rope_sin + tab);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float4 cc = c4[q], ss = s4[q];
                const float cv[4] = {cc.x, cc.y, cc.z, cc.w}, sv[4] = {ss.x, ss.y, ss.z, ss.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float x0 = __uint_as_float(v[8 * q + 2 * j]), x1 = __uint_as_float(v[8 * q + 2 * j + 1]);
                  v[8 * q + 2 * j] = __float_as_uint(x0 * cv[j] - x1 * sv[j]);
                  v[8 * q + 2 * j + 1] = __float_as_uint(x0 * sv[j] + x1 * cv[j]);
                }
              }
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.d) + off);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[i] = make_uint4(pack_bf16(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])),
                                  pack_bf16(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])),
                                  pack_bf16(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])),
                                  pack_bf16(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7])));
          } else if (EPI == EPI_STORE_BF16) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.d) + off);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[i] = make_uint4(pack_bf16(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])),
                                  pack_bf16(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])),
                                  pack_bf16(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])),
                                  pack_bf16(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7])));
          } else if (EPI == EPI_ACC_F32 || EPI == EPI_STORE_F32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.d) + off);
            const bool add = EPI == EPI_ACC_F32 && p.beta != 0.f;
            float4 old[8];
            if (add) {
#pragma unroll
              for (int i = 0; i < 8; ++i) old[i] = dst[i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float4 r = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                     __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
              if (add) {
                r.x += old[i].x; r.y += old[i].y; r.z += old[i].z; r.w += old[i].w;
              }
              dst[i] = r;
            }
          } else if (EPI == EPI_ACC_BF16) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.d) + off);
            const bool add = p.beta != 0.f;
            uint4 old[4];
            if (add) {
#pragma unroll
              for (int i = 0; i < 4; ++i) old[i] = dst[i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t o[4] = {old[i].x, old[i].y, old[i].z, old[i].w};
              uint32_t r[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float a = __uint_as_float(v[8 * i + 2 * j]), b = __uint_as_float(v[8 * i + 2 * j + 1]);
                if (add) {
                  const __nv_bfloat162 prev = *reinterpret_cast<__nv_bfloat162*>(&o[j]);
                  a += __low2float(prev);
                  b += __high2float(prev);
                }
                r[j] = pack_bf16(a, b);
              }
              dst[i] = make_uint4(r[0], r[1], r[2], r[3]);
            }
          }
        }
      }
      }  // sub
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&tmem_empty[acc]), 0));
        else mbar_arrive(&tmem_empty[acc]);
      }
      if (++acc == NACC) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  if (EPI == EPI_PUSH) __threadfence_system();   // my rows are in the peers' memory before the flag below
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's shared memory, barriers and tensor memory are idle as well
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
  if (EPI == EPI_PUSH && threadIdx.x == 0) {
    // the last CTA to get here tells every rank that this rank's rows have been delivered
    const unsigned int old = atomicInc(p.push_ticket, gridDim.x - 1);
    if (old == gridDim.x - 1) {
      __threadfence_system();
      signal_all(p.push_sig, p.push_slot, p.push_rank, p.push_n, p.push_seq);
    }
  }
}

// ------------------------------------------------------------------ host side
template <int A_MN, int B_MN, int EPI, int SCHED, int MT>
static int launch_mt(const GemmParams& p, int sms, cudaStream_t stream) {
  auto kernel = gemm_tcgen05_kernel<A_MN, B_MN, EPI, SCHED, MT, 0>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<EPI, MT>()) != cudaSuccess)
      return -3;
    configured = true;
  }
  kernel<<<sms, GEMM_THREADS, smem_bytes<EPI, MT>(), stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// CTA pairs: a cluster of two CTAs per 256x256 tile, as many pairs as the device keeps resident.
// Returns -20 when clusters of two with this much shared memory cannot be scheduled.
template <int A_MN, int B_MN, int EPI, int SCHED>
static int pairs_resident(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int sms) {
  auto kernel = gemm_tcgen05_kernel<A_MN, B_MN, EPI, SCHED, 1, 1>;
  attr->id = cudaLaunchAttributeClusterDimension;
  attr->val.clusterDim.x = 2;
  attr->val.clusterDim.y = 1;
  attr->val.clusterDim.z = 1;
  cfg->blockDim = dim3(GEMM_THREADS);
  cfg->dynamicSmemBytes = smem_bytes<EPI, 1, 1>();
  cfg->attrs = attr;
  cfg->numAttrs = 1;
  static int max_pairs = -1;
  if (max_pairs < 0) {
    max_pairs = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<EPI, 1, 1>()) == cudaSuccess) {
      int clusters = 0;
      cfg->gridDim = dim3(sms / 2 * 2);
      if (cudaOccupancyMaxActiveClusters(&clusters, kernel, cfg) == cudaSuccess) max_pairs = clusters;
      else cudaGetLastError();
    }
  }
  return max_pairs;
}

template <int A_MN, int B_MN, int EPI, int SCHED>
static int launch_pair(const GemmParams& p, int sms, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr;
  const int pairs = pairs_resident<A_MN, B_MN, EPI, SCHED>(&cfg, &attr, sms);
  if (pairs < 1) return -20;
  cfg.gridDim = dim3(2 * pairs);
  cfg.stream = stream;
  if (cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<A_MN, B_MN, EPI, SCHED, 1, 1>, p) != cudaSuccess) {
    cudaGetLastError();
    return -4;
  }
  return 0;
}

static int g_tile_mode = 0;   // 0 auto (single-CTA kinds), 1 force 128x256, 2 force 256x256 on one CTA,
                              // 3 force CTA pairs where legal, 4 auto with CTA pairs for large problems

enum TileKind : int { TILE_128 = 0, TILE_256 = 1, TILE_PAIR = 2 };

// 256-row tiles (one CTA with two sub-tiles, or a CTA pair) need whole 256-row tiles of one expert: the caller says
// whether its segments are padded to 256 rows.
// Measured in isolation (burst clocks) CTA pairs are the fastest kind everywhere: 16384 x 6144 x 4096 runs at
// 1351 TFLOP/s with 128x256 tiles and 1494 on pairs, grouped weight gradients gain 13-28 %.  Inside a training
// step, which runs against the 1000 W power cap for seconds, the same kernels pull the SM clock down further
// (median 1175 MHz against 1385 MHz with the single-CTA kinds, same power) and the step gets 7 % slower (3141 ms
// against 2940 ms, measured twice, alternating).  So the automatic choice uses the single-CTA kinds — 256x256 for
// long K, where the exposed epilogue is amortised, 128x256 otherwise — and pairs are opt-in (mode 3 or 4).
template <int SCHED>
static TileKind choose_tile(const GemmParams& p, int sms, bool pair_available) {
  const long long k_eff = SCHED == SCHED_WGRAD ? p.K / (p.num_experts > 0 ? p.num_experts : 1) : p.K;
  const bool legal = SCHED == SCHED_WGRAD ||
                     (p.tile_expert == nullptr ? p.num_m_tiles == nullptr : p.group_align256 != 0);
  const long long tiles256 = static_cast<long long>((p.M + 255) / 256) * ((p.N + BN - 1) / BN) *
                             (SCHED == SCHED_WGRAD ? p.num_experts : 1);
  if (!legal || g_tile_mode == 1) return TILE_128;
  if (g_tile_mode == 2) return TILE_256;
  if (pair_available && (g_tile_mode == 3 || (g_tile_mode == 4 && tiles256 >= sms / 2))) return TILE_PAIR;
  if (g_tile_mode == 3) return TILE_128;
  return tiles256 >= 2LL * sms && k_eff >= 6144 ? TILE_256 : TILE_128;
}

template <int A_MN, int B_MN, int EPI, int SCHED>
static bool pair_available(int sms) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr;
  return pairs_resident<A_MN, B_MN, EPI, SCHED>(&cfg, &attr, sms) >= sms / 2 - 8;   // (nearly) every SM in a pair
}

template <int A_MN, int B_MN, int EPI, int SCHED>
static int launch(const GemmParams& p, TileKind kind, int sms, cudaStream_t stream) {
  if (kind == TILE_PAIR) return launch_pair<A_MN, B_MN, EPI, SCHED>(p, sms, stream);
  if (kind == TILE_256) return launch_mt<A_MN, B_MN, EPI, SCHED, 2>(p, sms, stream);
  return launch_mt<A_MN, B_MN, EPI, SCHED, 1>(p, sms, stream);
}

// Convenience for entry points whose tensor maps do not depend on the tile kind.
template <int A_MN, int B_MN, int EPI, int SCHED>
static int launch(const GemmParams& p, int sms, cudaStream_t stream) {
  return launch<A_MN, B_MN, EPI, SCHED>(p, choose_tile<SCHED>(p, sms, pair_available<A_MN, B_MN, EPI, SCHED>(sms)),
                                        sms, stream);
}

static int sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

}  // namespace b2

using namespace b2;

// Arguments shared by the entry points below:
//   a, b           bf16 operands; layouts per entry point
//   lda, ldb       row pitch in elements
//   tile_expert    optional int32 [ceil(M/128)] expert of each 128-row tile (grouped problems)
//   num_m_tiles    optional device int32 scalar with the live tile count
//   status         device int32 word, set non-zero if an in-kernel wait ran out
extern "C" {

// 0 automatic among the single-CTA kinds, 1 always 128x256 tiles, 2 single-CTA 256x256 tiles wherever they are legal,
// 3 CTA pairs wherever legal, 4 automatic with CTA pairs for problems that fill the machine.
void b2_gemm_set_tile_mode(int mode) { g_tile_mode = mode; }

// y[M,N] = a[M,K] * w[e][N,K]^T      (a K-major, w K-major)
// epi: 0 bf16 store, 4 fp32 store.
int b2_gemm_nt(const void* a, const void* w, void* d, int M, int N, int K, long long lda, long long ldw,
               long long ldd, int num_experts, const int* tile_expert, const int* num_m_tiles, int group_align256,
               int epi, int* status, cudaStream_t stream) {
  if (N % 32 || K % 8) return -10;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.num_experts = num_experts; p.b_expert_rows = N; p.k_split = 0;
  p.tile_expert = tile_expert; p.num_m_tiles = num_m_tiles; p.d = d; p.ldd = ldd; p.status = status; p.beta = 0.f;
  p.group_align256 = group_align256;
  if (epi != EPI_STORE_BF16 && epi != EPI_STORE_F32) return -13;
  const int sms = sm_count();
  const bool pairs = epi == EPI_STORE_BF16 ? pair_available<0, 0, EPI_STORE_BF16, SCHED_FLAT>(sms)
                                           : pair_available<0, 0, EPI_STORE_F32, SCHED_FLAT>(sms);
  const TileKind kind = choose_tile<SCHED_FLAT>(p, sms, pairs);
  if (make_map(&p.map_a, a, K, M, lda, BM)) return -11;
  // a CTA of a pair stages 128 of the tile's 256 weight rows
  if (make_map(&p.map_b, w, K, static_cast<long long>(num_experts) * N, ldw, kind == TILE_PAIR ? BN / 2 : BN))
    return -12;
  if (epi == EPI_STORE_BF16) return launch<0, 0, EPI_STORE_BF16, SCHED_FLAT>(p, kind, sms, stream);
  return launch<0, 0, EPI_STORE_F32, SCHED_FLAT>(p, kind, sms, stream);
}

// h[M,F] = silu(a w1[e]^T) * (a w3[e]^T); optional gate/up pre-activations [M,F].
int b2_gemm_swiglu(const void* a, const void* w1, const void* w3, void* h, void* gate, void* up, int M, int F, int K,
                   long long lda, int num_experts, const int* tile_expert, const int* num_m_tiles, int group_align256,
                   int* status, cudaStream_t stream) {
  if (F % 128 || K % 8) return -10;
  GemmParams p{};
  if (make_map(&p.map_a, a, K, M, lda, BM)) return -11;
  if (make_map(&p.map_b, w1, K, static_cast<long long>(num_experts) * F, K, 128)) return -12;
  if (make_map(&p.map_b2, w3, K, static_cast<long long>(num_experts) * F, K, 128)) return -12;
  p.M = M; p.N = 2 * F; p.K = K; p.num_experts = num_experts; p.b_expert_rows = F; p.k_split = 0;
  p.tile_expert = tile_expert; p.num_m_tiles = num_m_tiles; p.d = h; p.d_gate = gate; p.d_up = up; p.ldd = F;
  p.status = status; p.group_align256 = group_align256;
  return launch<0, 0, EPI_SWIGLU, SCHED_FLAT>(p, sm_count(), stream);
}

// dx[M,N] = a[M,K] * w[e][K,N]     (w MN-major: its rows are the reduction index).
// If w2 is given, K = k_split + K2 and rows k >= k_split come from w2 (dx = dg W1 + du W3 in one pass).
int b2_gemm_nn(const void* a, const void* w, const void* w2, void* d, int M, int N, int K, int k_split, long long lda,
               long long ldw, long long ldd, int num_experts, const int* tile_expert, const int* num_m_tiles,
               int group_align256, int* status, cudaStream_t stream) {
  if (N % 32 || K % 64 || (w2 && k_split % 64)) return -10;
  GemmParams p{};
  const int rows = w2 ? k_split : K;
  if (make_map(&p.map_a, a, K, M, lda, BM)) return -11;
  if (make_map(&p.map_b, w, N, static_cast<long long>(num_experts) * rows, ldw, 64)) return -12;
  if (w2 && make_map(&p.map_b2, w2, N, static_cast<long long>(num_experts) * (K - k_split), ldw, 64)) return -12;
  p.M = M; p.N = N; p.K = K; p.num_experts = num_experts; p.b_expert_rows = rows; p.k_split = w2 ? k_split : 0;
  p.tile_expert = tile_expert; p.num_m_tiles = num_m_tiles; p.d = d; p.ldd = ldd; p.status = status;
  p.group_align256 = group_align256;
  return launch<0, 1, EPI_STORE_BF16, SCHED_FLAT>(p, sm_count(), stream);
}

// y[M,N] = a[M,K] * w[N,K]^T with the rotary embedding applied to columns [0, rope_cols) in the epilogue: column c
// belongs to head c / 128, pairs (2j, 2j+1) inside a head are rotated by the angle of table entry
// [row mod seq][j] (cos, sin: fp32 [seq, 64]).  rope_cols is a multiple of 128.
int b2_gemm_nt_rope(const void* a, const void* w, void* d, int M, int N, int K, long long lda, long long ldd,
                    const float* cos_t, const float* sin_t, int rope_cols, int seq, int* status,
                    cudaStream_t stream) {
  if (N % 32 || K % 8 || rope_cols % 128 || rope_cols > N || seq < 1) return -10;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.num_experts = 1; p.b_expert_rows = N; p.k_split = 0;
  p.d = d; p.ldd = ldd; p.status = status; p.beta = 0.f;
  p.rope_cos = cos_t; p.rope_sin = sin_t; p.rope_cols = rope_cols; p.rope_seq = seq;
  const int sms = sm_count();
  const TileKind kind = choose_tile<SCHED_FLAT>(p, sms, pair_available<0, 0, EPI_ROPE, SCHED_FLAT>(sms));
  if (make_map(&p.map_a, a, K, M, lda, BM)) return -11;
  if (make_map(&p.map_b, w, K, N, K, kind == TILE_PAIR ? BN / 2 : BN)) return -12;
  return launch<0, 0, EPI_ROPE, SCHED_FLAT>(p, kind, sms, stream);
}

static void fill_push(GemmParams& p, const unsigned long long* dst, const int* tag, const int* src, const float* w,
                      const unsigned long long* sig, int slot, int seq, int rank, int n, unsigned int* ticket) {
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.push_dst.ptr[i] = i < n ? reinterpret_cast<void*>(dst[i]) : nullptr;
    p.push_sig.ptr[i] = i < n ? reinterpret_cast<void*>(sig[i]) : nullptr;
  }
  p.push_tag = tag; p.push_src = src; p.push_w = w; p.push_slot = slot; p.push_seq = seq; p.push_rank = rank;
  p.push_n = n; p.push_ticket = ticket;
}

// Expert-parallel return fused into the epilogue.  The product a[M,K] * w[e][N,K]^T (NT) is not stored locally: row r
// is scaled by push_w[r] (null: 1) and written as bf16 into row push_tag[r] of rank push_src[r]'s buffer
// (``push_dst``: MAX_RANKS device addresses, row pitch N); rows with a negative tag are skipped.  When all CTAs are
// done the kernel writes ``seq`` into slot ``sig_slot`` of every rank's signal pad.  ``ticket``: a zero-initialised
// device word that the kernel leaves at zero.
int b2_gemm_nt_push(const void* a, const void* w, int M, int N, int K, long long lda, int num_experts,
                    const int* tile_expert, const int* num_m_tiles, int group_align256,
                    const unsigned long long* push_dst, const int* push_tag, const int* push_src, const float* push_w,
                    const unsigned long long* sig, int sig_slot, int seq, int rank, int n, unsigned int* ticket,
                    int* status, cudaStream_t stream) {
  if (N % 32 || K % 8 || n < 1 || n > MAX_RANKS) return -10;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.num_experts = num_experts; p.b_expert_rows = N; p.k_split = 0;
  p.tile_expert = tile_expert; p.num_m_tiles = num_m_tiles; p.d = nullptr; p.ldd = N; p.status = status;
  p.group_align256 = group_align256;
  fill_push(p, push_dst, push_tag, push_src, push_w, sig, sig_slot, seq, rank, n, ticket);
  const int sms = sm_count();
  const TileKind kind = choose_tile<SCHED_FLAT>(p, sms, pair_available<0, 0, EPI_PUSH, SCHED_FLAT>(sms));
  if (make_map(&p.map_a, a, K, M, lda, BM)) return -11;
  if (make_map(&p.map_b, w, K, static_cast<long long>(num_experts) * N, K, kind == TILE_PAIR ? BN / 2 : BN))
    return -12;
  return launch<0, 0, EPI_PUSH, SCHED_FLAT>(p, kind, sms, stream);
}

// The same for a[M,K] * w[e][K,N] with the reduction continued over w2 (dx = dgate W1 + dup W3).
int b2_gemm_nn_push(const void* a, const void* w, const void* w2, int M, int N, int K, int k_split, long long lda,
                    int num_experts, const int* tile_expert, const int* num_m_tiles, int group_align256,
                    const unsigned long long* push_dst, const int* push_tag, const int* push_src, const float* push_w,
                    const unsigned long long* sig, int sig_slot, int seq, int rank, int n, unsigned int* ticket,
                    int* status, cudaStream_t stream) {
  if (N % 32 || K % 64 || (w2 && k_split % 64) || n < 1 || n > MAX_RANKS) return -10;
  GemmParams p{};
  const int rows = w2 ? k_split : K;
  if (make_map(&p.map_a, a, K, M, lda, BM)) return -11;
  if (make_map(&p.map_b, w, N, static_cast<long long>(num_experts) * rows, N, 64)) return -12;
  if (w2 && make_map(&p.map_b2, w2, N, static_cast<long long>(num_experts) * (K - k_split), N, 64)) return -12;
  p.M = M; p.N = N; p.K = K; p.num_experts = num_experts; p.b_expert_rows = rows; p.k_split = w2 ? k_split : 0;
  p.tile_expert = tile_expert; p.num_m_tiles = num_m_tiles; p.d = nullptr; p.ldd = N; p.status = status;
  p.group_align256 = group_align256;
  fill_push(p, push_dst, push_tag, push_src, push_w, sig, sig_slot, seq, rank, n, ticket);
  return launch<0, 1, EPI_PUSH, SCHED_FLAT>(p, sm_count(), stream);
}

// dw[e][M,N] (+)= a[rows_e, M]^T * b[rows_e, N]   (both MN-major; rows_e from cumulative offsets, or all R rows
// when expert_offsets is null).  out_kind: 1 fp32 (+= if beta), 2 bf16 (+= if beta).
int b2_gemm_tn(const void* a, const void* b, void* d, int M, int N, int R, long long lda, long long ldb,
               long long ldd, int num_experts, const int* expert_offsets, int out_kind, float beta, int* status,
               cudaStream_t stream) {
  if (N % 32 || M % 8) return -10;
  GemmParams p{};
  if (make_map(&p.map_a, a, M, R, lda, 64)) return -11;
  if (make_map(&p.map_b, b, N, R, ldb, 64)) return -12;
  p.M = M; p.N = N; p.K = R; p.num_experts = num_experts; p.b_expert_rows = 0; p.k_split = 0;
  p.expert_offsets = expert_offsets; p.d = d; p.ldd = ldd; p.d_expert_stride = static_cast<long long>(M) * ldd;
  p.beta = beta; p.status = status;
  if (expert_offsets) {
    if (out_kind == 1) return launch<1, 1, EPI_ACC_F32, SCHED_WGRAD>(p, sm_count(), stream);
    if (out_kind == 2) return launch<1, 1, EPI_ACC_BF16, SCHED_WGRAD>(p, sm_count(), stream);
  } else {
    if (out_kind == 1) return launch<1, 1, EPI_ACC_F32, SCHED_FLAT>(p, sm_count(), stream);
    if (out_kind == 2) return launch<1, 1, EPI_ACC_BF16, SCHED_FLAT>(p, sm_count(), stream);
  }
  return -13;
}

}  // extern "C"
