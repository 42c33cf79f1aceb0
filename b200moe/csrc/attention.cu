// Causal grouped-query flash attention for head_dim 128 on tcgen05 tensor cores:
// forward, and the backward pass as two kernels (dK/dV per key tile, dQ per query
// tile).  Inputs are bf16 views [B, S, H, 128] with a common token pitch (the fused
// QKV projection, already rotated by the RoPE kernel); Q/K/V/dO tiles come in by TMA
// (plain per-CTA tile loads) in the 128-byte-swizzled layout, so the same
// shared-memory tile serves as a K-major or an MN-major MMA operand.  Scores and
// probabilities live in tensor memory: S = Q K^T lands in TMEM, the softmax warps turn
// it into bf16 P in place, and P feeds the next MMA straight from TMEM (A operand in
// tensor memory), so P never touches shared memory.
//
// Forward, one CTA per (128 queries, head, batch), 320 threads:
//   warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 softmax / correction / epilogue
//   (two threads per query row, 64 key columns each).  Two S buffers let QK^T of tile j+1 run under the
//   softmax of tile j; O is rescaled only when a row maximum grew by more than 2^8.
// Backward kernels run 320 threads: two softmax groups split the 128 columns of a tile.
// Backward dK/dV, one CTA per (128 keys, kv head, batch): loops over the 4 query heads
//   of the group and their causal query tiles with S^T = K Q^T, dP^T = V dO^T, so P^T
//   and dS^T are A operands in TMEM; dV and dK accumulate in TMEM over the whole loop
//   (the GQA reduction needs no atomics).
// Backward dQ, one CTA per (128 queries, head, batch): recomputes S and dP per key tile
//   and accumulates dQ += dS K in TMEM.
// Every barrier wait is bounded; a wait that runs out sets the status word.
#include "ptx.cuh"
#include "tensormap.cuh"

namespace b2 {

constexpr int HD = 128;
constexpr int TQ = 128;
constexpr int TK = 128;
constexpr int TILE_BYTES = 128 * HD * 2;      // 32 KiB: two swizzle atoms of [128 rows x 64 cols]
constexpr int ATOM_BYTES = 16384;
constexpr int ATTN_THREADS = 192;
constexpr int ATTN_BWD_THREADS = 320;   // TMA warp, MMA warp, two softmax groups of four warps

struct AttnParams {
  CUtensorMap map_q, map_k, map_v, map_do;
  int B, S, Hq, Hkv;
  int causal;             // 1: keys after the query are masked; 0: every query sees every key
  float scale;            // 1/sqrt(head_dim)
  float scale_log2;       // scale * log2(e)
  __nv_bfloat16* out;     // forward: [B,S,Hq,128] contiguous
  float* lse;             // [B,Hq,S] natural-log row sums (forward writes, backward reads)
  const float* delta;     // [B,Hq,S] rowsum(dO * O) (backward)
  __nv_bfloat16* dq;      // [B,S,Hq,128]
  __nv_bfloat16* dk;      // [B,S,Hkv,128]
  __nv_bfloat16* dv;      // [B,S,Hkv,128]
  long long dq_pitch, dk_pitch, dv_pitch;   // elements per token of the gradient outputs
  const float* rope_cos;  // backward, optional: [S, 64] tables of the rotation that was applied to q and k before the
  const float* rope_sin;  // forward pass; dq and dk are then stored rotated back (gradients of the unrotated q, k)
  int* status;
};

// Transposed rotary embedding on 32 consecutive columns (16 adjacent pairs) of one head, in registers:
// (d0, d1) -> (d0 c + d1 s, d1 c - d0 s).  ``first_pair`` = (column of a[0] within the head) / 2.
__device__ __forceinline__ void unrotate32(uint32_t (&a)[32], const float* cos_t, const float* sin_t, size_t pos,
                                           int first_pair) {
  const float4* c4 = reinterpret_cast<const float4*>(cos_t + pos * 64 + first_pair);
  const float4* s4 = reinterpret_cast<const float4*>(sin_t + pos * 64 + first_pair);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float4 cc = c4[q], ss = s4[q];
    const float cv[4] = {cc.x, cc.y, cc.z, cc.w}, sv[4] = {ss.x, ss.y, ss.z, ss.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float d0 = __uint_as_float(a[8 * q + 2 * j]), d1 = __uint_as_float(a[8 * q + 2 * j + 1]);
      a[8 * q + 2 * j] = __float_as_uint(d0 * cv[j] + d1 * sv[j]);
      a[8 * q + 2 * j + 1] = __float_as_uint(d1 * cv[j] - d0 * sv[j]);
    }
  }
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// K-major operand inside a [128 x 128] tile stored as two atoms: 16-element k-step ks (0..7).
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int ks) {
  return umma_smem_desc(tile + (ks >> 2) * ATOM_BYTES + (ks & 3) * 32, 16, 1024);
}
// The same tile read as an MN-major operand: MN runs along the 128 columns (two 64-column atoms,
// ATOM_BYTES apart), K along the rows; k-step ks covers rows [16 ks, 16 ks + 16).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int ks) {
  return umma_smem_desc(tile + ks * 2048, ATOM_BYTES, 1024);
}

__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int col0, int row0) {
  tma_load_2d(dst, map, bar, col0, row0);
  tma_load_2d(dst + ATOM_BYTES, map, bar, col0 + 64, row0);
}

#define ATTN_FAIL(code)            \
  {                                \
    *abort_flag = 1;               \
    atomicExch(p.status, code);    \
  }

// ================================================================= forward
struct FwdBars {
  uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full[2], o_done, mx_ready;
};

__global__ void __launch_bounds__(ATTN_BWD_THREADS, 1) attn_fwd_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;            // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;        // 2 stages
  float* s_rowmax = reinterpret_cast<float*>(sV + 2 * TILE_BYTES);   // [2 buffers][2 halves][128] + [2][128] sums
  FwdBars* bars = reinterpret_cast<FwdBars*>(s_rowmax + 6 * TQ);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = p.S / TQ;
  const int qt = q_tiles - 1 - blockIdx.x;      // long tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int n_kv = p.causal ? qt + 1 : q_tiles;
  const int row_q = b * p.S + qt * TQ;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_empty[s], 1);
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_full[s], 8);
    }
    mbar_init(&bars->o_done, 1);
    mbar_init(&bars->mx_ready, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_o = tmem + 256;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&bars->q_full, TILE_BYTES);
      load_tile(sQ, &p.map_q, &bars->q_full, h * HD, row_q);
      for (int j = 0; j < n_kv && !*abort_flag; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        const int row_k = b * p.S + j * TK;
        if (!mbar_wait(&bars->k_empty[s], ph)) { ATTN_FAIL(201); break; }
        mbar_expect_tx(&bars->k_full[s], TILE_BYTES);
        load_tile(sK + s * TILE_BYTES, &p.map_k, &bars->k_full[s], hk * HD, row_k);
        if (!mbar_wait(&bars->v_empty[s], ph)) { ATTN_FAIL(202); break; }
        mbar_expect_tx(&bars->v_full[s], TILE_BYTES);
        load_tile(sV + s * TILE_BYTES, &p.map_v, &bars->v_full[s], hk * HD, row_k);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = mbar_wait(&bars->q_full, 0);
      if (!ok) ATTN_FAIL(203);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&bars->k_full[s], (j >> 1) & 1)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(tmem + s * 128, desc_kmajor(q_addr, ks), desc_kmajor(k_addr, ks), idesc_qk, ks != 0);
        umma_commit(&bars->k_empty[s]);
        umma_commit(&bars->s_full[s]);
        return true;
      };
      if (ok && !issue_s(0)) { ATTN_FAIL(204); ok = false; }
      if (ok && n_kv > 1 && !issue_s(1)) { ATTN_FAIL(204); ok = false; }
      for (int j = 0; j < n_kv && ok && !*abort_flag; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&bars->p_full[s], (j >> 1) & 1) || !mbar_wait(&bars->v_full[s], (j >> 1) & 1)) {
          ATTN_FAIL(205);
          break;
        }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + s * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ts(tmem_o, tmem + s * 128 + (ks >> 2) * 64 + (ks & 3) * 8, desc_mnmajor(v_addr, ks), idesc_pv,
                       (j | ks) != 0);
        umma_commit(&bars->v_empty[s]);
        umma_commit(&bars->o_done);
        if (j + 2 < n_kv && !issue_s(j + 2)) { ATTN_FAIL(204); break; }
      }
    }
  } else {
    // Two softmax groups of four warps; group ``half`` owns key columns [64 half, 64 half + 64) of every
    // score tile.  The two threads that share a query row exchange their partial row maxima through shared
    // memory (one bounded mbarrier phase per tile) and keep separate partial row sums until the end.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;                       // query row inside the tile
    const int col0 = half * 64;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    for (int j = 0; j < n_kv && !*abort_flag; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&bars->s_full[s], (j >> 1) & 1)) { ATTN_FAIL(206); break; }
      tc_fence_after();
      const uint32_t ts = tmem + s * 128 + lane_base + col0;
      uint32_t raw[2][32];
      tmem_ld_32x32(ts, raw[0]);
      tmem_ld_32x32(ts + 32, raw[1]);
      tmem_ld_wait();
      if (p.causal && j == qt) {                       // diagonal tile: keys after the query are masked
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + c * 32 + i > r) raw[c][i] = 0xff800000u;   // -inf
      }
      float mpart[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mpart[i] = -INFINITY;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mpart[i & 7] = fmaxf(mpart[i & 7], __uint_as_float(raw[c][i]));
      float mx = fmaxf(fmaxf(fmaxf(mpart[0], mpart[1]), fmaxf(mpart[2], mpart[3])),
                       fmaxf(fmaxf(mpart[4], mpart[5]), fmaxf(mpart[6], mpart[7])));
      // exchange with the thread that owns the other 64 columns of this row
      s_rowmax[(s * 2 + half) * TQ + r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->mx_ready);
      if (!mbar_wait(&bars->mx_ready, j & 1)) { ATTN_FAIL(209); break; }
      mx = fmaxf(fmaxf(mx, s_rowmax[(s * 2 + (half ^ 1)) * TQ + r]), m_ref);
      const bool need = (mx - m_ref) * p.scale_log2 > 8.f;      // also true on the first tile (m_ref = -inf)
      const bool any = __any_sync(0xffffffffu, need);
      float alpha = 1.f;
      if (any) {
        alpha = ex2((m_ref - mx) * p.scale_log2);               // 0 on the first tile
        m_ref = mx;
      }
      const float neg = -m_ref * p.scale_log2;
      float part[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // independent partial sums: no long add chain
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float x0 = fmaf(__uint_as_float(raw[c][i]), p.scale_log2, neg);
          const float x1 = fmaf(__uint_as_float(raw[c][i + 1]), p.scale_log2, neg);
          const float p0 = ex2(x0), p1 = ex2(x1);
          part[(i >> 1) & 7] += p0 + p1;
          packed[c * 16 + (i >> 1)] = pack_bf16(p0, p1);
        }
      const float sum = ((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7]));
      l = l * alpha + sum;
      // P (bf16 pairs) overwrites the first 32 of the 64 columns this thread has just read
      tmem_st_32x32(ts, packed);
      if (j > 0) {
        if (!mbar_wait(&bars->o_done, (j - 1) & 1)) { ATTN_FAIL(207); break; }
        tc_fence_after();
        if (any) {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + lane_base + col0 + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + lane_base + col0 + c * 32, o);
          }
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[s]);
    }
    // epilogue: combine the two partial row sums, normalise, store this thread's 64 output columns
    if (!*abort_flag) {
      s_rowmax[(4 + half) * TQ + r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->mx_ready);
      if (!mbar_wait(&bars->mx_ready, n_kv & 1)) ATTN_FAIL(210);
      l += s_rowmax[(4 + (half ^ 1)) * TQ + r];
      if (!mbar_wait(&bars->o_done, (n_kv - 1) & 1)) ATTN_FAIL(208);
      tc_fence_after();
      const float inv = 1.f / l;
      const size_t token = static_cast<size_t>(row_q + r);
      __nv_bfloat16* dst = p.out + (token * p.Hq + h) * HD + col0;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + lane_base + col0 + c * 32, o);
        tmem_ld_wait();
        uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          d4[i] = make_uint4(pack_bf16(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv),
                             pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv),
                             pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv),
                             pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv));
      }
      if (half == 0) p.lse[(static_cast<size_t>(b) * p.Hq + h) * p.S + qt * TQ + r] = m_ref * p.scale + logf(l);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ================================================================= backward: delta = rowsum(dO * O)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                  float* __restrict__ delta, int B, int S, int Hq) {
  // one warp per (token, head); delta layout [B, Hq, S]
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int total = B * S * Hq;
  if (warp >= total) return;
  const int h = warp % Hq;
  const int token = warp / Hq;
  const size_t base = static_cast<size_t>(warp) * HD + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(dout + base);
  const uint2 o = *reinterpret_cast<const uint2*>(out + base);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 o0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o.x));
  const float2 o1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o.y));
  float s = a0.x * o0.x + a0.y * o0.y + a1.x * o1.x + a1.y * o1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    const int b = token / S, pos = token - b * S;
    delta[(static_cast<size_t>(b) * Hq + h) * S + pos] = s;
  }
}

// ================================================================= backward: dK, dV
struct KvBars {
  uint64_t kv_full, qd_full[2], qd_empty[2], st_full, dpt_full, p_ready, ds_ready, acc_done;
};

// TMEM: S^T / P^T [0,128), dP^T / dS^T [128,256), dV [256,384), dK [384,512).
// 320 threads: warp 0 TMA, warp 1 MMA, warps 2-9 two softmax groups; group g handles query columns
// [64 g, 64 g + 64) of the 128 x 128 tile (two warps per scheduler hide each other's latency).
// MMA order per query tile: dV(it), S^T(it+1), dK(it), dP^T(it+1) - S^T of the next tile runs on the
// tensor core while the softmax warps turn dP^T into dS^T.
__global__ void __launch_bounds__(ATTN_BWD_THREADS, 1) attn_bwd_dkv_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;             // 2 stages
  uint8_t* sDO = sQ + 2 * TILE_BYTES;        // 2 stages
  KvBars* bars = reinterpret_cast<KvBars*>(sDO + 2 * TILE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = p.S / TQ;
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int q_first = p.causal ? kt : 0;           // causal: query tiles kt .. q_tiles-1
  const int per_head = q_tiles - q_first;
  const int iters = group * per_head;
  const int row_k = b * p.S + kt * TK;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->qd_full[s], 1);
      mbar_init(&bars->qd_empty[s], 1);
    }
    mbar_init(&bars->st_full, 1);
    mbar_init(&bars->dpt_full, 1);
    mbar_init(&bars->p_ready, 8);
    mbar_init(&bars->ds_ready, 8);
    mbar_init(&bars->acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_st = tmem, t_dpt = tmem + 128, t_dv = tmem + 256, t_dk = tmem + 384;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&bars->kv_full, 2 * TILE_BYTES);
      load_tile(sK, &p.map_k, &bars->kv_full, hk * HD, row_k);
      load_tile(sV, &p.map_v, &bars->kv_full, hk * HD, row_k);
      for (int it = 0; it < iters && !*abort_flag; ++it) {
        const int s = it & 1;
        const int hq = hk * group + it / per_head;
        const int qi = q_first + it % per_head;
        const int row_q = b * p.S + qi * TQ;
        if (!mbar_wait(&bars->qd_empty[s], ((it >> 1) & 1) ^ 1)) { ATTN_FAIL(211); break; }
        mbar_expect_tx(&bars->qd_full[s], 2 * TILE_BYTES);
        load_tile(sQ + s * TILE_BYTES, &p.map_q, &bars->qd_full[s], hq * HD, row_q);
        load_tile(sDO + s * TILE_BYTES, &p.map_do, &bars->qd_full[s], hq * HD, row_q);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 128, 0, 0);   // both operands K-major
      constexpr uint32_t idesc_tn = umma_idesc_bf16(128, 128, 0, 1);   // A from TMEM, B MN-major
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      auto issue_st = [&](int it) {          // S^T[key, q] = K Q^T
        const uint32_t q_addr = smem_u32(sQ + (it & 1) * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(t_st, desc_kmajor(k_addr, ks), desc_kmajor(q_addr, ks), idesc_kk, ks != 0);
        umma_commit(&bars->st_full);
      };
      auto issue_dpt = [&](int it) {         // dP^T[key, q] = V dO^T
        const uint32_t do_addr = smem_u32(sDO + (it & 1) * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(t_dpt, desc_kmajor(v_addr, ks), desc_kmajor(do_addr, ks), idesc_kk, ks != 0);
        umma_commit(&bars->dpt_full);
      };
      bool ok = mbar_wait(&bars->kv_full, 0) && mbar_wait(&bars->qd_full[0], 0);
      if (!ok) ATTN_FAIL(212);
      if (ok) {
        tc_fence_after();
        issue_st(0);
        issue_dpt(0);
      }
      for (int it = 0; it < iters && ok && !*abort_flag; ++it) {
        const int s = it & 1;
        const uint32_t ph = it & 1;
        const uint32_t q_addr = smem_u32(sQ + s * TILE_BYTES), do_addr = smem_u32(sDO + s * TILE_BYTES);
        if (!mbar_wait(&bars->p_ready, ph)) { ATTN_FAIL(214); break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)      // dV[key, d] += P^T[key, q] dO[q, d]
          umma_bf16_ts(t_dv, t_st + (ks >> 2) * 64 + (ks & 3) * 8, desc_mnmajor(do_addr, ks), idesc_tn, (it | ks) != 0);
        const bool more = it + 1 < iters;
        if (more) {
          if (!mbar_wait(&bars->qd_full[(it + 1) & 1], ((it + 1) >> 1) & 1)) { ATTN_FAIL(213); break; }
          tc_fence_after();
          issue_st(it + 1);                 // overwrites P^T only after dV above (same-thread issue order)
        }
        if (!mbar_wait(&bars->ds_ready, ph)) { ATTN_FAIL(215); break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)      // dK[key, d] += dS^T[key, q] Q[q, d]
          umma_bf16_ts(t_dk, t_dpt + (ks >> 2) * 64 + (ks & 3) * 8, desc_mnmajor(q_addr, ks), idesc_tn, (it | ks) != 0);
        umma_commit(&bars->qd_empty[s]);
        umma_commit(&bars->acc_done);
        if (more) issue_dpt(it + 1);        // overwrites dS^T only after dK above
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;                      // which 64 query columns this thread handles
    const int r = quad * 32 + lane;                        // key row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int col0 = half * 64;
    for (int it = 0; it < iters && !*abort_flag; ++it) {
      const int hq = hk * group + it / per_head;
      const int qi = q_first + it % per_head;
      const uint32_t ph = it & 1;
      const size_t stat = (static_cast<size_t>(b) * p.Hq + hq) * p.S + qi * TQ + col0;
      // statistics of my 64 query columns: lane i keeps those of columns 32c + i and the warp shuffles them
      float lse_reg[2], dl_reg[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        lse_reg[c] = p.lse[stat + c * 32 + lane] * 1.4426950408889634f;
        dl_reg[c] = p.delta[stat + c * 32 + lane];
      }
      if (!mbar_wait(&bars->st_full, ph)) { ATTN_FAIL(216); break; }
      tc_fence_after();
      const bool diag = p.causal && qi == kt;
      uint32_t pk[32];
      float pf[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(t_st + lane_base + col0 + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float lq = __shfl_sync(0xffffffffu, lse_reg[c], i);
          pf[c * 32 + i] = ex2(fmaf(__uint_as_float(raw[i]), p.scale_log2, -lq));
        }
      }
      if (diag) {                                           // key after query
#pragma unroll
        for (int q = 0; q < 64; ++q)
          if (r > col0 + q) pf[q] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 64; i += 2) pk[i >> 1] = pack_bf16(pf[i], pf[i + 1]);
      // P^T as bf16 pairs, written over the columns this thread has just read: queries 0-63 land in columns
      // [0,32), queries 64-127 in [64,96)
      tmem_st_32x32(t_st + lane_base + col0, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_ready);
      if (!mbar_wait(&bars->dpt_full, ph)) { ATTN_FAIL(217); break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(t_dpt + lane_base + col0 + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int q = c * 32 + i;
          const float dq0 = __shfl_sync(0xffffffffu, dl_reg[c], i), dq1 = __shfl_sync(0xffffffffu, dl_reg[c], i + 1);
          const float d0 = pf[q] * (__uint_as_float(raw[i]) - dq0) * p.scale;
          const float d1 = pf[q + 1] * (__uint_as_float(raw[i + 1]) - dq1) * p.scale;
          pk[q >> 1] = pack_bf16(d0, d1);
        }
      }
      tmem_st_32x32(t_dpt + lane_base + col0, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_ready);
    }
    if (!*abort_flag && half == 0) {
      if (!mbar_wait(&bars->acc_done, (iters - 1) & 1)) ATTN_FAIL(218);
      tc_fence_after();
      const size_t token = static_cast<size_t>(row_k + r);
      __nv_bfloat16* dvp = p.dv + token * p.dv_pitch + hk * HD;
      __nv_bfloat16* dkp = p.dk + token * p.dk_pitch + hk * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t a[32], k2[32];
        tmem_ld_32x32(t_dv + lane_base + c * 32, a);
        tmem_ld_32x32(t_dk + lane_base + c * 32, k2);
        tmem_ld_wait();
        if (p.rope_cos) unrotate32(k2, p.rope_cos, p.rope_sin, token % static_cast<size_t>(p.S), c * 16);
        uint4* d4 = reinterpret_cast<uint4*>(dvp + c * 32);
        uint4* k4 = reinterpret_cast<uint4*>(dkp + c * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          d4[i] = make_uint4(pack_bf16(__uint_as_float(a[8 * i]), __uint_as_float(a[8 * i + 1])),
                             pack_bf16(__uint_as_float(a[8 * i + 2]), __uint_as_float(a[8 * i + 3])),
                             pack_bf16(__uint_as_float(a[8 * i + 4]), __uint_as_float(a[8 * i + 5])),
                             pack_bf16(__uint_as_float(a[8 * i + 6]), __uint_as_float(a[8 * i + 7])));
          k4[i] = make_uint4(pack_bf16(__uint_as_float(k2[8 * i]), __uint_as_float(k2[8 * i + 1])),
                             pack_bf16(__uint_as_float(k2[8 * i + 2]), __uint_as_float(k2[8 * i + 3])),
                             pack_bf16(__uint_as_float(k2[8 * i + 4]), __uint_as_float(k2[8 * i + 5])),
                             pack_bf16(__uint_as_float(k2[8 * i + 6]), __uint_as_float(k2[8 * i + 7])));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ================================================================= backward: dQ
struct DqBars {
  uint64_t qd_full, kv_full[2], kv_empty[2], s_full, s_taken, dp_full, ds_ready, acc_done;
};

// TMEM: S [0,128), dP / dS [128,256), dQ [256,384).  320 threads like the dK/dV kernel: softmax group g
// handles key columns [64 g, 64 g + 64).  P stays in registers, so S of the next key tile is issued as soon
// as both groups have read S (s_taken) and runs under the dS computation.
__global__ void __launch_bounds__(ATTN_BWD_THREADS, 1) attn_bwd_dq_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + TILE_BYTES;
  uint8_t* sK = sDO + TILE_BYTES;            // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;         // 2 stages
  DqBars* bars = reinterpret_cast<DqBars*>(sV + 2 * TILE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tiles = p.S / TQ;
  const int qt = q_tiles - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int n_kv = p.causal ? qt + 1 : q_tiles;
  const int row_q = b * p.S + qt * TQ;

  if (threadIdx.x == 0) {
    mbar_init(&bars->qd_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->s_taken, 8);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->ds_ready, 8);
    mbar_init(&bars->acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_s = tmem, t_dp = tmem + 128, t_dq = tmem + 256;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(&bars->qd_full, 2 * TILE_BYTES);
      load_tile(sQ, &p.map_q, &bars->qd_full, h * HD, row_q);
      load_tile(sDO, &p.map_do, &bars->qd_full, h * HD, row_q);
      for (int j = 0; j < n_kv && !*abort_flag; ++j) {
        const int s = j & 1;
        const int row_k = b * p.S + j * TK;
        if (!mbar_wait(&bars->kv_empty[s], ((j >> 1) & 1) ^ 1)) { ATTN_FAIL(221); break; }
        mbar_expect_tx(&bars->kv_full[s], 2 * TILE_BYTES);
        load_tile(sK + s * TILE_BYTES, &p.map_k, &bars->kv_full[s], hk * HD, row_k);
        load_tile(sV + s * TILE_BYTES, &p.map_v, &bars->kv_full[s], hk * HD, row_k);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_kk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_tn = umma_idesc_bf16(128, 128, 0, 1);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO);
      auto issue_s = [&](int j) {           // S[q, key] = Q K^T
        const uint32_t k_addr = smem_u32(sK + (j & 1) * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(t_s, desc_kmajor(q_addr, ks), desc_kmajor(k_addr, ks), idesc_kk, ks != 0);
        umma_commit(&bars->s_full);
      };
      auto issue_dp = [&](int j) {          // dP[q, key] = dO V^T
        const uint32_t v_addr = smem_u32(sV + (j & 1) * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_bf16_ss(t_dp, desc_kmajor(do_addr, ks), desc_kmajor(v_addr, ks), idesc_kk, ks != 0);
        umma_commit(&bars->dp_full);
      };
      bool ok = mbar_wait(&bars->qd_full, 0) && mbar_wait(&bars->kv_full[0], 0);
      if (!ok) ATTN_FAIL(222);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      for (int j = 0; j < n_kv && ok && !*abort_flag; ++j) {
        const int s = j & 1;
        const uint32_t ph = j & 1;
        const bool more = j + 1 < n_kv;
        if (more) {
          if (!mbar_wait(&bars->kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1) || !mbar_wait(&bars->s_taken, ph)) {
            ATTN_FAIL(223);
            break;
          }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(&bars->ds_ready, ph)) { ATTN_FAIL(224); break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + s * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)      // dQ[q, d] += dS[q, key] K[key, d]
          umma_bf16_ts(t_dq, t_dp + (ks >> 2) * 64 + (ks & 3) * 8, desc_mnmajor(k_addr, ks), idesc_tn, (j | ks) != 0);
        umma_commit(&bars->kv_empty[s]);
        umma_commit(&bars->acc_done);
        if (more) issue_dp(j + 1);          // overwrites dS only after dQ above
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;                        // query row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int col0 = half * 64;
    const size_t stat = (static_cast<size_t>(b) * p.Hq + h) * p.S + qt * TQ + r;
    const float lse2 = p.lse[stat] * 1.4426950408889634f;
    const float dl = p.delta[stat];
    for (int j = 0; j < n_kv && !*abort_flag; ++j) {
      const uint32_t ph = j & 1;
      if (!mbar_wait(&bars->s_full, ph)) { ATTN_FAIL(225); break; }
      tc_fence_after();
      float pf[64];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(t_s + lane_base + col0 + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) pf[c * 32 + i] = ex2(fmaf(__uint_as_float(raw[i]), p.scale_log2, -lse2));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_taken);
      if (p.causal && j == qt) {                                        // diagonal tile: keys after the query
#pragma unroll
        for (int k = 0; k < 64; ++k)
          if (col0 + k > r) pf[k] = 0.f;
      }
      if (!mbar_wait(&bars->dp_full, ph)) { ATTN_FAIL(226); break; }
      tc_fence_after();
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(t_dp + lane_base + col0 + c * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const int k = c * 32 + i;
          const float d0 = pf[k] * (__uint_as_float(raw[i]) - dl) * p.scale;
          const float d1 = pf[k + 1] * (__uint_as_float(raw[i + 1]) - dl) * p.scale;
          pk[k >> 1] = pack_bf16(d0, d1);
        }
      }
      tmem_st_32x32(t_dp + lane_base + col0, pk);          // dS pairs over the columns just read
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_ready);
    }
    if (!*abort_flag && half == 0) {
      if (!mbar_wait(&bars->acc_done, (n_kv - 1) & 1)) ATTN_FAIL(227);
      tc_fence_after();
      const size_t token = static_cast<size_t>(row_q + r);
      __nv_bfloat16* dst = p.dq + token * p.dq_pitch + h * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t a[32];
        tmem_ld_32x32(t_dq + lane_base + c * 32, a);
        tmem_ld_wait();
        if (p.rope_cos) unrotate32(a, p.rope_cos, p.rope_sin, token % static_cast<size_t>(p.S), c * 16);
        uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          d4[i] = make_uint4(pack_bf16(__uint_as_float(a[8 * i]), __uint_as_float(a[8 * i + 1])),
                             pack_bf16(__uint_as_float(a[8 * i + 2]), __uint_as_float(a[8 * i + 3])),
                             pack_bf16(__uint_as_float(a[8 * i + 4]), __uint_as_float(a[8 * i + 5])),
                             pack_bf16(__uint_as_float(a[8 * i + 6]), __uint_as_float(a[8 * i + 7])));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ================================================================= host
// [tokens, heads*128] bf16 with token pitch ``pitch`` elements; box = [128 tokens, 64 columns].
static int g_last_encode_result = 0;     // CUresult of the last tensor-map encode that failed (diagnostics)

static int attn_map(CUtensorMap* map, const void* base, long long tokens, int heads, long long pitch) {
  EncodeTiledFn fn = encode_fn();      // binds this thread's context first (tensormap.cuh)
  if (!fn) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(heads) * HD, static_cast<cuuint64_t>(tokens)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch) * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) g_last_encode_result = static_cast<int>(rc);
  return rc == CUDA_SUCCESS ? 0 : -2;
}

constexpr int FWD_SMEM = 5 * TILE_BYTES + 1024 + 6 * TQ * 4 + 512;
constexpr int BWD_SMEM = 6 * TILE_BYTES + 1024 + 512;

}  // namespace b2

using namespace b2;

extern "C" {

// After an entry point returned -11 (a tensor map could not be encoded): the driver's result code of that encode.
int b2_attention_last_encode_result() { return g_last_encode_result; }

// q: [B,S,Hq,128], k, v: [B,S,Hkv,128] bf16 with token pitches (elements); out [B,S,Hq,128] contiguous; lse [B,Hq,S].
int b2_attention_fwd_ex(const void* q, const void* k, const void* v, long long q_pitch, long long k_pitch,
                        long long v_pitch, void* out, float* lse, int B, int S, int Hq, int Hkv, float scale,
                        int causal, int* status, cudaStream_t stream) {
  if (S % 128 || Hq % Hkv || q_pitch % 8 || k_pitch % 8 || v_pitch % 8) return -10;
  AttnParams p{};
  const long long tokens = static_cast<long long>(B) * S;
  if (attn_map(&p.map_q, q, tokens, Hq, q_pitch) || attn_map(&p.map_k, k, tokens, Hkv, k_pitch) ||
      attn_map(&p.map_v, v, tokens, Hkv, v_pitch))
    return -11;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal != 0;
  p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse; p.status = status;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess)
      return -3;
    set = true;
  }
  attn_fwd_kernel<<<dim3(S / TQ, Hq, B), ATTN_BWD_THREADS, FWD_SMEM, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Causal form (the one the model uses).
int b2_attention_fwd(const void* q, const void* k, const void* v, long long q_pitch, long long k_pitch,
                     long long v_pitch, void* out, float* lse, int B, int S, int Hq, int Hkv, float scale, int* status,
                     cudaStream_t stream) {
  return b2_attention_fwd_ex(q, k, v, q_pitch, k_pitch, v_pitch, out, lse, B, S, Hq, Hkv, scale, 1, status, stream);
}

int b2_attention_bwd_rope(const void* dout, const void* q, const void* k, const void* v, const void* out,
                          const float* lse, long long q_pitch, long long k_pitch, long long v_pitch, float* delta,
                          void* dq, void* dk, void* dv, long long dq_pitch, long long dk_pitch, long long dv_pitch,
                          int B, int S, int Hq, int Hkv, float scale, int causal, const float* rope_cos,
                          const float* rope_sin, int* status, cudaStream_t stream);

// dout, out: [B,S,Hq,128] contiguous; delta: fp32 [B,Hq,S] scratch; dq [B,S,Hq,128], dk, dv [B,S,Hkv,128] with
// token pitches dq_pitch, dk_pitch, dv_pitch (they may be views into one fused gradient buffer).
int b2_attention_bwd_ex(const void* dout, const void* q, const void* k, const void* v, const void* out,
                        const float* lse, long long q_pitch, long long k_pitch, long long v_pitch, float* delta,
                        void* dq, void* dk, void* dv, long long dq_pitch, long long dk_pitch, long long dv_pitch,
                        int B, int S, int Hq, int Hkv, float scale, int causal, int* status, cudaStream_t stream) {
  return b2_attention_bwd_rope(dout, q, k, v, out, lse, q_pitch, k_pitch, v_pitch, delta, dq, dk, dv, dq_pitch,
                               dk_pitch, dv_pitch, B, S, Hq, Hkv, scale, causal, nullptr, nullptr, status, stream);
}

// The same with optional rotary tables (fp32 [S, 64]): q and k are the ROTATED tensors the forward pass saw, and dq,
// dk are stored rotated back, i.e. as gradients of the unrotated projections.
int b2_attention_bwd_rope(const void* dout, const void* q, const void* k, const void* v, const void* out,
                          const float* lse, long long q_pitch, long long k_pitch, long long v_pitch, float* delta,
                          void* dq, void* dk, void* dv, long long dq_pitch, long long dk_pitch, long long dv_pitch,
                          int B, int S, int Hq, int Hkv, float scale, int causal, const float* rope_cos,
                          const float* rope_sin, int* status, cudaStream_t stream) {
  if (S % 128 || Hq % Hkv) return -10;
  AttnParams p{};
  const long long tokens = static_cast<long long>(B) * S;
  // -11 / -12 / -13 / -14: the tensor map of q / k / v / dout could not be encoded (base not 16-byte aligned, pitch
  // not a multiple of 8 elements, ...); b2_attention_last_encode_result() has the driver's code
  if (q_pitch % 8 || k_pitch % 8 || v_pitch % 8) return -10;
  if (attn_map(&p.map_q, q, tokens, Hq, q_pitch)) return -11;
  if (attn_map(&p.map_k, k, tokens, Hkv, k_pitch)) return -12;
  if (attn_map(&p.map_v, v, tokens, Hkv, v_pitch)) return -13;
  if (attn_map(&p.map_do, dout, tokens, Hq, static_cast<long long>(Hq) * HD)) return -14;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal != 0;
  p.lse = const_cast<float*>(lse); p.delta = delta; p.dq = static_cast<__nv_bfloat16*>(dq);
  p.dk = static_cast<__nv_bfloat16*>(dk); p.dv = static_cast<__nv_bfloat16*>(dv); p.status = status;
  p.dq_pitch = dq_pitch; p.dk_pitch = dk_pitch; p.dv_pitch = dv_pitch;
  p.rope_cos = rope_cos; p.rope_sin = rope_sin;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM) != cudaSuccess)
      return -3;
    set = true;
  }
  const long long warps = tokens * Hq;
  attn_delta_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(out), delta, B, S, Hq);
  attn_bwd_dkv_kernel<<<dim3(S / TK, Hkv, B), ATTN_BWD_THREADS, BWD_SMEM, stream>>>(p);
  attn_bwd_dq_kernel<<<dim3(S / TQ, Hq, B), ATTN_BWD_THREADS, BWD_SMEM, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int b2_attention_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse,
                     long long q_pitch, long long k_pitch, long long v_pitch, float* delta, void* dq, void* dk,
                     void* dv, long long dq_pitch, long long dk_pitch, long long dv_pitch, int B, int S, int Hq,
                     int Hkv, float scale, int* status, cudaStream_t stream) {
  return b2_attention_bwd_ex(dout, q, k, v, out, lse, q_pitch, k_pitch, v_pitch, delta, dq, dk, dv, dq_pitch, dk_pitch,
                             dv_pitch, B, S, Hq, Hkv, scale, 1, status, stream);
}

}  // extern "C"
