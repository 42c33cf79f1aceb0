// Expert-routing kernels for one GPU's share of the MoE block: the dispatch plan
// (a stable counting sort of the (token, j) slots by expert, computed by one CTA
// with no host round trip), the row gather into the padded expert-major layout,
// the weighted combine and their backward duals.
//
// Layout contract.  Slots are numbered s = 2*token + j.  Expert e owns rows
// [seg_start[e], seg_start[e] + count[e]) of the permuted buffer, in slot order;
// every segment is padded with zero rows to a multiple of 256 so a GEMM tile
// never straddles two experts.  ``slot_row[s]`` is the row of slot s,
// ``row_slot[r]`` the slot of row r (-1 for padding), ``offs[e]`` the padded
// cumulative segment ends, ``tile_expert[i]`` the expert of 128-row tile i and
// ``meta = {live tiles, live rows}``.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "debug.cuh"

namespace b2 {

constexpr int PLAN_THREADS = 1024;
constexpr int ALIGN_ROWS = 256;   // segment padding; tile tables are per 128-row unit
constexpr int TILE_ROWS = 128;

__global__ void __launch_bounds__(PLAN_THREADS) moe_plan_kernel(const long long* __restrict__ idx, int slots, int E,
                                                                int* __restrict__ slot_row, int* __restrict__ row_slot,
                                                                int* __restrict__ offs, int* __restrict__ tile_expert,
                                                                int* __restrict__ meta, int* __restrict__ counts_out,
                                                                int capacity_rows) {
  extern __shared__ uint8_t plan_smem[];
  uint32_t* local = reinterpret_cast<uint32_t*>(plan_smem);               // [E][PLAN_THREADS] exclusive prefix
  int* warp_tot = reinterpret_cast<int*>(local + static_cast<size_t>(E) * PLAN_THREADS);  // [32]
  int* seg_start = warp_tot + 32;                                         // [E]
  int* seg_count = seg_start + E;                                         // [E]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (slots + PLAN_THREADS - 1) / PLAN_THREADS;
  const int s0 = min(slots, tid * per), s1 = min(slots, s0 + per);

  for (int e = 0; e < E; ++e) local[e * PLAN_THREADS + tid] = 0;
  for (int s = s0; s < s1; ++s) local[min(max(static_cast<int>(idx[s]), 0), E - 1) * PLAN_THREADS + tid] += 1;
  __syncthreads();
  // exclusive scan over threads for each expert
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
      if (lane == 31) seg_count[e] = winc;
    }
    __syncthreads();
    local[e * PLAN_THREADS + tid] = static_cast<uint32_t>(inc - mine + warp_tot[warp]);
    __syncthreads();
  }
  if (tid == 0) {
    int row = 0, tile = 0;
    for (int e = 0; e < E; ++e) {
      seg_start[e] = row;
      const int padded = (seg_count[e] + ALIGN_ROWS - 1) / ALIGN_ROWS * ALIGN_ROWS;
      for (int t = 0; t < padded / TILE_ROWS; ++t) tile_expert[tile++] = e;
      row += padded;
      offs[e] = row;
      if (counts_out) counts_out[e] = seg_count[e];
    }
    meta[0] = tile;
    meta[1] = row;
    meta[2] = row > capacity_rows ? 1 : 0;   // overflow flag (cannot happen with capacity = slots + E*127)
  }
  __syncthreads();
  const int live_rows = meta[1];
  for (int r = tid; r < min(live_rows, capacity_rows); r += PLAN_THREADS) row_slot[r] = -1;
  __syncthreads();
  for (int s = s0; s < s1; ++s) {
    const int e = min(max(static_cast<int>(idx[s]), 0), E - 1);
    const int pos = local[e * PLAN_THREADS + tid];
    local[e * PLAN_THREADS + tid] = static_cast<uint32_t>(pos + 1);
    const int row = seg_start[e] + pos;
    slot_row[s] = row;
    if (row < capacity_rows) row_slot[row] = s;
  }
}

struct alignas(16) vec16 {
  uint32_t v[4];
};

// x_perm[r] = scale(slot) * x[slot / 2] for live rows, zeros for padding; one warp per row.
// ``scale`` is null (dispatch) or the per-slot routing weight (backward of combine).
// With ``y_perm``/``dweights`` the kernel also emits dweights[slot] = <x[token], y_perm[r]>.
__global__ void __launch_bounds__(256) moe_gather_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const int* __restrict__ row_slot,
                                                         const int* __restrict__ meta,
                                                         const float* __restrict__ scale,
                                                         const __nv_bfloat16* __restrict__ y_perm,
                                                         float* __restrict__ dweights,
                                                         __nv_bfloat16* __restrict__ x_perm, int D, int capacity_rows,
                                                         int slots) {
  const int live_rows = min(meta[1], capacity_rows);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = blockIdx.x * 8 + warp; r < live_rows; r += gridDim.x * 8) {
    const int slot = row_slot[r];
    __nv_bfloat16* dst = x_perm + static_cast<size_t>(r) * D;
    if (slot < 0) {
      for (int c = lane * 8; c < D; c += 256) *reinterpret_cast<vec16*>(dst + c) = vec16{{0, 0, 0, 0}};
      continue;
    }
    if (!dbg_in_range(slot, 0, slots, 411)) continue;
    const __nv_bfloat16* src = x + static_cast<size_t>(slot >> 1) * D;
    if (!scale) {
      for (int c = lane * 8; c < D; c += 256) *reinterpret_cast<vec16*>(dst + c) = *reinterpret_cast<const vec16*>(src + c);
      continue;
    }
    const float w = scale[slot];
    float dot = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      const vec16 in = *reinterpret_cast<const vec16*>(src + c);
      vec16 yv{{0, 0, 0, 0}};
      if (y_perm) yv = *reinterpret_cast<const vec16*>(y_perm + static_cast<size_t>(r) * D + c);
      vec16 out;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in.v[i]));
        const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&yv.v[i]));
        dot += f.x * g.x + f.y * g.y;
        const __nv_bfloat162 o = __floats2bfloat162_rn(f.x * w, f.y * w);
        out.v[i] = *reinterpret_cast<const uint32_t*>(&o);
      }
      *reinterpret_cast<vec16*>(dst + c) = out;
    }
    if (dweights) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (lane == 0) dweights[slot] = dot;
    }
  }
}

// out[t] = (residual[t] +) w0 * y[slot_row[2t]] + w1 * y[slot_row[2t+1]]   (weights null => 1); one warp per token.
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y_perm,
                                                          const int* __restrict__ slot_row,
                                                          const float* __restrict__ weights,
                                                          const __nv_bfloat16* __restrict__ residual,
                                                          __nv_bfloat16* __restrict__ out, int T, int D, int rows) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    const int r0 = slot_row[2 * t], r1 = slot_row[2 * t + 1];
    if (!dbg_in_range(r0, 0, rows, 412) || !dbg_in_range(r1, 0, rows, 412)) continue;
    const float w0 = weights ? weights[2 * t] : 1.f, w1 = weights ? weights[2 * t + 1] : 1.f;
    const __nv_bfloat16* a = y_perm + static_cast<size_t>(r0) * D;
    const __nv_bfloat16* b = y_perm + static_cast<size_t>(r1) * D;
    for (int c = lane * 8; c < D; c += 256) {
      const vec16 va = *reinterpret_cast<const vec16*>(a + c);
      const vec16 vb = *reinterpret_cast<const vec16*>(b + c);
      vec16 vr{{0, 0, 0, 0}};
      if (residual) vr = *reinterpret_cast<const vec16*>(residual + static_cast<size_t>(t) * D + c);
      vec16 o;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&va.v[i]));
        const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vb.v[i]));
        const float2 fr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr.v[i]));
        const __nv_bfloat162 r = __floats2bfloat162_rn(fr.x + w0 * fa.x + w1 * fb.x, fr.y + w0 * fa.y + w1 * fb.y);
        o.v[i] = *reinterpret_cast<const uint32_t*>(&r);
      }
      *reinterpret_cast<vec16*>(out + static_cast<size_t>(t) * D + c) = o;
    }
  }
}

}  // namespace b2

using namespace b2;
typedef __nv_bfloat16 bf16;

static int sm_count_moe() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

extern "C" {

// idx: int64 [slots] expert of each slot.  Outputs int32: slot_row [slots], row_slot [capacity_rows],
// offs [E], tile_expert [capacity_rows/128], meta [4], counts (optional) [E].
int b2_moe_plan(const long long* idx, int slots, int E, int* slot_row, int* row_slot, int* offs, int* tile_expert,
                int* meta, int* counts, int capacity_rows, cudaStream_t s) {
  if (E < 1) return -10;
  const size_t smem = static_cast<size_t>(E) * PLAN_THREADS * 4 + 32 * 4 + 2 * E * 4;
  if (smem > 200 * 1024) return -11;
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    set = true;
  }
  moe_plan_kernel<<<1, PLAN_THREADS, smem, s>>>(idx, slots, E, slot_row, row_slot, offs, tile_expert, meta, counts,
                                               capacity_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int b2_moe_gather(const void* x, const int* row_slot, const int* meta, const float* scale, const void* y_perm,
                  float* dweights, void* x_perm, int D, int capacity_rows, int slots, cudaStream_t s) {
  if (D % 8) return -10;
  moe_gather_kernel<<<sm_count_moe() * 8, 256, 0, s>>>((const bf16*)x, row_slot, meta, scale, (const bf16*)y_perm, dweights,
                                            (bf16*)x_perm, D, capacity_rows, slots);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int b2_moe_combine(const void* y_perm, const int* slot_row, const float* weights, const void* residual, void* out,
                   int T, int D, int rows, cudaStream_t s) {
  if (D % 8) return -10;
  moe_combine_kernel<<<min((T + 7) / 8, sm_count_moe() * 8), 256, 0, s>>>((const bf16*)y_perm, slot_row, weights,
                                                               (const bf16*)residual, (bf16*)out, T, D, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"

B2_DEFINE_DEBUG_READER(b2_moe_debug_read)
