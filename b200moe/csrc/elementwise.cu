// Memory-bound kernels of the training step: RMSNorm (with fused residual add),
// router (skinny GEMV, softmax/top-2 and their backward), SwiGLU backward,
// cross-entropy (in-place gradient), AdamW, embedding, RoPE.
// bf16 activations move as 16-byte vectors; all arithmetic is fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) total += scratch[i];
  return total;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* scratch) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = -INFINITY;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) total = fmaxf(total, scratch[i]);
  return total;
}

// ------------------------------------------------------------------ RMSNorm
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_CHUNKS = 4;  // D <= 256 * 8 * 4 = 8192

// y = (x [+ delta]) * rstd * w ; optionally writes the sum.  One CTA per row (grid-stride); CH = 8-element
// vectors per thread (compile time, so the row stays in registers as packed bf16).
template <int CH>
__global__ void __launch_bounds__(NORM_THREADS) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  const __nv_bfloat16* __restrict__ delta,
                                                                  const float* __restrict__ w,
                                                                  __nv_bfloat16* __restrict__ sum_out,
                                                                  __nv_bfloat16* __restrict__ y,
                                                                  float* __restrict__ rstd, int rows, int D, float eps) {
  __shared__ float scratch[NORM_THREADS / 32];
  float wv[CH][8];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int col = (c * NORM_THREADS + threadIdx.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) wv[c][i] = col < D ? w[col + i] : 0.f;
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * D;
    bf16x8 raw[CH];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int col = (c * NORM_THREADS + threadIdx.x) * 8;
      if (col < D) {
        raw[c] = *reinterpret_cast<const bf16x8*>(x + base + col);
        float v[8];
        unpack8(raw[c], v);
        if (delta) {
          float d[8];
          unpack8(*reinterpret_cast<const bf16x8*>(delta + base + col), d);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += d[i];
          // the sum is rounded to bf16 once; the norm sees the rounded value, like the unfused path
          raw[c] = pack8(v);
          *reinterpret_cast<bf16x8*>(sum_out + base + col) = raw[c];
          unpack8(raw[c], v);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
      }
    }
    const float total = block_sum<NORM_THREADS>(ss, scratch);
    const float r = rsqrtf(total / D + eps);
    if (threadIdx.x == 0) rstd[row] = r;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int col = (c * NORM_THREADS + threadIdx.x) * 8;
      if (col < D) {
        float v[8], o[8];
        unpack8(raw[c], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = v[i] * r * wv[c][i];
        *reinterpret_cast<bf16x8*>(y + base + col) = pack8(o);
      }
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) [+ residual]; dw partial per CTA.
// One CTA per row (grid-stride).  The loads of the CTA's next row are issued before the current row is reduced and
// stored, so each thread keeps two rows' worth of 16-byte loads in flight across the block-wide reduction.
template <int CH>
struct NormRow {
  bf16x8 dy[CH], x[CH];
  float r;
};

template <int CH>
__device__ __forceinline__ void norm_row_load(NormRow<CH>& row, const __nv_bfloat16* __restrict__ dy,
                                              const __nv_bfloat16* __restrict__ x, const float* __restrict__ rstd,
                                              int index, int D) {
  const size_t base = static_cast<size_t>(index) * D;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int col = (c * NORM_THREADS + threadIdx.x) * 8;
    if (col < D) {
      row.dy[c] = *reinterpret_cast<const bf16x8*>(dy + base + col);
      row.x[c] = *reinterpret_cast<const bf16x8*>(x + base + col);
    }
  }
  row.r = rstd[index];
}

template <int CH>
__device__ __forceinline__ void norm_row_finish(const NormRow<CH>& row, float (&dw_acc)[CH][8],
                                                const float (&wv)[CH][8],
                                                const __nv_bfloat16* __restrict__ residual,
                                                __nv_bfloat16* __restrict__ dx, int index, int D, float* scratch) {
  const size_t base = static_cast<size_t>(index) * D;
  const float r = row.r;
  float dot = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int col = (c * NORM_THREADS + threadIdx.x) * 8;
    if (col < D) {
      float dyv[8], xv[8];
      unpack8(row.dy[c], dyv);
      unpack8(row.x[c], xv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = xv[i] * r;
        dw_acc[c][i] += dyv[i] * xh;
        dot += dyv[i] * wv[c][i] * xh;
      }
    }
  }
  const float mean = block_sum<NORM_THREADS>(dot, scratch) / D;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int col = (c * NORM_THREADS + threadIdx.x) * 8;
    if (col < D) {
      float dyv[8], xv[8], o[8];
      unpack8(row.dy[c], dyv);
      unpack8(row.x[c], xv);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = r * (dyv[i] * wv[c][i] - xv[i] * r * mean);
      if (residual) {
        float res[8];
        unpack8(*reinterpret_cast<const bf16x8*>(residual + base + col), res);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += res[i];
      }
      *reinterpret_cast<bf16x8*>(dx + base + col) = pack8(o);
    }
  }
}

template <int CH>
__global__ void __launch_bounds__(NORM_THREADS) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                  const __nv_bfloat16* __restrict__ x,
                                                                  const float* __restrict__ w,
                                                                  const float* __restrict__ rstd,
                                                                  const __nv_bfloat16* __restrict__ residual,
                                                                  __nv_bfloat16* __restrict__ dx,
                                                                  float* __restrict__ dw_partial, int rows, int D) {
  __shared__ float scratch[NORM_THREADS / 32];
  float dw_acc[CH][8];
  float wv[CH][8];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int col = (c * NORM_THREADS + threadIdx.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      dw_acc[c][i] = 0.f;
      wv[c][i] = col < D ? w[col + i] : 0.f;
    }
  }
  NormRow<CH> a, b;
  int row = blockIdx.x;
  if (row < rows) norm_row_load(a, dy, x, rstd, row, D);
  while (row < rows) {
    const int next = row + gridDim.x;
    if (next < rows) norm_row_load(b, dy, x, rstd, next, D);
    norm_row_finish(a, dw_acc, wv, residual, dx, row, D, scratch);
    if (next >= rows) break;
    const int after = next + gridDim.x;
    if (after < rows) norm_row_load(a, dy, x, rstd, after, D);
    norm_row_finish(b, dw_acc, wv, residual, dx, next, D, scratch);
    row = after;
  }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int col = (c * NORM_THREADS + threadIdx.x) * 8;
    if (col < D) {
#pragma unroll
      for (int i = 0; i < 8; ++i) dw_partial[static_cast<size_t>(blockIdx.x) * D + col + i] = dw_acc[c][i];
    }
  }
}

// out[col] = sum over parts of partial[part][col].  One CTA per 32 columns: lane = column (coalesced 128-byte
// reads), the eight warps take every eighth part, shared memory adds the eight partial sums.
__global__ void __launch_bounds__(256) column_sum_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                        int parts, int D) {
  __shared__ float acc[8][33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 32 + lane;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (col < D) {
    int p = warp;
    for (; p + 24 < parts; p += 32) {
      s0 += partial[static_cast<size_t>(p) * D + col];
      s1 += partial[static_cast<size_t>(p + 8) * D + col];
      s2 += partial[static_cast<size_t>(p + 16) * D + col];
      s3 += partial[static_cast<size_t>(p + 24) * D + col];
    }
    for (; p < parts; p += 8) s0 += partial[static_cast<size_t>(p) * D + col];
  }
  acc[warp][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (warp == 0 && col < D) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += acc[i][lane];
    out[col] = s;
  }
}

// ------------------------------------------------------------------ skinny linear (router: N <= 16 outputs)
constexpr int SKINNY_MAX_N = 16;

// logits[t, n] = sum_k x[t,k] w[n,k]; one warp per token, weights in shared memory.
__global__ void __launch_bounds__(256) skinny_nt_kernel(const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ w, float* __restrict__ out,
                                                        int T, int N, int K) {
  extern __shared__ __nv_bfloat16 ws[];
  for (int i = threadIdx.x * 8; i < N * K; i += blockDim.x * 8)
    *reinterpret_cast<bf16x8*>(ws + i) = *reinterpret_cast<const bf16x8*>(w + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    float acc[SKINNY_MAX_N];
#pragma unroll
    for (int n = 0; n < SKINNY_MAX_N; ++n) acc[n] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
      float xv[8];
      unpack8(*reinterpret_cast<const bf16x8*>(x + static_cast<size_t>(t) * K + k), xv);
#pragma unroll
      for (int n = 0; n < SKINNY_MAX_N; ++n) {
        if (n < N) {
          float wv[8];
          unpack8(*reinterpret_cast<const bf16x8*>(ws + n * K + k), wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[n] += xv[i] * wv[i];
        }
      }
    }
#pragma unroll
    for (int n = 0; n < SKINNY_MAX_N; ++n) {
      if (n < N) {
        const float s = warp_sum(acc[n]);
        if (lane == 0) out[static_cast<size_t>(t) * N + n] = s;
      }
    }
  }
}

// dx[t,k] = sum_n dy[t,n] w[n,k]  (bf16 out)
__global__ void __launch_bounds__(256) skinny_nn_kernel(const float* __restrict__ dy,
                                                        const __nv_bfloat16* __restrict__ w,
                                                        __nv_bfloat16* __restrict__ dx, int T, int N, int K) {
  extern __shared__ __nv_bfloat16 ws[];
  for (int i = threadIdx.x * 8; i < N * K; i += blockDim.x * 8)
    *reinterpret_cast<bf16x8*>(ws + i) = *reinterpret_cast<const bf16x8*>(w + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    float d[SKINNY_MAX_N];
#pragma unroll
    for (int n = 0; n < SKINNY_MAX_N; ++n) d[n] = n < N ? dy[static_cast<size_t>(t) * N + n] : 0.f;
    for (int k = lane * 8; k < K; k += 256) {
      float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int n = 0; n < SKINNY_MAX_N; ++n) {
        if (n < N) {
          float wv[8];
          unpack8(*reinterpret_cast<const bf16x8*>(ws + n * K + k), wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += d[n] * wv[i];
        }
      }
      *reinterpret_cast<bf16x8*>(dx + static_cast<size_t>(t) * K + k) = pack8(o);
    }
  }
}

// dw[n,k] += sum_t dy[t,n] x[t,k]   (fp32 accumulate with atomics; each CTA reduces a token range first)
__global__ void __launch_bounds__(256) skinny_tn_kernel(const float* __restrict__ dy,
                                                        const __nv_bfloat16* __restrict__ x, float* __restrict__ dw,
                                                        int T, int N, int K, int tokens_per_cta) {
  const int t0 = blockIdx.x * tokens_per_cta;
  const int t1 = min(T, t0 + tokens_per_cta);
  for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
    float acc[SKINNY_MAX_N][8];
#pragma unroll
    for (int n = 0; n < SKINNY_MAX_N; ++n)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[n][i] = 0.f;
    for (int t = t0; t < t1; ++t) {
      float xv[8];
      unpack8(*reinterpret_cast<const bf16x8*>(x + static_cast<size_t>(t) * K + k), xv);
#pragma unroll
      for (int n = 0; n < SKINNY_MAX_N; ++n) {
        if (n < N) {
          const float d = dy[static_cast<size_t>(t) * N + n];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[n][i] += d * xv[i];
        }
      }
    }
#pragma unroll
    for (int n = 0; n < SKINNY_MAX_N; ++n) {
      if (n < N) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(dw + static_cast<size_t>(n) * K + k + i, acc[n][i]);
      }
    }
  }
}

// ------------------------------------------------------------------ router softmax / top-2
constexpr int ROUTER_MAX_E = 64;

__global__ void router_top2_fwd_kernel(const float* __restrict__ logits, float* __restrict__ weights,
                                       long long* __restrict__ idx, float* __restrict__ probs, int T, int E) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float p[ROUTER_MAX_E];
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) {
    p[e] = logits[static_cast<size_t>(t) * E + e];
    mx = fmaxf(mx, p[e]);
  }
  float sum = 0.f;
  for (int e = 0; e < E; ++e) {
    p[e] = __expf(p[e] - mx);
    sum += p[e];
  }
  const float inv = 1.f / sum;
  int a = 0, b = -1;
  float pa = -1.f, pb = -1.f;
  for (int e = 0; e < E; ++e) {
    p[e] *= inv;
    probs[static_cast<size_t>(t) * E + e] = p[e];
    if (p[e] > pa) {           // strict: ties keep the lower index first, like topk
      pb = pa; b = a;
      pa = p[e]; a = e;
    } else if (p[e] > pb) {
      pb = p[e]; b = e;
    }
  }
  if (b < 0) {                 // only reachable with non-finite logits: keep the indices valid
    b = a == 0 ? 1 : 0;
    pb = p[b];
  }
  const float s = pa + pb;
  weights[2 * t] = pa / s;
  weights[2 * t + 1] = pb / s;
  idx[2 * t] = a;
  idx[2 * t + 1] = b;
}

__global__ void router_top2_bwd_kernel(const float* __restrict__ dweights, const float* __restrict__ probs,
                                       const long long* __restrict__ idx, const float* __restrict__ weights,
                                       float* __restrict__ dlogits, int T, int E) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int a = static_cast<int>(idx[2 * t]), b = static_cast<int>(idx[2 * t + 1]);
  const float wa = weights[2 * t], wb = weights[2 * t + 1];
  const float da = dweights[2 * t], db = dweights[2 * t + 1];
  const float pa = probs[static_cast<size_t>(t) * E + a], pb = probs[static_cast<size_t>(t) * E + b];
  const float s = pa + pb;
  const float inner = da * wa + db * wb;
  const float dpa = (da - inner) / s, dpb = (db - inner) / s;
  const float dot = dpa * pa + dpb * pb;
  for (int e = 0; e < E; ++e) {
    const float p = probs[static_cast<size_t>(t) * E + e];
    const float dp = e == a ? dpa : (e == b ? dpb : 0.f);
    dlogits[static_cast<size_t>(t) * E + e] = p * (dp - dot);
  }
}

// ------------------------------------------------------------------ SwiGLU backward
// dgu[r, 0:F] = dh * u * silu'(g); dgu[r, F:2F] = dh * silu(g); h = silu(g) * u
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gate,
                                  const __nv_bfloat16* __restrict__ up, __nv_bfloat16* __restrict__ dgu,
                                  __nv_bfloat16* __restrict__ h, const int* __restrict__ live_rows, int rows, int F) {
  const int limit = live_rows ? min(rows, *live_rows) : rows;
  const size_t per_row = F / 8;
  const size_t total = static_cast<size_t>(limit) * per_row;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = i / per_row;
    const size_t col = (i - row * per_row) * 8;
    float d[8], g[8], u[8], og[8], ou[8], oh[8];
    unpack8(*reinterpret_cast<const bf16x8*>(dh + row * F + col), d);
    unpack8(*reinterpret_cast<const bf16x8*>(gate + row * F + col), g);
    unpack8(*reinterpret_cast<const bf16x8*>(up + row * F + col), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sig = 1.f / (1.f + __expf(-g[j]));
      const float sl = g[j] * sig;
      og[j] = d[j] * u[j] * sig * (1.f + g[j] * (1.f - sig));
      ou[j] = d[j] * sl;
      oh[j] = sl * u[j];
    }
    *reinterpret_cast<bf16x8*>(dgu + row * 2 * F + col) = pack8(og);
    *reinterpret_cast<bf16x8*>(dgu + row * 2 * F + F + col) = pack8(ou);
    if (h) *reinterpret_cast<bf16x8*>(h + row * F + col) = pack8(oh);
  }
}

// ------------------------------------------------------------------ cross entropy (in place)
// logits[t,:] <- (softmax(logits[t,:]) - onehot(target)) * scale ; loss += (lse - logit[target]) * scale
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(__nv_bfloat16* __restrict__ logits,
                                                                  const long long* __restrict__ targets,
                                                                  float* __restrict__ loss, int T, int V, float scale) {
  __shared__ float scratch[CE_THREADS / 32];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __nv_bfloat16* row = logits + static_cast<size_t>(t) * V;
    float mx = -INFINITY;
    for (int c = threadIdx.x * 8; c < V; c += CE_THREADS * 8) {
      float v[8];
      unpack8(*reinterpret_cast<const bf16x8*>(row + c), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, v[i]);
    }
    mx = block_max<CE_THREADS>(mx, scratch);
    float sum = 0.f;
    for (int c = threadIdx.x * 8; c < V; c += CE_THREADS * 8) {
      float v[8];
      unpack8(*reinterpret_cast<const bf16x8*>(row + c), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += __expf(v[i] - mx);
    }
    sum = block_sum<CE_THREADS>(sum, scratch);
    const float inv = 1.f / sum;
    const int target = static_cast<int>(targets[t]);
    if (threadIdx.x == 0) {
      const float picked = __bfloat162float(row[target]);
      atomicAdd(loss, (logf(sum) + mx - picked) * scale);
    }
    __syncthreads();
    for (int c = threadIdx.x * 8; c < V; c += CE_THREADS * 8) {
      float v[8];
      unpack8(*reinterpret_cast<const bf16x8*>(row + c), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = __expf(v[i] - mx) * inv;
        if (c + i == target) v[i] -= 1.f;
        v[i] *= scale;
      }
      *reinterpret_cast<bf16x8*>(row + c) = pack8(v);
    }
  }
}

// The same with the whole row held in registers (V <= CE_THREADS * 8 * CE_REG_CHUNKS): one read and one write of
// the logits instead of three reads and one write.  ``loss_scale`` weighs the row's loss in ``loss`` (1/T for a
// mean over T tokens), ``grad_scale`` multiplies the gradient written back (1/T times whatever the caller
// back-propagates into the loss).
constexpr int CE_REG_CHUNKS = 8;
__global__ void __launch_bounds__(CE_THREADS, 2) cross_entropy_reg_kernel(__nv_bfloat16* __restrict__ logits,
                                                                      const long long* __restrict__ targets,
                                                                      float* __restrict__ loss, int T, int V,
                                                                      float loss_scale, float grad_scale) {
  __shared__ float scratch[CE_THREADS / 32];
  float local_loss = 0.f;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __nv_bfloat16* row = logits + static_cast<size_t>(t) * V;
    bf16x8 raw[CE_REG_CHUNKS];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < CE_REG_CHUNKS; ++k) {
      const int c = (k * CE_THREADS + threadIdx.x) * 8;
      if (c < V) {
        raw[k] = *reinterpret_cast<const bf16x8*>(row + c);
        float v[8];
        unpack8(raw[k], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) mx = fmaxf(mx, v[i]);
      }
    }
    mx = block_max<CE_THREADS>(mx, scratch);
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < CE_REG_CHUNKS; ++k) {
      const int c = (k * CE_THREADS + threadIdx.x) * 8;
      if (c < V) {
        float v[8];
        unpack8(raw[k], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += __expf(v[i] - mx);
      }
    }
    sum = block_sum<CE_THREADS>(sum, scratch);
    const float inv = 1.f / sum;
    const int target = static_cast<int>(targets[t]);
#pragma unroll
    for (int k = 0; k < CE_REG_CHUNKS; ++k) {
      const int c = (k * CE_THREADS + threadIdx.x) * 8;
      if (c < V) {
        float v[8];
        unpack8(raw[k], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (c + i == target) local_loss += (logf(sum) + mx - v[i]) * loss_scale;
          v[i] = __expf(v[i] - mx) * inv;
          if (c + i == target) v[i] -= 1.f;
          v[i] *= grad_scale;
        }
        *reinterpret_cast<bf16x8*>(row + c) = pack8(v);
      }
    }
  }
  // one atomic per CTA: the thread that met a target holds that row's loss
  local_loss = block_sum<CE_THREADS>(local_loss, scratch);
  if (threadIdx.x == 0 && local_loss != 0.f) atomicAdd(loss, local_loss);
}

__global__ void scale_bf16_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ factor, size_t n8) {
  const float f = *factor;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float v[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= f;
    reinterpret_cast<bf16x8*>(x)[i] = pack8(v);
  }
}

// ------------------------------------------------------------------ AdamW
template <typename T>
__device__ __forceinline__ float ldf(const T* p, size_t i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void stf(T* p, size_t i, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, size_t i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void ld8<float>(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  unpack8(*reinterpret_cast<const bf16x8*>(p), f);
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void st8<float>(float* p, const float (&f)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<bf16x8*>(p) = pack8(f);
}

// p <- p(1 - lr*wd); m, v moments; p <- p - a_t m/(sqrt(v)+eps).  Optional bf16 copy of the new p.
// Eight elements per thread as 16/32-byte vectors; the last n % 8 elements go one by one.
template <typename P, typename G, typename S>
__global__ void adamw_kernel(P* __restrict__ p, const G* __restrict__ g, S* __restrict__ m, S* __restrict__ v,
                             __nv_bfloat16* __restrict__ p_bf16, size_t n, float lr, float beta1, float beta2,
                             float eps, float wd, float a_t, float grad_scale) {
  const size_t vecs = n / 8;
  const float decay = 1.f - lr * wd;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < vecs;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t o = i * 8;
    float pv[8], gv[8], mv[8], vv[8];
    ld8(p + o, pv);
    ld8(g + o, gv);
    ld8(m + o, mv);
    ld8(v + o, vv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = gv[j] * grad_scale;
      mv[j] = beta1 * mv[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      pv[j] = pv[j] * decay - a_t * mv[j] / (sqrtf(vv[j]) + eps);
    }
    st8(p + o, pv);
    st8(m + o, mv);
    st8(v + o, vv);
    if (p_bf16) st8(p_bf16 + o, pv);
  }
  if (blockIdx.x == 0) {
    for (size_t i = vecs * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const float gj = ldf(g, i) * grad_scale;
      const float mj = beta1 * ldf(m, i) + (1.f - beta1) * gj;
      const float vj = beta2 * ldf(v, i) + (1.f - beta2) * gj * gj;
      const float pj = ldf(p, i) * decay - a_t * mj / (sqrtf(vj) + eps);
      stf(p, i, pj);
      stf(m, i, mj);
      stf(v, i, vj);
      if (p_bf16) p_bf16[i] = __float2bfloat16_rn(pj);
    }
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int T, int D) {
  const int per_row = D / 8;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < static_cast<size_t>(T) * per_row;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / per_row, c = (i - t * per_row) * 8;
    *reinterpret_cast<bf16x8*>(out + t * D + c) =
        *reinterpret_cast<const bf16x8*>(table + static_cast<size_t>(ids[t]) * D + c);
  }
}
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                     float* __restrict__ grad, int T, int D) {
  const int per_row = D / 8;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < static_cast<size_t>(T) * per_row;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / per_row, c = (i - t * per_row) * 8;
    float v[8];
    unpack8(*reinterpret_cast<const bf16x8*>(dy + t * D + c), v);
    float* dst = grad + static_cast<size_t>(ids[t]) * D + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, v[j]);
  }
}

// ------------------------------------------------------------------ RoPE (adjacent pairs), in place
// x: [B, S, H, hd] with token pitch ``pitch`` elements (a view into the fused QKV buffer); rotates heads
// [0, H).  sign = +1 forward, -1 backward (the transpose rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, int tokens, int S, int H, int hd, long long pitch,
                            float sign) {
  const int vec_per_head = hd / 8;
  const size_t total = static_cast<size_t>(tokens) * H * vec_per_head;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec_per_head);
    const int h = static_cast<int>((i / vec_per_head) % H);
    const size_t tok = i / (static_cast<size_t>(vec_per_head) * H);
    const int pos = static_cast<int>(tok % S);
    __nv_bfloat16* ptr = x + tok * pitch + static_cast<size_t>(h) * hd + v * 8;
    float f[8];
    unpack8(*reinterpret_cast<const bf16x8*>(ptr), f);
    const float4 c = *reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(pos) * (hd / 2) + v * 4);
    float4 s = *reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(pos) * (hd / 2) + v * 4);
    s.x *= sign; s.y *= sign; s.z *= sign; s.w *= sign;
    const float cc[4] = {c.x, c.y, c.z, c.w}, sn[4] = {s.x, s.y, s.z, s.w};
    float o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[2 * j] = f[2 * j] * cc[j] - f[2 * j + 1] * sn[j];
      o[2 * j + 1] = f[2 * j] * sn[j] + f[2 * j + 1] * cc[j];
    }
    *reinterpret_cast<bf16x8*>(ptr) = pack8(o);
  }
}

// SM count of the current device (grids are sized as a multiple of it).
static inline int sm_count_ew() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}
static inline int grid_for(size_t work, int threads, int per_sm = 16) {
  size_t blocks = (work + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  const size_t cap = static_cast<size_t>(sm_count_ew()) * per_sm;
  return static_cast<int>(blocks > cap ? cap : blocks);
}
static inline int ok() { return cudaGetLastError() == cudaSuccess ? 0 : -1; }

}  // namespace b2

using namespace b2;
typedef __nv_bfloat16 bf16;

extern "C" {

int b2_rmsnorm_fwd(const void* x, const void* delta, const float* w, void* sum_out, void* y, float* rstd, int rows,
                   int D, float eps, cudaStream_t s) {
  if (D % 8 || D > NORM_THREADS * 8 * NORM_MAX_CHUNKS) return -10;
  const int grid = min(rows, sm_count_ew() * 8);
#define B2_NORM_FWD(CH)                                                                                         \
  rmsnorm_fwd_kernel<CH><<<grid, NORM_THREADS, 0, s>>>((const bf16*)x, (const bf16*)delta, w, (bf16*)sum_out, \
                                                       (bf16*)y, rstd, rows, D, eps)
  if (D <= 2048) B2_NORM_FWD(1);
  else if (D <= 4096) B2_NORM_FWD(2);
  else B2_NORM_FWD(4);
#undef B2_NORM_FWD
  return ok();
}

// dw_partial: fp32 [parts, D] scratch with parts = b2_rmsnorm_bwd_parts(rows); dw: fp32 [D] (overwritten).
// two CTAs are resident per SM (registers): one wave, and as few partial rows as possible for the column sum
int b2_rmsnorm_bwd_parts(int rows) { return min(rows, sm_count_ew() * 2); }
int b2_rmsnorm_bwd(const void* dy, const void* x, const float* w, const float* rstd, const void* residual, void* dx,
                   float* dw_partial, float* dw, int rows, int D, cudaStream_t s) {
  if (D % 8 || D > NORM_THREADS * 8 * NORM_MAX_CHUNKS) return -10;
  const int parts = b2_rmsnorm_bwd_parts(rows);
#define B2_NORM_BWD(CH)                                                                                       \
  rmsnorm_bwd_kernel<CH><<<parts, NORM_THREADS, 0, s>>>((const bf16*)dy, (const bf16*)x, w, rstd,             \
                                                        (const bf16*)residual, (bf16*)dx, dw_partial, rows, D)
  if (D <= 2048) B2_NORM_BWD(1);
  else if (D <= 4096) B2_NORM_BWD(2);
  else B2_NORM_BWD(4);
#undef B2_NORM_BWD
  column_sum_kernel<<<(D + 31) / 32, 256, 0, s>>>(dw_partial, dw, parts, D);
  return ok();
}

int b2_skinny_nt(const void* x, const void* w, float* out, int T, int N, int K, cudaStream_t s) {
  if (N > SKINNY_MAX_N || K % 8 || (N * K) % 8) return -10;
  const size_t smem = static_cast<size_t>(N) * K * 2;
  if (smem > 200 * 1024) return -11;
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(skinny_nt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(skinny_nn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    set = true;
  }
  skinny_nt_kernel<<<min((T + 7) / 8, sm_count_ew() * 2), 256, smem, s>>>((const bf16*)x, (const bf16*)w, out, T, N, K);
  return ok();
}
int b2_skinny_nn(const float* dy, const void* w, void* dx, int T, int N, int K, cudaStream_t s) {
  if (N > SKINNY_MAX_N || K % 8) return -10;
  const size_t smem = static_cast<size_t>(N) * K * 2;
  if (smem > 200 * 1024) return -11;
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(skinny_nn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    set = true;
  }
  skinny_nn_kernel<<<min((T + 7) / 8, sm_count_ew() * 2), 256, smem, s>>>(dy, (const bf16*)w, (bf16*)dx, T, N, K);
  return ok();
}
int b2_skinny_tn(const float* dy, const void* x, float* dw, int T, int N, int K, cudaStream_t s) {
  if (N > SKINNY_MAX_N || K % 8) return -10;
  const int ctas = min(sm_count_ew() * 2, (T + 31) / 32);
  const int per = (T + ctas - 1) / ctas;
  skinny_tn_kernel<<<ctas, 256, 0, s>>>(dy, (const bf16*)x, dw, T, N, K, per);
  return ok();
}

int b2_router_top2_fwd(const float* logits, float* weights, long long* idx, float* probs, int T, int E,
                       cudaStream_t s) {
  if (E > ROUTER_MAX_E || E < 2) return -10;
  router_top2_fwd_kernel<<<(T + 127) / 128, 128, 0, s>>>(logits, weights, idx, probs, T, E);
  return ok();
}
int b2_router_top2_bwd(const float* dweights, const float* probs, const long long* idx, const float* weights,
                       float* dlogits, int T, int E, cudaStream_t s) {
  router_top2_bwd_kernel<<<(T + 127) / 128, 128, 0, s>>>(dweights, probs, idx, weights, dlogits, T, E);
  return ok();
}

int b2_swiglu_bwd(const void* dh, const void* gate, const void* up, void* dgu, void* h, const int* live_rows, int rows,
                  int F, cudaStream_t s) {
  if (F % 8) return -10;
  swiglu_bwd_kernel<<<grid_for(static_cast<size_t>(rows) * F / 8, 256), 256, 0, s>>>(
      (const bf16*)dh, (const bf16*)gate, (const bf16*)up, (bf16*)dgu, (bf16*)h, live_rows, rows, F);
  return ok();
}

// loss must be zeroed by the caller; scale is usually 1/T (mean over tokens).
int b2_cross_entropy(void* logits, const long long* targets, float* loss, int T, int V, float scale, cudaStream_t s) {
  if (V % 8) return -10;
  cross_entropy_kernel<<<min(T, sm_count_ew() * 4), CE_THREADS, 0, s>>>((bf16*)logits, targets, loss, T, V, scale);
  return ok();
}
// Loss and gradient scaled separately; rows up to 32768 entries stay in registers (one read, one write).
int b2_cross_entropy2(void* logits, const long long* targets, float* loss, int T, int V, float loss_scale,
                      float grad_scale, cudaStream_t s) {
  if (V % 8) return -10;
  if (V > CE_THREADS * 8 * CE_REG_CHUNKS && loss_scale != grad_scale) return -11;   // the streaming kernel has one scale
  if (V <= CE_THREADS * 8 * CE_REG_CHUNKS) {
    cross_entropy_reg_kernel<<<min(T, sm_count_ew() * 4), CE_THREADS, 0, s>>>((bf16*)logits, targets, loss, T, V,
                                                                              loss_scale, grad_scale);
    return ok();
  }
  cross_entropy_kernel<<<min(T, sm_count_ew() * 4), CE_THREADS, 0, s>>>((bf16*)logits, targets, loss, T, V, loss_scale);
  return ok();
}
int b2_scale_bf16(void* x, const float* factor, long long n, cudaStream_t s) {
  if (n % 8) return -10;
  scale_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((bf16*)x, factor, n / 8);
  return ok();
}

// dtype codes: 0 fp32, 1 bf16.  p_bf16 may be null.
int b2_adamw(void* p, const void* g, void* m, void* v, void* p_bf16, long long n, int p_dt, int g_dt, int s_dt,
             float lr, float beta1, float beta2, float eps, float wd, float a_t, float grad_scale, cudaStream_t s) {
  const int grid = grid_for((n + 7) / 8, 256, 16);
#define B2_ADAMW(P, G, S)                                                                                      \
  adamw_kernel<P, G, S><<<grid, 256, 0, s>>>((P*)p, (const G*)g, (S*)m, (S*)v, (bf16*)p_bf16, n, lr, beta1, beta2, \
                                             eps, wd, a_t, grad_scale)
  const int code = p_dt * 4 + g_dt * 2 + s_dt;
  switch (code) {
    case 0: B2_ADAMW(float, float, float); break;
    case 1: B2_ADAMW(float, float, bf16); break;
    case 2: B2_ADAMW(float, bf16, float); break;
    case 3: B2_ADAMW(float, bf16, bf16); break;
    case 4: B2_ADAMW(bf16, float, float); break;
    case 5: B2_ADAMW(bf16, float, bf16); break;
    case 6: B2_ADAMW(bf16, bf16, float); break;
    case 7: B2_ADAMW(bf16, bf16, bf16); break;
    default: return -10;
  }
#undef B2_ADAMW
  return ok();
}
int b2_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t s) {
  cast_f32_bf16_kernel<<<grid_for(n, 256, 32), 256, 0, s>>>(src, (bf16*)dst, n);
  return ok();
}

int b2_embedding_fwd(const long long* ids, const void* table, void* out, int T, int D, cudaStream_t s) {
  if (D % 8) return -10;
  embedding_fwd_kernel<<<grid_for(static_cast<size_t>(T) * D / 8, 256), 256, 0, s>>>(ids, (const bf16*)table,
                                                                                    (bf16*)out, T, D);
  return ok();
}
int b2_embedding_bwd(const long long* ids, const void* dy, float* grad, int T, int D, cudaStream_t s) {
  if (D % 8) return -10;
  embedding_bwd_kernel<<<grid_for(static_cast<size_t>(T) * D / 8, 256), 256, 0, s>>>(ids, (const bf16*)dy, grad, T, D);
  return ok();
}

int b2_rope(void* x, const float* cos_t, const float* sin_t, int tokens, int S, int H, int hd, long long pitch,
            float sign, cudaStream_t s) {
  if (hd % 8 || pitch % 8) return -10;
  rope_kernel<<<grid_for(static_cast<size_t>(tokens) * H * hd / 8, 256), 256, 0, s>>>((bf16*)x, cos_t, sin_t, tokens, S,
                                                                                     H, hd, pitch, sign);
  return ok();
}

}  // extern "C"

namespace b2 {
// The device-wide nanosecond clock, stored when the stream reaches this launch: two of these bracket a region
// with one clock for every SM (CUDA events measure the same span; this form can be read by other kernels too).
__global__ void timestamp_kernel(unsigned long long* out) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *out = t;
}
}  // namespace b2

extern "C" int b2_device_timestamp(unsigned long long* out, cudaStream_t s) {
  b2::timestamp_kernel<<<1, 1, 0, s>>>(out);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
