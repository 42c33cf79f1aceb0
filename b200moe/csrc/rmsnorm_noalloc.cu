// Allocation-free RMSNorm backward: see rmsnorm_noalloc.h for who needs it and
// the rules of use.  The per-block partial sums of the gain gradient live in a
// file-scope device array instead of a caller-provided buffer.
#include "rmsnorm_noalloc.h"

#include <cuda_bf16.h>
#include <stdint.h>

#include <mutex>

namespace {

constexpr int THREADS = 256;
constexpr int MAX_CHUNKS = B2_NOALLOC_MAX_D / (THREADS * 8);   // 8-element vectors per thread
constexpr int MAX_DEVICES = 64;

// Partial gain gradients, one row of D floats per block.  In host code this name
// is only a handle; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_partials[B2_NOALLOC_PARTS * B2_NOALLOC_MAX_D];

struct alignas(16) Pack8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const Pack8 raw = *reinterpret_cast<const Pack8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(raw.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  Pack8 raw;
#pragma unroll
  for (int i = 0; i < 4; ++i) raw.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<Pack8*>(p) = raw;
}

__device__ __forceinline__ float block_total(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) total += scratch[i];
  return total;
}

__global__ void __launch_bounds__(THREADS) bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy,
                                                           const __nv_bfloat16* __restrict__ x,
                                                           const float* __restrict__ w, const float* __restrict__ rstd,
                                                           const __nv_bfloat16* __restrict__ residual,
                                                           __nv_bfloat16* __restrict__ dx, float* __restrict__ partials,
                                                           int rows, int D) {
  __shared__ float scratch[THREADS / 32];
  float acc[MAX_CHUNKS][8], gain[MAX_CHUNKS][8];
#pragma unroll
  for (int c = 0; c < MAX_CHUNKS; ++c) {
    const int col = (c * THREADS + threadIdx.x) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc[c][i] = 0.f;
      gain[c][i] = col < D ? w[col + i] : 0.f;
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * D;
    const float r = rstd[row];
    float g[MAX_CHUNKS][8], xh[MAX_CHUNKS][8];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) {
      const int col = (c * THREADS + threadIdx.x) * 8;
      if (col < D) {
        float dyv[8], xv[8];
        load8(dy + base + col, dyv);
        load8(x + base + col, xv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[c][i] = xv[i] * r;
          acc[c][i] += dyv[i] * xh[c][i];
          g[c][i] = dyv[i] * gain[c][i];
          dot += g[c][i] * xh[c][i];
        }
      }
    }
    const float mean = block_total(dot, scratch) / D;
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) {
      const int col = (c * THREADS + threadIdx.x) * 8;
      if (col < D) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = r * (g[c][i] - xh[c][i] * mean);
        if (residual) {
          float res[8];
          load8(residual + base + col, res);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += res[i];
        }
        store8(dx + base + col, o);
      }
    }
  }
  // every block writes its whole row of the scratch, so nothing stale is ever summed
#pragma unroll
  for (int c = 0; c < MAX_CHUNKS; ++c) {
    const int col = (c * THREADS + threadIdx.x) * 8;
    if (col < D) {
#pragma unroll
      for (int i = 0; i < 8; ++i) partials[static_cast<size_t>(blockIdx.x) * D + col + i] = acc[c][i];
    }
  }
}

__global__ void sum_parts_kernel(const float* __restrict__ partials, float* __restrict__ dw, int parts, int D) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= D) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partials[static_cast<size_t>(p) * D + col];
  dw[col] = s;
}

std::mutex g_lock;
float* g_scratch_ptr[MAX_DEVICES] = {};

// Device address of g_partials on the current device, looked up once per device.
int scratch_for_current_device(float** out) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) return -4;
  if (device < 0 || device >= MAX_DEVICES) return -5;
  std::lock_guard<std::mutex> guard(g_lock);
  if (!g_scratch_ptr[device]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_partials) != cudaSuccess || ptr == nullptr) return -6;
    g_scratch_ptr[device] = static_cast<float*>(ptr);
  }
  *out = g_scratch_ptr[device];
  return 0;
}

}  // namespace

extern "C" int b2_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd,
                                      const void* residual, void* dx, float* dw, int rows, int D,
                                      cudaStream_t stream) {
  if (!dy || !x || !w || !rstd || !dx || !dw) return -1;
  if (rows < 1 || D < 8 || D % 8) return -2;
  if (D > B2_NOALLOC_MAX_D) return -3;
  // the kernels move eight bf16 per 16-byte access: a pointer off that grid would fault on the device
  const uintptr_t wide = reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) |
                         reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(residual);
  const uintptr_t narrow = reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(rstd) |
                           reinterpret_cast<uintptr_t>(dw);
  if ((wide & 15) || (narrow & 3)) return -8;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  const int parts = rows < B2_NOALLOC_PARTS ? rows : B2_NOALLOC_PARTS;
  bwd_rows_kernel<<<parts, THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), w, rstd,
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(dx), scratch, rows, D);
  // cudaPeekAtLastError: report this launch without consuming an error some earlier, unrelated call left behind
  if (cudaPeekAtLastError() != cudaSuccess) return -7;
  sum_parts_kernel<<<(D + 255) / 256, 256, 0, stream>>>(scratch, dw, parts, D);
  return cudaPeekAtLastError() == cudaSuccess ? 0 : -7;
}

extern "C" const char* b2_rmsnorm_bwd_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "null pointer among dy, x, w, rstd, dx, dw";
    case -2: return "rows must be >= 1 and D a positive multiple of 8";
    case -3: return "D exceeds B2_NOALLOC_MAX_D (8192): the built-in scratch cannot hold the partial sums";
    case -4: return "cudaGetDevice failed";
    case -5: return "device ordinal beyond the 64 this library tracks";
    case -6: return "cudaGetSymbolAddress failed for the built-in scratch";
    case -7: return "kernel launch failed (or an earlier CUDA error is still pending on this thread)";
    case -8: return "dy, x, dx and residual must be 16-byte aligned, w, rstd and dw 4-byte aligned";
    default: return "unknown code";
  }
}
