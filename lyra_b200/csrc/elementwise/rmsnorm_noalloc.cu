// Allocation-free RMSNorm backward: see rmsnorm_noalloc.h for who needs it, the limits and the sharing rules.
#include "rmsnorm_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace {

constexpr int NA_THREADS = 256;
constexpr int NA_MAXV = LYRA_RMSNORM_NOALLOC_MAX_C / (8 * NA_THREADS);  // 16-byte vectors per thread per row
constexpr int NA_MAX_DEVICES = 64;

// Per-block partial sums of the scale gradient: [LYRA_RMSNORM_NOALLOC_BLOCKS][C]. In host code this name is only a
// handle for the runtime; the device address is obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_partial_scratch[LYRA_RMSNORM_NOALLOC_BLOCKS * LYRA_RMSNORM_NOALLOC_MAX_C];

struct alignas(16) Vec8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ float na_block_sum(float v, float* red) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < NA_THREADS / 32; ++i) t += red[i];
  return t;
}

// Same mathematics as the regular backward kernel: g = dy * scale, dx = (g - xhat * mean(g * xhat)) * rstd,
// per-block partial of dscale = sum over the block's rows of dy * xhat, written to `partial[blockIdx.x][:]`.
__global__ void __launch_bounds__(NA_THREADS) na_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                                                                    const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                                                                    __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int C) {
  __shared__ float red[NA_THREADS / 32];
  const int nvec = C / 8;
  float ds[NA_MAXV][8];
#pragma unroll
  for (int j = 0; j < NA_MAXV; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) ds[j][i] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const Vec8* xr = reinterpret_cast<const Vec8*>(x + (long long)row * C);
    const Vec8* gr = reinterpret_cast<const Vec8*>(dy + (long long)row * C);
    const float rstd = rstd_in[row];
    float xh[NA_MAXV][8], g[NA_MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NA_MAXV; ++j) {
      const int c = threadIdx.x + j * NA_THREADS;
      if (c < nvec) {
        const Vec8 xv = xr[c], dv = gr[c];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 xf = __bfloat1622float2(xv.v[i]), df = __bfloat1622float2(dv.v[i]);
          xh[j][2 * i] = xf.x * rstd;
          xh[j][2 * i + 1] = xf.y * rstd;
          g[j][2 * i] = df.x * scale[c * 8 + 2 * i];
          g[j][2 * i + 1] = df.y * scale[c * 8 + 2 * i + 1];
          ds[j][2 * i] += df.x * xh[j][2 * i];
          ds[j][2 * i + 1] += df.y * xh[j][2 * i + 1];
          dot += g[j][2 * i] * xh[j][2 * i] + g[j][2 * i + 1] * xh[j][2 * i + 1];
        }
      }
    }
    const float mean = na_block_sum(dot, red) / C;
    Vec8* dr = reinterpret_cast<Vec8*>(dx + (long long)row * C);
#pragma unroll
    for (int j = 0; j < NA_MAXV; ++j) {
      const int c = threadIdx.x + j * NA_THREADS;
      if (c < nvec) {
        Vec8 o;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          o.v[i] = __floats2bfloat162_rn((g[j][2 * i] - xh[j][2 * i] * mean) * rstd, (g[j][2 * i + 1] - xh[j][2 * i + 1] * mean) * rstd);
        dr[c] = o;
      }
    }
  }
  // every launched block writes its whole row of partials (zeros if it had no rows), so no clearing is needed
#pragma unroll
  for (int j = 0; j < NA_MAXV; ++j) {
    const int c = threadIdx.x + j * NA_THREADS;
    if (c < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) partial[(long long)blockIdx.x * C + c * 8 + i] = ds[j][i];
    }
  }
}

// dscale[c] = sum over blocks (ascending) of partial[b][c]
__global__ void na_reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ dscale, int blocks, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float t = 0.f;
  for (int b = 0; b < blocks; ++b) t += partial[(long long)b * C + c];
  dscale[c] = t;
}

float* g_scratch_addr[NA_MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device; looked up once per device.
int scratch_for_current_device(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES) return LYRA_NOALLOC_ERR_SYMBOL;
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_partial_scratch);
    if (e != cudaSuccess || !p) {
      fprintf(stderr, "[lyra_b200] rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return LYRA_NOALLOC_ERR_SYMBOL;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int lyra_rmsnorm_bwd_noalloc(const void* x, const float* scale, const float* rstd, const void* dy, void* dx, float* dscale, int rows,
                                        int C, void* stream) {
  if (C > LYRA_RMSNORM_NOALLOC_MAX_C) {
    fprintf(stderr, "[lyra_b200] rmsnorm_bwd_noalloc: C = %d exceeds the built-in scratch (max %d); use lyra_rmsnorm_bwd with your own buffer\n", C,
            LYRA_RMSNORM_NOALLOC_MAX_C);
    return LYRA_NOALLOC_ERR_TOO_LARGE;
  }
  if (C <= 0 || C % 8 || rows < 0) {
    fprintf(stderr, "[lyra_b200] rmsnorm_bwd_noalloc: C = %d must be a positive multiple of 8 and rows = %d non-negative\n", C, rows);
    return LYRA_NOALLOC_ERR_BAD_SHAPE;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int blocks = rows < LYRA_RMSNORM_NOALLOC_BLOCKS ? rows : LYRA_RMSNORM_NOALLOC_BLOCKS;
  if (blocks < 1) blocks = 1;
  na_rmsnorm_bwd_kernel<<<blocks, NA_THREADS, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), scale, rstd, reinterpret_cast<const __nv_bfloat16*>(dy),
                                                       reinterpret_cast<__nv_bfloat16*>(dx), scratch, rows, C);
  na_reduce_partials_kernel<<<(C + 255) / 256, 256, 0, s>>>(scratch, dscale, blocks, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
