// Quantisation kernels (bandwidth bound, one pass over the data each):
//   mxfp4_decode      : GPT-OSS expert weights, 32 e2m1 values per 16-byte block with one e8m0 exponent -> bf16
//                       (lyra/gpt_oss.py:20-34 in the reference does this with a table lookup in XLA)
//   fp8_quantize_2d   : [L, R, C] fp32/bf16 -> e4m3 values + one fp32 scale per (br x bc) block (amax / 448; lyra/nn/quant.py:55-73)
//   fp8_dequantize_2d : the inverse, value * scale rounded to bf16
//   fp8_quantize_rows : one scale per row of D values (KV-cache update, block (1, D); lyra/model.py:221-226)
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

// One thread per 16-byte block: 32 outputs (64 bytes).
__global__ void mxfp4_decode_kernel(const uint4* __restrict__ blocks, const uint8_t* __restrict__ scales, uint4* __restrict__ out, long long n_blocks) {
  // e2m1 magnitudes times two, so the table is integral: 0, .5, 1, 1.5, 2, 3, 4, 6
  const float lut[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_blocks; i += (long long)gridDim.x * blockDim.x) {
    const uint4 raw = blocks[i];
    const float sc = exp2f(static_cast<float>(static_cast<int>(scales[i]) - 127));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (w[j] >> (8 * b)) & 0xffu;
        const uint32_t lo = byte & 0xfu, hi = byte >> 4;
        const float flo = (lo & 8u) ? -lut[lo & 7u] : lut[lo & 7u];
        const float fhi = (hi & 8u) ? -lut[hi & 7u] : lut[hi & 7u];
        o[j * 4 + b] = pack2(flo * sc, fhi * sc);
      }
    }
    uint4* dst = out + i * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
  }
}

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  return m;
}

// grid (C / bc, R / br, L); one CTA per scale block.
template <typename T>
__global__ void fp8_quantize_2d_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, int R, int C, int br, int bc) {
  __shared__ float red[32];
  const long long base = ((long long)blockIdx.z * R + (long long)blockIdx.y * br) * C + (long long)blockIdx.x * bc;
  const int n = br * bc;
  float amax = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) amax = fmaxf(amax, fabsf(ldf(x, base + (long long)(i / bc) * C + i % bc)));
  amax = block_max(amax, red);
  const float sc = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;   // IEEE division: the build uses fast-math, the scales must match the CPU formula
  const float inv = __frcp_rn(sc);
  if (threadIdx.x == 0) scale[((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x] = sc;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const long long at = base + (long long)(i / bc) * C + i % bc;
    const float v = fminf(fmaxf(__fmul_rn(ldf(x, at), inv), -448.f), 448.f);
    q[at] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
  }
}

// 16 values per thread; bc % 16 == 0.
__global__ void fp8_dequantize_2d_kernel(const uint4* __restrict__ q, const float* __restrict__ scale, uint4* __restrict__ out, long long n16, int R, int C,
                                         int br, int bc) {
  const int c16 = C / 16, sb_r = R / br, sb_c = C / bc;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const long long row_all = i / c16;
    const int col = static_cast<int>(i % c16) * 16;
    const long long l = row_all / R;
    const int r = static_cast<int>(row_all % R);
    const float sc = scale[(l * sb_r + r / br) * sb_c + col / bc];
    const uint4 raw = q[i];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(static_cast<uint16_t>((w[u] >> (16 * h)) & 0xffffu), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<__half2*>(&hr));
        o[2 * u + h] = pack2(f.x * sc, f.y * sc);
      }
    }
    out[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    out[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// One warp per row of D values (D % 32 == 0, D <= 1024).
template <typename T>
__global__ void fp8_quantize_rows_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, long long rows, int D,
                                         long long x_row_stride, long long q_row_stride) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float amax = 0.f;
  for (int c = lane; c < D; c += 32) amax = fmaxf(amax, fabsf(ldf(x, row * x_row_stride + c)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float sc = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;   // IEEE division: the build uses fast-math, the scales must match the CPU formula
  const float inv = __frcp_rn(sc);
  if (lane == 0) scale[row] = sc;
  for (int c = lane; c < D; c += 32) {
    const float v = fminf(fmaxf(__fmul_rn(ldf(x, row * x_row_stride + c), inv), -448.f), 448.f);
    q[row * q_row_stride + c] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
  }
}

int grid_for(long long n, int block) {
  const long long b = (n + block - 1) / block;
  return static_cast<int>(b < 1 ? 1 : (b > 148LL * 16 ? 148LL * 16 : b));
}

}  // namespace

extern "C" int lyra_mxfp4_decode(const void* blocks, const void* scales, void* out, long long n_blocks, cudaStream_t stream) {
  if (n_blocks <= 0) return 0;
  mxfp4_decode_kernel<<<grid_for(n_blocks, 256), 256, 0, stream>>>(static_cast<const uint4*>(blocks), static_cast<const uint8_t*>(scales),
                                                                  static_cast<uint4*>(out), n_blocks);
  return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

extern "C" int lyra_fp8_quantize_2d(const void* x, int x_bf16, void* q, float* scale, int L, int R, int C, int br, int bc, cudaStream_t stream) {
  if (L <= 0 || R <= 0 || C <= 0) return 0;
  if (R % br || C % bc || L > 65535 || R / br > 65535) return -101;
  dim3 grid(C / bc, R / br, L);
  if (x_bf16)
    fp8_quantize_2d_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scale, R, C, br, bc);
  else
    fp8_quantize_2d_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<uint8_t*>(q), scale, R, C, br, bc);
  return cudaGetLastError() == cudaSuccess ? 0 : -102;
}

extern "C" int lyra_fp8_dequantize_2d(const void* q, const float* scale, void* out, int L, int R, int C, int br, int bc, cudaStream_t stream) {
  if (L <= 0 || R <= 0 || C <= 0) return 0;
  if (R % br || C % bc || bc % 16) return -103;
  const long long n16 = (long long)L * R * C / 16;
  fp8_dequantize_2d_kernel<<<grid_for(n16, 256), 256, 0, stream>>>(static_cast<const uint4*>(q), scale, static_cast<uint4*>(out), n16, R, C, br, bc);
  return cudaGetLastError() == cudaSuccess ? 0 : -104;
}

extern "C" int lyra_fp8_quantize_rows(const void* x, int x_bf16, void* q, float* scale, long long rows, int D, long long x_row_stride,
                                      long long q_row_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D % 32 || D > 1024) return -105;
  const int wpb = 8;
  const int grid = static_cast<int>((rows + wpb - 1) / wpb);
  if (x_bf16)
    fp8_quantize_rows_kernel<__nv_bfloat16><<<grid, wpb * 32, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), scale, rows, D,
                                                                           x_row_stride, q_row_stride);
  else
    fp8_quantize_rows_kernel<float><<<grid, wpb * 32, 0, stream>>>(static_cast<const float*>(x), static_cast<uint8_t*>(q), scale, rows, D, x_row_stride,
                                                                   q_row_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : -106;
}
