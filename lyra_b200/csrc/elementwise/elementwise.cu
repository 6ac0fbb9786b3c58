// Bandwidth-bound fused kernels: RMSNorm (fwd / bwd), clamped SwiGLU (fwd / bwd), per-head QK RMS-norm + RoPE,
// and the MoE row movement (scatter into the padded expert-sorted layout, weighted top-k combine and its gradients).
// All move 16 bytes per thread per access; reductions are fixed-order (deterministic, no float atomics).
// Semantics: lyra/model.py:183-191 (rotate, rms_norm), lyra/kernels/common.py:98-114 (swiglu), lyra/model.py:519-557
// (permute / combine).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/tmap.h"

namespace lyra {

struct alignas(16) BF8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void unpack8(const BF8& b, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(b.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ BF8 pack8(const float (&f)[8]) {
  BF8 b;
#pragma unroll
  for (int i = 0; i < 4; ++i) b.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return b;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// ------------------------------------------------------------------------------------------------ RMSNorm
constexpr int RN_THREADS = 256;
constexpr int RN_MAXV = 4;  // up to 4 x 8 columns per thread -> C <= 8192

__global__ void __launch_bounds__(RN_THREADS) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                                                                 __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows, int C, float eps) {
  __shared__ float red[RN_THREADS / 32];
  const int nvec = C / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const BF8* xr = reinterpret_cast<const BF8*>(x + (long long)row * C);
    float v[RN_MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
      const int c = threadIdx.x + j * RN_THREADS;
      if (c < nvec) {
        unpack8(xr[c], v[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[j][i] * v[j][i];
      }
    }
    const float rstd = rsqrtf(block_sum(ss, red) / C + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    BF8* yr = reinterpret_cast<BF8*>(y + (long long)row * C);
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
      const int c = threadIdx.x + j * RN_THREADS;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = v[j][i] * rstd * scale[c * 8 + i];
        yr[c] = pack8(o);
      }
    }
  }
}

// One warp per row for C = NV * 256 (NV 16-byte vectors per lane): no block-wide barrier, NV independent 16-byte loads in
// flight per lane. The block-per-row kernel above pays two __syncthreads per row and holds one vector per thread at C = 2048.
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                                                               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows, float eps) {
  constexpr int C = NV * 256;
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int row = warp; row < rows; row += nwarps) {
    const BF8* xr = reinterpret_cast<const BF8*>(x + (long long)row * C);
    BF8 raw[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) raw[j] = xr[lane + 32 * j];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float v[8];
      unpack8(raw[j], v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
    const float rstd = rsqrtf(ss / C + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    BF8* yr = reinterpret_cast<BF8*>(y + (long long)row * C);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float v[8], o[8];
      unpack8(raw[j], v);
      const float4 s0 = reinterpret_cast<const float4*>(scale)[(lane + 32 * j) * 2], s1 = reinterpret_cast<const float4*>(scale)[(lane + 32 * j) * 2 + 1];
      o[0] = v[0] * rstd * s0.x; o[1] = v[1] * rstd * s0.y; o[2] = v[2] * rstd * s0.z; o[3] = v[3] * rstd * s0.w;
      o[4] = v[4] * rstd * s1.x; o[5] = v[5] * rstd * s1.y; o[6] = v[6] * rstd * s1.z; o[7] = v[7] * rstd * s1.w;
      yr[lane + 32 * j] = pack8(o);
    }
  }
}

// dx = (g - xhat * mean(g * xhat)) * rstd with g = dy * scale; dscale partial per block = sum_rows dy * xhat
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                                                                 const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                                                                 __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int C) {
  __shared__ float red[RN_THREADS / 32];
  const int nvec = C / 8;
  float ds[RN_MAXV][8];
#pragma unroll
  for (int j = 0; j < RN_MAXV; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) ds[j][i] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const BF8* xr = reinterpret_cast<const BF8*>(x + (long long)row * C);
    const BF8* gr = reinterpret_cast<const BF8*>(dy + (long long)row * C);
    const float rstd = rstd_in[row];
    float xh[RN_MAXV][8], g[RN_MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
      const int c = threadIdx.x + j * RN_THREADS;
      if (c < nvec) {
        float xv[8], dv[8];
        unpack8(xr[c], xv);
        unpack8(gr[c], dv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[j][i] = xv[i] * rstd;
          g[j][i] = dv[i] * scale[c * 8 + i];
          ds[j][i] += dv[i] * xh[j][i];
          dot += g[j][i] * xh[j][i];
        }
      }
    }
    const float mean = block_sum(dot, red) / C;
    BF8* dr = reinterpret_cast<BF8*>(dx + (long long)row * C);
#pragma unroll
    for (int j = 0; j < RN_MAXV; ++j) {
      const int c = threadIdx.x + j * RN_THREADS;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (g[j][i] - xh[j][i] * mean) * rstd;
        dr[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < RN_MAXV; ++j) {
    const int c = threadIdx.x + j * RN_THREADS;
    if (c < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) partial[(long long)blockIdx.x * C + c * 8 + i] = ds[j][i];
    }
  }
}

// Warp-per-row backward for C = NV * 256 <= 2048: x and dy stay packed in registers between the two passes, every warp keeps
// its own dscale partial (row `warp` of `partial`, which therefore has one row per warp of the launch).
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                                                               const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dy,
                                                               __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int nwarps) {
  constexpr int C = NV * 256;
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (warp >= nwarps) return;
  float ds[NV][8];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) ds[j][i] = 0.f;
  for (int row = warp; row < rows; row += nwarps) {
    const BF8* xr = reinterpret_cast<const BF8*>(x + (long long)row * C);
    const BF8* gr = reinterpret_cast<const BF8*>(dy + (long long)row * C);
    BF8 xraw[NV], graw[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      xraw[j] = xr[lane + 32 * j];
      graw[j] = gr[lane + 32 * j];
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float xv[8], dv[8];
      unpack8(xraw[j], xv);
      unpack8(graw[j], dv);
      const float* sc = scale + (lane + 32 * j) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = xv[i] * rstd;
        ds[j][i] += dv[i] * xh;
        dot += dv[i] * sc[i] * xh;
      }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
    const float mean = dot / C;
    BF8* dr = reinterpret_cast<BF8*>(dx + (long long)row * C);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float xv[8], dv[8], o[8];
      unpack8(xraw[j], xv);
      unpack8(graw[j], dv);
      const float* sc = scale + (lane + 32 * j) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = (dv[i] * sc[i] - xv[i] * rstd * mean) * rstd;
      dr[lane + 32 * j] = pack8(o);
    }
  }
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    float* out = partial + (long long)warp * C + (lane + 32 * j) * 8;
    reinterpret_cast<float4*>(out)[0] = make_float4(ds[j][0], ds[j][1], ds[j][2], ds[j][3]);
    reinterpret_cast<float4*>(out)[1] = make_float4(ds[j][4], ds[j][5], ds[j][6], ds[j][7]);
  }
}

// ------------------------------------------------------------------------------------------------ SwiGLU
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// `rows_dev` (optional): device-resident number of leading rows that hold data; rows beyond it are left untouched (the
// expert-parallel receive buffers are sized for the worst case and mostly empty).
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ pre, __nv_bfloat16* __restrict__ out, long long M, int H, float beta, float limit,
                                  const int* __restrict__ rows_dev) {
  const int hv = H / 8;
  if (rows_dev) M = min(M, (long long)*rows_dev);
  const long long total = M * hv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / hv;
    const int c = int(i % hv);
    float g[8], l[8], o[8];
    unpack8(reinterpret_cast<const BF8*>(pre + m * 2 * H)[c], g);
    unpack8(reinterpret_cast<const BF8*>(pre + m * 2 * H + H)[c], l);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gc = fminf(g[k], limit), lc = fminf(fmaxf(l[k], -limit), limit);
      o[k] = (lc + 1.f) * gc * sigmoidf_(beta * gc);
    }
    reinterpret_cast<BF8*>(out + m * H)[c] = pack8(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ pre, const __nv_bfloat16* __restrict__ dact, __nv_bfloat16* __restrict__ dpre,
                                  long long M, int H, float beta, float limit, const int* __restrict__ rows_dev) {
  const int hv = H / 8;
  if (rows_dev) M = min(M, (long long)*rows_dev);
  const long long total = M * hv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / hv;
    const int c = int(i % hv);
    float g[8], l[8], d[8], dg[8], dl[8];
    unpack8(reinterpret_cast<const BF8*>(pre + m * 2 * H)[c], g);
    unpack8(reinterpret_cast<const BF8*>(pre + m * 2 * H + H)[c], l);
    unpack8(reinterpret_cast<const BF8*>(dact + m * H)[c], d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gc = fminf(g[k], limit), lc = fminf(fmaxf(l[k], -limit), limit);
      const float s = sigmoidf_(beta * gc);
      dg[k] = g[k] <= limit ? d[k] * (lc + 1.f) * (s + gc * beta * s * (1.f - s)) : 0.f;
      dl[k] = (l[k] >= -limit && l[k] <= limit) ? d[k] * gc * s : 0.f;
    }
    reinterpret_cast<BF8*>(dpre + m * 2 * H)[c] = pack8(dg);
    reinterpret_cast<BF8*>(dpre + m * 2 * H + H)[c] = pack8(dl);
  }
}

// ------------------------------------------------------------------------------------------------ QK-norm + RoPE (forward)
// x, y [rows = B*T*N, D]; one warp per row; cos/sin [T, D/2]. Optional RMS norm over D with `scale`. The N heads of a token are
// contiguous in x and consecutive tokens are `x_token_stride` elements apart (N * D for a tensor of its own, more for a slice
// of a fused q | k | v projection); y is contiguous.
__global__ void qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale, const float* __restrict__ cosv,
                                       const float* __restrict__ sinv, __nv_bfloat16* __restrict__ y, long long rows, int T, int N, int D, float eps,
                                       long long x_token_stride) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int t = int((row / N) % T);
  const int half = D / 2;
  const __nv_bfloat16* xr = x + (row / N) * x_token_stride + (row % N) * D;
  float a[2], b[2];  // elements lane, lane+32 of each half (D <= 128)
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int i = lane + j * 32;
    a[j] = i < half ? __bfloat162float(xr[i]) : 0.f;
    b[j] = i < half ? __bfloat162float(xr[i + half]) : 0.f;
    ss += a[j] * a[j] + b[j] * b[j];
  }
  float rstd = 1.f;
  if (scale) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
    rstd = rsqrtf(ss / D + eps);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int i = lane + j * 32;
    if (i < half) {
      // the normalised value is rounded to bf16 before the rotation, as in the unfused composition
      float x1 = a[j] * rstd, x2 = b[j] * rstd;
      if (scale) {
        x1 = __bfloat162float(__float2bfloat16(x1 * scale[i]));
        x2 = __bfloat162float(__float2bfloat16(x2 * scale[i + half]));
      }
      const float c = cosv[(long long)t * half + i], s = sinv[(long long)t * half + i];
      y[row * D + i] = __float2bfloat16(x1 * c - x2 * s);
      y[row * D + i + half] = __float2bfloat16(x2 * c + x1 * s);
    }
  }
}

// ------------------------------------------------------------------------------------------------ MoE row movement
// out[dest[f*K + k]] = xn[f]; one block per token.
__global__ void scatter_rows_kernel(const __nv_bfloat16* __restrict__ xn, const long long* __restrict__ dest, __nv_bfloat16* __restrict__ out,
                                    int F, int K, int C) {
  const int f = blockIdx.x;
  const int nvec = C / 8;
  const BF8* src = reinterpret_cast<const BF8*>(xn + (long long)f * C);
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    const BF8 v = src[c];
    for (int k = 0; k < K; ++k) reinterpret_cast<BF8*>(out + dest[(long long)f * K + k] * C)[c] = v;
  }
}

// out[f] = sum_k scores[f,k] * rows[dest[f*K + k]]  (fp32 accumulate, k ascending)
__global__ void combine_rows_kernel(const __nv_bfloat16* __restrict__ rows, const long long* __restrict__ dest, const float* __restrict__ scores,
                                    __nv_bfloat16* __restrict__ out, int F, int K, int C) {
  const int f = blockIdx.x;
  const int nvec = C / 8;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < K; ++k) {
      float v[8];
      unpack8(reinterpret_cast<const BF8*>(rows + dest[(long long)f * K + k] * C)[c], v);
      const float s = scores[(long long)f * K + k];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += s * v[i];
    }
    reinterpret_cast<BF8*>(out + (long long)f * C)[c] = pack8(acc);
  }
}

// d_rows[dest[f*K+k]] = scores[f,k] * dout[f];  dscores[f,k] = <rows[dest[f*K+k]], dout[f]>
__global__ void __launch_bounds__(256) combine_rows_bwd_kernel(const __nv_bfloat16* __restrict__ rows, const __nv_bfloat16* __restrict__ dout,
                                                               const long long* __restrict__ dest, const float* __restrict__ scores,
                                                               __nv_bfloat16* __restrict__ d_rows, float* __restrict__ dscores, int F, int K, int C) {
  __shared__ float red[8];
  const int f = blockIdx.x;
  const int nvec = C / 8;
  for (int k = 0; k < K; ++k) {
    const long long r = dest[(long long)f * K + k];
    const float s = scores[(long long)f * K + k];
    float dot = 0.f;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float g[8], v[8], o[8];
      unpack8(reinterpret_cast<const BF8*>(dout + (long long)f * C)[c], g);
      unpack8(reinterpret_cast<const BF8*>(rows + r * C)[c], v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dot += g[i] * v[i];
        o[i] = s * g[i];
      }
      reinterpret_cast<BF8*>(d_rows + r * C)[c] = pack8(o);
    }
    const float total = block_sum(dot, red);
    if (threadIdx.x == 0) dscores[(long long)f * K + k] = total;
  }
}

// Deterministic embedding gradient (sorted segment-sum, lyra/kernels/embs.py:22-29): positions are sorted by token id;
// the block at the first position of each run of equal ids sums the run's gradient rows in order (fp32) and adds the
// sum into that id's row of the gradient buffer. One writer per row: no atomics, fixed summation order.
template <typename G>
__global__ void embedding_grad_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ order,
                                      const __nv_bfloat16* __restrict__ g, G* __restrict__ grad, int F, int C) {
  const int i = blockIdx.x;
  const long long id = sorted_ids[i];
  if (i > 0 && sorted_ids[i - 1] == id) return;
  int end = i + 1;
  while (end < F && sorted_ids[end] == id) ++end;
  for (int c = threadIdx.x; c < C / 8; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = i; j < end; ++j) {
      float v[8];
      unpack8(reinterpret_cast<const BF8*>(g + order[j] * C)[c], v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += v[k];
    }
    G* dst = grad + id * C + c * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) dst[k] = G(float(dst[k]) + acc[k]);
  }
}

static inline int ew_grid(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 32;
  return int(b < cap ? (b > 0 ? b : 1) : cap);
}

}  // namespace lyra

using namespace lyra;
#define S_(x) reinterpret_cast<cudaStream_t>(x)
#define BFP(x) reinterpret_cast<__nv_bfloat16*>(x)
#define CBFP(x) reinterpret_cast<const __nv_bfloat16*>(x)

extern "C" int lyra_rmsnorm_fwd(const void* x, const float* scale, void* y, float* rstd, int rows, int C, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (C % 8 || C > 8 * RN_THREADS * RN_MAXV) return -40;
  if (C % 256 == 0 && C <= 4096 && (reinterpret_cast<uintptr_t>(scale) & 15) == 0) {   // warp-per-row kernels
    const int blocks = (rows + 7) / 8 < sm_count() * 8 ? (rows + 7) / 8 : sm_count() * 8;
    switch (C / 256) {
      case 1: rmsnorm_fwd_warp_kernel<1><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, BFP(y), rstd, rows, eps); break;
      case 2: rmsnorm_fwd_warp_kernel<2><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, BFP(y), rstd, rows, eps); break;
      case 4: rmsnorm_fwd_warp_kernel<4><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, BFP(y), rstd, rows, eps); break;
      case 8: rmsnorm_fwd_warp_kernel<8><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, BFP(y), rstd, rows, eps); break;
      case 16: rmsnorm_fwd_warp_kernel<16><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, BFP(y), rstd, rows, eps); break;
      default: goto block_kernel;
    }
    LYRA_CHECK_LAUNCH();
    return 0;
  }
block_kernel:
  const int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
  rmsnorm_fwd_kernel<<<grid, RN_THREADS, 0, S_(stream)>>>(CBFP(x), scale, BFP(y), rstd, rows, C, eps);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_rmsnorm_bwd(const void* x, const float* scale, const float* rstd, const void* dy, void* dx, float* partial, int rows, int C,
                                int nblk, void* stream) {
  if (rows <= 0) return 0;
  if (C % 8 || C > 8 * RN_THREADS * RN_MAXV) return -40;
  if (C % 256 == 0 && C <= 2048) {   // warp-per-row kernel: `nblk` rows of `partial` = `nblk` warps
    const int blocks = (nblk + 7) / 8;
    switch (C / 256) {
      case 1: rmsnorm_bwd_warp_kernel<1><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, rstd, CBFP(dy), BFP(dx), partial, rows, nblk); break;
      case 2: rmsnorm_bwd_warp_kernel<2><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, rstd, CBFP(dy), BFP(dx), partial, rows, nblk); break;
      case 4: rmsnorm_bwd_warp_kernel<4><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, rstd, CBFP(dy), BFP(dx), partial, rows, nblk); break;
      case 8: rmsnorm_bwd_warp_kernel<8><<<blocks, 256, 0, S_(stream)>>>(CBFP(x), scale, rstd, CBFP(dy), BFP(dx), partial, rows, nblk); break;
      default: goto block_kernel;
    }
    LYRA_CHECK_LAUNCH();
    return 0;
  }
block_kernel:
  rmsnorm_bwd_kernel<<<nblk, RN_THREADS, 0, S_(stream)>>>(CBFP(x), scale, rstd, CBFP(dy), BFP(dx), partial, rows, C);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_swiglu_fwd(const void* pre, void* out, long long M, int H, float beta, float limit, void* stream) {
  if (M <= 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(M * (H / 8), 256), 256, 0, S_(stream)>>>(CBFP(pre), BFP(out), M, H, beta, limit, nullptr);
  LYRA_CHECK_LAUNCH();
  return 0;
}

// As above for the first *rows_dev rows only (rows_dev: int32 on the device, read by the kernel).
extern "C" int lyra_swiglu_fwd_rows(const void* pre, void* out, long long M, int H, float beta, float limit, const int* rows_dev, void* stream) {
  if (M <= 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(M * (H / 8), 256), 256, 0, S_(stream)>>>(CBFP(pre), BFP(out), M, H, beta, limit, rows_dev);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_swiglu_bwd(const void* pre, const void* dact, void* dpre, long long M, int H, float beta, float limit, void* stream) {
  if (M <= 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(M * (H / 8), 256), 256, 0, S_(stream)>>>(CBFP(pre), CBFP(dact), BFP(dpre), M, H, beta, limit, nullptr);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_swiglu_bwd_rows(const void* pre, const void* dact, void* dpre, long long M, int H, float beta, float limit, const int* rows_dev,
                                    void* stream) {
  if (M <= 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(M * (H / 8), 256), 256, 0, S_(stream)>>>(CBFP(pre), CBFP(dact), BFP(dpre), M, H, beta, limit, rows_dev);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_qknorm_rope_fwd(const void* x, const float* scale, const float* cosv, const float* sinv, void* y, int B, int T, int N, int D,
                                    float eps, long long x_token_stride, void* stream) {
  const long long rows = (long long)B * T * N;
  if (rows <= 0) return 0;
  if (D > 128 || D % 2 || x_token_stride < (long long)N * D) return -41;
  qknorm_rope_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, S_(stream)>>>(CBFP(x), scale, cosv, sinv, BFP(y), rows, T, N, D, eps, x_token_stride);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_scatter_rows(const void* xn, const long long* dest, void* out, int F, int K, int C, void* stream) {
  if (F <= 0) return 0;
  if (C % 8) return -42;
  scatter_rows_kernel<<<F, 128, 0, S_(stream)>>>(CBFP(xn), dest, BFP(out), F, K, C);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_combine_rows(const void* rows, const long long* dest, const float* scores, void* out, int F, int K, int C, void* stream) {
  if (F <= 0) return 0;
  if (C % 8) return -42;
  combine_rows_kernel<<<F, 128, 0, S_(stream)>>>(CBFP(rows), dest, scores, BFP(out), F, K, C);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_combine_rows_bwd(const void* rows, const void* dout, const long long* dest, const float* scores, void* d_rows, float* dscores,
                                     int F, int K, int C, void* stream) {
  if (F <= 0) return 0;
  if (C % 8) return -42;
  combine_rows_bwd_kernel<<<F, 256, 0, S_(stream)>>>(CBFP(rows), CBFP(dout), dest, scores, BFP(d_rows), dscores, F, K, C);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_embedding_grad(const long long* sorted_ids, const long long* order, const void* g, void* grad, int grad_bf16, int F, int C,
                                   void* stream) {
  if (F <= 0) return 0;
  if (C % 8) return -42;
  if (grad_bf16) embedding_grad_kernel<__nv_bfloat16><<<F, 128, 0, S_(stream)>>>(sorted_ids, order, CBFP(g), BFP(grad), F, C);
  else embedding_grad_kernel<float><<<F, 128, 0, S_(stream)>>>(sorted_ids, order, CBFP(g), reinterpret_cast<float*>(grad), F, C);
  LYRA_CHECK_LAUNCH();
  return 0;
}
