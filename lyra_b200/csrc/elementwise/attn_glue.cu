// Fused glue around the attention kernel, forward and backward, one warp per row, deterministic reductions:
//   * per-head QK RMS-norm + half-split RoPE              (lyra/model.py:315-323, 183-191)
//   * SDPA output gate t *= 2*sigmoid(logit) followed by tanh-XSA t -= tanh(alpha_h) (t . v_hat) v_hat
//     with v_hat the token's own unit value vector shared by the GQA group (lyra/model.py:343-360)
// Tensors are token-major [B, T, N, D] bf16, D in {64, 128}. Parameter gradients (norm scale, alpha) are written as
// per-block partial sums that the caller adds up.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/tmap.h"

namespace lyra {

constexpr int GL_WARPS = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// ------------------------------------------------------------------------------------------------ QK-norm + RoPE backward
// rows = B*T*N; lane owns elements {lane, lane+32} of each half (half = D/2 <= 64).
// dy -> dx; dscale partial [gridDim.x, D] (only when scale != nullptr).
template <int D>
__global__ void __launch_bounds__(GL_WARPS * 32) qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                                                                         const float* __restrict__ cosv, const float* __restrict__ sinv,
                                                                         const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                                                                         float* __restrict__ partial, long long rows, int T, int N, float eps) {
  constexpr int HALF = D / 2, PER = HALF / 32;  // 1 or 2 element pairs per lane
  __shared__ float sh[GL_WARPS][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float ds1[PER], ds2[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) ds1[j] = ds2[j] = 0.f;
  for (long long row = (long long)blockIdx.x * GL_WARPS + warp; row < rows; row += (long long)gridDim.x * GL_WARPS) {
    const int t = int((row / N) % T);
    const __nv_bfloat16* xr = x + row * D;
    const __nv_bfloat16* gr = dy + row * D;
    float x1[PER], x2[PER], g1[PER], g2[PER];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = lane + j * 32;
      x1[j] = __bfloat162float(xr[i]);
      x2[j] = __bfloat162float(xr[i + HALF]);
      ss += x1[j] * x1[j] + x2[j] * x2[j];
      const float d1 = __bfloat162float(gr[i]), d2 = __bfloat162float(gr[i + HALF]);
      const float c = cosv[(long long)t * HALF + i], s = sinv[(long long)t * HALF + i];
      g1[j] = d1 * c + d2 * s;   // transpose of the rotation
      g2[j] = d2 * c - d1 * s;
    }
    if (scale) {
      const float rstd = rsqrtf(warp_sum(ss) / D + eps);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int i = lane + j * 32;
        const float h1 = x1[j] * rstd, h2 = x2[j] * rstd;
        ds1[j] += g1[j] * h1;
        ds2[j] += g2[j] * h2;
        g1[j] *= scale[i];
        g2[j] *= scale[i + HALF];
        dot += g1[j] * h1 + g2[j] * h2;
        x1[j] = h1;
        x2[j] = h2;
      }
      const float mean = warp_sum(dot) / D;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        g1[j] = (g1[j] - x1[j] * mean) * rstd;
        g2[j] = (g2[j] - x2[j] * mean) * rstd;
      }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = lane + j * 32;
      dx[row * D + i] = __float2bfloat16(g1[j]);
      dx[row * D + i + HALF] = __float2bfloat16(g2[j]);
    }
  }
  if (scale) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      sh[warp][lane + j * 32] = ds1[j];
      sh[warp][lane + j * 32 + HALF] = ds2[j];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      float t = 0.f;
      for (int w = 0; w < GL_WARPS; ++w) t += sh[w][c];
      partial[(long long)blockIdx.x * D + c] = t;
    }
  }
}

// ------------------------------------------------------------------------------------------------ gate + XSA
// One warp per (token, kv head); it walks the `rep` query heads of the group. PER = D/32 elements per lane.
// logits [B*T, Nq] bf16 (nullptr: no gate); alpha [Nq] fp32 (nullptr: no XSA).
template <int D>
__global__ void __launch_bounds__(GL_WARPS * 32) gate_xsa_fwd_kernel(const __nv_bfloat16* __restrict__ t, const __nv_bfloat16* __restrict__ logits,
                                                                      const __nv_bfloat16* __restrict__ v, const float* __restrict__ alpha,
                                                                      __nv_bfloat16* __restrict__ out, long long groups, int Nq, int Nkv) {
  constexpr int PER = D / 32;
  const int rep = Nq / Nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long grp = (long long)blockIdx.x * GL_WARPS + warp; grp < groups; grp += (long long)gridDim.x * GL_WARPS) {
    const long long tok = grp / Nkv;
    const int kvh = int(grp % Nkv);
    float vn[PER];
    if (alpha) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        vn[j] = __bfloat162float(v[(tok * Nkv + kvh) * D + lane + j * 32]);
        ss += vn[j] * vn[j];
      }
      const float r = rsqrtf(warp_sum(ss) + 1e-10f);
#pragma unroll
      for (int j = 0; j < PER; ++j) vn[j] = bf16_round(vn[j] * r);
    }
    for (int q = 0; q < rep; ++q) {
      const int h = kvh * rep + q;
      const long long base = (tok * Nq + h) * D;
      float g = 1.f;
      if (logits) g = bf16_round(2.f / (1.f + __expf(-__bfloat162float(logits[tok * Nq + h]))));
      float tg[PER];
      float coef = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        tg[j] = bf16_round(__bfloat162float(t[base + lane + j * 32]) * g);
        if (alpha) coef += tg[j] * vn[j];
      }
      if (alpha) {
        coef = warp_sum(coef);
        const float a = tanhf(alpha[h]);
#pragma unroll
        for (int j = 0; j < PER; ++j) tg[j] -= a * coef * vn[j];
      }
#pragma unroll
      for (int j = 0; j < PER; ++j) out[base + lane + j * 32] = __float2bfloat16(tg[j]);
    }
  }
}

// Backward. d_out -> d_t, d_logits [B*T, Nq] bf16, d_v [B, T, Nkv, D] bf16, alpha partial [gridDim.x, Nq].
template <int D>
__global__ void __launch_bounds__(GL_WARPS * 32) gate_xsa_bwd_kernel(const __nv_bfloat16* __restrict__ t, const __nv_bfloat16* __restrict__ logits,
                                                                      const __nv_bfloat16* __restrict__ v, const float* __restrict__ alpha,
                                                                      const __nv_bfloat16* __restrict__ d_out, __nv_bfloat16* __restrict__ d_t,
                                                                      __nv_bfloat16* __restrict__ d_logits, __nv_bfloat16* __restrict__ d_v,
                                                                      float* __restrict__ alpha_partial, long long groups, int Nq, int Nkv) {
  constexpr int PER = D / 32;
  extern __shared__ float sh_alpha[];  // [GL_WARPS][Nq]
  const int rep = Nq / Nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (alpha) {
    for (int i = threadIdx.x; i < GL_WARPS * Nq; i += blockDim.x) sh_alpha[i] = 0.f;
    __syncthreads();
  }
  for (long long grp = (long long)blockIdx.x * GL_WARPS + warp; grp < groups; grp += (long long)gridDim.x * GL_WARPS) {
    const long long tok = grp / Nkv;
    const int kvh = int(grp % Nkv);
    float vraw[PER], vn[PER], dvn[PER];
    float r = 0.f;
    if (alpha) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        vraw[j] = __bfloat162float(v[(tok * Nkv + kvh) * D + lane + j * 32]);
        ss += vraw[j] * vraw[j];
        dvn[j] = 0.f;
      }
      r = rsqrtf(warp_sum(ss) + 1e-10f);
#pragma unroll
      for (int j = 0; j < PER; ++j) vn[j] = vraw[j] * r;
    }
    for (int q = 0; q < rep; ++q) {
      const int h = kvh * rep + q;
      const long long base = (tok * Nq + h) * D;
      float g = 1.f;
      if (logits) g = 2.f / (1.f + __expf(-__bfloat162float(logits[tok * Nq + h])));
      float traw[PER], dtg[PER];
      float coef = 0.f, dov = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        traw[j] = __bfloat162float(t[base + lane + j * 32]);
        dtg[j] = __bfloat162float(d_out[base + lane + j * 32]);
        if (alpha) {
          coef += traw[j] * g * vn[j];
          dov += dtg[j] * vn[j];
        }
      }
      if (alpha) {
        coef = warp_sum(coef);
        dov = warp_sum(dov);
        const float a = tanhf(alpha[h]);
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          dvn[j] -= a * (coef * dtg[j] + dov * traw[j] * g);   // uses d_out before it is projected
          dtg[j] -= a * dov * vn[j];
        }
        if (lane == 0) sh_alpha[warp * Nq + h] += -coef * dov * (1.f - a * a);
      }
      float dgate = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        dgate += dtg[j] * traw[j];
        d_t[base + lane + j * 32] = __float2bfloat16(dtg[j] * g);
      }
      if (logits) {
        dgate = warp_sum(dgate);
        if (lane == 0) d_logits[tok * Nq + h] = __float2bfloat16(dgate * g * (1.f - 0.5f * g));
      }
    }
    if (alpha) {
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < PER; ++j) dot += dvn[j] * vn[j];
      dot = warp_sum(dot);
#pragma unroll
      for (int j = 0; j < PER; ++j) d_v[(tok * Nkv + kvh) * D + lane + j * 32] = __float2bfloat16(r * (dvn[j] - vn[j] * dot));
    }
  }
  if (alpha) {
    __syncthreads();
    for (int h = threadIdx.x; h < Nq; h += blockDim.x) {
      float s = 0.f;
      for (int w = 0; w < GL_WARPS; ++w) s += sh_alpha[w * Nq + h];
      alpha_partial[(long long)blockIdx.x * Nq + h] = s;
    }
  }
}

static inline int glue_grid(long long rows) {
  long long b = (rows + GL_WARPS - 1) / GL_WARPS;
  const long long cap = (long long)sm_count() * 8;
  return int(b < cap ? (b > 0 ? b : 1) : cap);
}

}  // namespace lyra

using namespace lyra;
#define GS(x) reinterpret_cast<cudaStream_t>(x)
#define GB(x) reinterpret_cast<__nv_bfloat16*>(x)
#define GC(x) reinterpret_cast<const __nv_bfloat16*>(x)

// Returns the number of blocks used (rows of `partial`), or a negative error code.
extern "C" int lyra_qknorm_rope_bwd(const void* x, const float* scale, const float* cosv, const float* sinv, const void* dy, void* dx, float* partial,
                                    int B, int T, int N, int D, float eps, int max_blocks, void* stream) {
  const long long rows = (long long)B * T * N;
  if (rows <= 0) return 0;
  int grid = glue_grid(rows);
  if (grid > max_blocks) grid = max_blocks;
  if (D == 128) qknorm_rope_bwd_kernel<128><<<grid, GL_WARPS * 32, 0, GS(stream)>>>(GC(x), scale, cosv, sinv, GC(dy), GB(dx), partial, rows, T, N, eps);
  else if (D == 64) qknorm_rope_bwd_kernel<64><<<grid, GL_WARPS * 32, 0, GS(stream)>>>(GC(x), scale, cosv, sinv, GC(dy), GB(dx), partial, rows, T, N, eps);
  else return -60;
  if (cudaGetLastError() != cudaSuccess) return -3;
  return grid;
}

extern "C" int lyra_gate_xsa_fwd(const void* t, const void* logits, const void* v, const float* alpha, void* out, long long tokens, int Nq, int Nkv,
                                 int D, void* stream) {
  const long long groups = tokens * Nkv;
  if (groups <= 0) return 0;
  const int grid = glue_grid(groups);
  if (D == 128) gate_xsa_fwd_kernel<128><<<grid, GL_WARPS * 32, 0, GS(stream)>>>(GC(t), GC(logits), GC(v), alpha, GB(out), groups, Nq, Nkv);
  else if (D == 64) gate_xsa_fwd_kernel<64><<<grid, GL_WARPS * 32, 0, GS(stream)>>>(GC(t), GC(logits), GC(v), alpha, GB(out), groups, Nq, Nkv);
  else return -60;
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_gate_xsa_bwd(const void* t, const void* logits, const void* v, const float* alpha, const void* d_out, void* d_t, void* d_logits,
                                 void* d_v, float* alpha_partial, long long tokens, int Nq, int Nkv, int D, int max_blocks, void* stream) {
  const long long groups = tokens * Nkv;
  if (groups <= 0) return 0;
  int grid = glue_grid(groups);
  if (grid > max_blocks) grid = max_blocks;
  const size_t smem = size_t(GL_WARPS) * Nq * sizeof(float);
  if (D == 128)
    gate_xsa_bwd_kernel<128><<<grid, GL_WARPS * 32, smem, GS(stream)>>>(GC(t), GC(logits), GC(v), alpha, GC(d_out), GB(d_t), GB(d_logits), GB(d_v),
                                                                          alpha_partial, groups, Nq, Nkv);
  else if (D == 64)
    gate_xsa_bwd_kernel<64><<<grid, GL_WARPS * 32, smem, GS(stream)>>>(GC(t), GC(logits), GC(v), alpha, GC(d_out), GB(d_t), GB(d_logits), GB(d_v),
                                                                         alpha_partial, groups, Nq, Nkv);
  else return -60;
  if (cudaGetLastError() != cudaSuccess) return -3;
  return grid;
}

// ------------------------------------------------------------------------------------------------ KV cache append (one new position)
// k, v: the new keys and values of one position, [B, Nkv, D] addressed by (batch, head) element strides; caches [B, Nkv, cap, D],
// bf16 or e4m3 with one fp32 scale per (batch, head, position) (the (1, D) block of the cache quantisation, lyra/model.py:221-226;
// same formula as the row quantiser: scale = amax / 448 in IEEE division, values multiplied by the rounded reciprocal). The
// position is read on the device, so the launch is the same for every token of a CUDA-graph decode loop. One warp per
// (batch, head, k | v).
namespace lyra {
template <bool F8>
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, long long ksb, long long ksh,
                                 long long vsb, long long vsh, void* __restrict__ kc, void* __restrict__ vc, float* __restrict__ ks, float* __restrict__ vs, int B, int Nkv,
                                 int cap, int D, const int* __restrict__ pos_dev) {
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= 2 * B * Nkv) return;
  const int which = w & 1, bh = w >> 1, b = bh / Nkv, h = bh % Nkv;
  const int pos = *pos_dev;
  if (pos < 0 || pos >= cap) return;
  const __nv_bfloat16* src = which ? v + b * vsb + h * vsh : k + b * ksb + h * ksh;
  const long long row = (static_cast<long long>(bh) * cap + pos);
  if (!F8) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(which ? vc : kc) + row * D;
    for (int c = lane; c < D; c += 32) dst[c] = src[c];
  } else {
    float amax = 0.f;
    for (int c = lane; c < D; c += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[c])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
    const float inv = __frcp_rn(sc);
    if (lane == 0) (which ? vs : ks)[row] = sc;
    uint8_t* dst = reinterpret_cast<uint8_t*>(which ? vc : kc) + row * D;
    for (int c = lane; c < D; c += 32) {
      const float x = fminf(fmaxf(__fmul_rn(__bfloat162float(src[c]), inv), -448.f), 448.f);
      dst[c] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
    }
  }
}
}  // namespace lyra

extern "C" int lyra_kv_append(const void* k, const void* v, long long ksb, long long ksh, long long vsb, long long vsh, void* kc, void* vc, float* ks, float* vs, int B, int Nkv, int cap,
                              int D, const int* pos_dev, int f8, void* stream) {
  if (B <= 0 || Nkv <= 0) return 0;
  const int warps = 2 * B * Nkv, wpb = 8;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (f8)
    lyra::kv_append_kernel<true><<<(warps + wpb - 1) / wpb, wpb * 32, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(k), reinterpret_cast<const __nv_bfloat16*>(v),
                                                                               ksb, ksh, vsb, vsh, kc, vc, ks, vs, B, Nkv, cap, D, pos_dev);
  else
    lyra::kv_append_kernel<false><<<(warps + wpb - 1) / wpb, wpb * 32, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(k), reinterpret_cast<const __nv_bfloat16*>(v),
                                                                                ksb, ksh, vsb, vsh, kc, vc, ks, vs, B, Nkv, cap, D, pos_dev);
  LYRA_CHECK_LAUNCH();
  return 0;
}
