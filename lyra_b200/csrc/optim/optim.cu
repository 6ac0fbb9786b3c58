// Fused optimizer element kernels (numerics of lyra/training/optimizer.py:129-163).
//
// Every kernel reads a device-side `enabled` flag (1 = gradients finite) instead of a host value, so
// the non-finite-gradient step skip costs no host synchronisation: with enabled == 0 the learning rate
// is 0, momentum / betas are 1 and the gradient counts as 0 - parameters and moments keep their values.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/tmap.h"

namespace lyra {

template <typename G>
__device__ __forceinline__ float load_grad(const G* g, long long i);
template <>
__device__ __forceinline__ float load_grad<float>(const float* g, long long i) { return g[i]; }
template <>
__device__ __forceinline__ float load_grad<__nv_bfloat16>(const __nv_bfloat16* g, long long i) { return __bfloat162float(g[i]); }

// Adam with bias correction, bf16 first moment, fp32 second moment, no weight decay.
// Optionally refreshes the bf16 compute copy of the parameter in the same pass.
template <typename G>
__global__ void adam_kernel(float* __restrict__ p, const G* __restrict__ g, __nv_bfloat16* __restrict__ mu, float* __restrict__ nu,
                            __nv_bfloat16* __restrict__ shadow, long long n, float lr, float b1, float b2, const int* __restrict__ count,
                            float eps, const float* __restrict__ enabled) {
  const float en = *enabled;
  const bool on = en != 0.f;
  const float keep1 = on ? b1 : 1.f, keep2 = on ? b2 : 1.f, lr_e = on ? lr : 0.f;
  const float t = float(*count + 1);
  const float c1 = 1.f / (1.f - powf(b1, t)), c2 = 1.f / (1.f - powf(b2, t));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gv = on ? load_grad<G>(g, i) : 0.f;
    const float m = __bfloat162float(__float2bfloat16(keep1 * __bfloat162float(mu[i]) + (1.f - keep1) * gv));
    const float v = keep2 * nu[i] + (1.f - keep2) * gv * gv;
    mu[i] = __float2bfloat16(m);
    nu[i] = v;
    const float w = p[i] - lr_e * (m * c1) / (sqrtf(v * c2) + eps);
    p[i] = w;
    if (shadow) shadow[i] = __float2bfloat16(w);
  }
}

// Muon parameter update: p <- p - lr * (ns * ns_scale + wd * p), `ns` bf16 in the parameter's own layout.
__global__ void muon_update_kernel(float* __restrict__ p, const __nv_bfloat16* __restrict__ ns, __nv_bfloat16* __restrict__ shadow,
                                   long long n, float lr, float ns_scale, float wd, const float* __restrict__ enabled) {
  const float lr_e = (*enabled != 0.f) ? lr : 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float w0 = p[i];
    const float w = w0 - lr_e * (__bfloat162float(ns[i]) * ns_scale + wd * w0);
    p[i] = w;
    if (shadow) shadow[i] = __float2bfloat16(w);
  }
}

// Muon momentum: m <- momentum * m + g * clip  (fp32 math, stored bf16);  d <- g * clip + nesterov * m  (bf16).
// `clip` holds one factor per matrix; matrix index of element i is (i / inner) % n_mat_mod style via two extents:
// element i belongs to matrix  (i / stride_hi) * mats_lo + (i / stride_lo) % mats_lo  which covers both plain stacks
// ([G, m, n]: mats_lo = 1, stride_hi = m*n) and SwiGLU up-projections ([G, C, 2, H]: mats_lo = 2, stride_lo = H, stride_hi = C*2*H).
template <typename G>
__global__ void muon_moment_kernel(const G* __restrict__ g, __nv_bfloat16* __restrict__ moment, __nv_bfloat16* __restrict__ d,
                                   const float* __restrict__ clip, long long n, long long stride_hi, long long stride_lo, int mats_lo,
                                   float momentum, float nesterov, const float* __restrict__ enabled) {
  const bool on = *enabled != 0.f;
  const float mom = on ? momentum : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long mat = (i / stride_hi) * mats_lo + (mats_lo > 1 ? (i / stride_lo) % mats_lo : 0);
    const float gv = on ? load_grad<G>(g, i) * clip[mat] : 0.f;
    const float m = __bfloat162float(__float2bfloat16(mom * __bfloat162float(moment[i]) + gv));
    moment[i] = __float2bfloat16(m);
    d[i] = __float2bfloat16(nesterov >= 0.f ? gv + nesterov * m : m);
  }
}

static inline int grid_for(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  return int(b < cap ? (b > 0 ? b : 1) : cap);
}

}  // namespace lyra

using namespace lyra;

extern "C" int lyra_adam(float* p, const void* g, int g_bf16, void* mu, float* nu, void* shadow, long long n, float lr, float b1, float b2,
                         const int* count, float eps, const float* enabled, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (g_bf16)
    adam_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, s>>>(p, reinterpret_cast<const __nv_bfloat16*>(g), reinterpret_cast<__nv_bfloat16*>(mu), nu,
                                                           reinterpret_cast<__nv_bfloat16*>(shadow), n, lr, b1, b2, count, eps, enabled);
  else
    adam_kernel<float><<<grid_for(n), 256, 0, s>>>(p, reinterpret_cast<const float*>(g), reinterpret_cast<__nv_bfloat16*>(mu), nu,
                                                   reinterpret_cast<__nv_bfloat16*>(shadow), n, lr, b1, b2, count, eps, enabled);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_muon_update(float* p, const void* ns, void* shadow, long long n, float lr, float ns_scale, float wd, const float* enabled,
                                void* stream) {
  if (n <= 0) return 0;
  muon_update_kernel<<<grid_for(n), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      p, reinterpret_cast<const __nv_bfloat16*>(ns), reinterpret_cast<__nv_bfloat16*>(shadow), n, lr, ns_scale, wd, enabled);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_muon_moment(const void* g, int g_bf16, void* moment, void* d, const float* clip, long long n, long long stride_hi,
                                long long stride_lo, int mats_lo, float momentum, float nesterov, const float* enabled, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (g_bf16)
    muon_moment_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(g), reinterpret_cast<__nv_bfloat16*>(moment),
                                                                  reinterpret_cast<__nv_bfloat16*>(d), clip, n, stride_hi, stride_lo, mats_lo,
                                                                  momentum, nesterov, enabled);
  else
    muon_moment_kernel<float><<<grid_for(n), 256, 0, s>>>(reinterpret_cast<const float*>(g), reinterpret_cast<__nv_bfloat16*>(moment),
                                                          reinterpret_cast<__nv_bfloat16*>(d), clip, n, stride_hi, stride_lo, mats_lo, momentum,
                                                          nesterov, enabled);
  LYRA_CHECK_LAUNCH();
  return 0;
}
