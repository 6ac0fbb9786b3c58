// Routing of a mixture-of-experts layer after the fp32 router product (lyra/model.py:418-491 in the reference, where it is a
// chain of XLA ops): top-k over the routed experts, softmax over the selected logits, the two auxiliary-loss terms, per-expert
// counts and the stable expert-sorted permutation of the assignments - three launches instead of some fifteen framework ops,
// and every reduction in a fixed order (no floating-point atomics), so two runs give the same bits.
//
//   route_kernel        one warp per token: log-sum-exp and softmax of the row, k rounds of warp arg-max (ties: lower expert
//                       first, like lax.top_k), scores = softmax over the selected logits; per block of 32 tokens: column sums
//                       of the softmax, sum of lse^2, per-expert counts and every assignment's rank among the block's
//                       earlier assignments to the same expert
//   route_finish_kernel one block: totals over blocks (in block order), exclusive prefixes per expert over blocks and over
//                       experts, aux = lb_weight * E * sum_e mean_softmax_e * count_e / (F k) + z_weight * mean(lse^2)
//   route_scatter_kernel order[start_e + rank] = assignment: the counting-sort permutation (token order kept inside an expert)
//   route_bwd_kernel    one warp per token: gradient of the logits from the gradients of the scores and of the aux loss
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../common/tmap.h"

namespace {

constexpr int ROWS_PER_BLOCK = 32;
constexpr int WARPS = 8;
constexpr int MAX_EXPERTS = 256;   // routed experts (8 per lane)
constexpr int MAX_K = 8;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int EPL>   // experts per lane: expert e lives in lane e % 32, slot e / 32
__global__ void __launch_bounds__(WARPS * 32) route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int F, int Er, int k,
                                                           long long* __restrict__ idx, float* __restrict__ scores, float* __restrict__ lse_out,
                                                           float* __restrict__ part_colsum, float* __restrict__ part_z, int* __restrict__ block_counts,
                                                           int* __restrict__ local_rank) {
  __shared__ float colsum_s[WARPS][MAX_EXPERTS];
  __shared__ float z_s[WARPS];
  __shared__ int sel_s[ROWS_PER_BLOCK * MAX_K];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * ROWS_PER_BLOCK;
  float colsum[EPL];
#pragma unroll
  for (int s = 0; s < EPL; ++s) colsum[s] = 0.f;
  float zsum = 0.f;
  for (int r = warp; r < ROWS_PER_BLOCK; r += WARPS) {
    const int f = row0 + r;
    if (f >= F) {
      for (int j = lane; j < k; j += 32) sel_s[r * MAX_K + j] = -1;
      continue;
    }
    float v[EPL];
    float mx = -INFINITY;
#pragma unroll
    for (int s = 0; s < EPL; ++s) {
      const int e = s * 32 + lane;
      v[s] = e < Er ? logits[(long long)f * Er + e] + (bias ? bias[e] : 0.f) : -INFINITY;
      mx = fmaxf(mx, v[s]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < EPL; ++s) sum += (s * 32 + lane < Er) ? expf(v[s] - mx) : 0.f;
    sum = warp_sum(sum);
    const float lse = mx + logf(sum);
    if (lane == 0) lse_out[f] = lse;
    zsum += lse * lse;   // same value in every lane
#pragma unroll
    for (int s = 0; s < EPL; ++s)
      if (s * 32 + lane < Er) colsum[s] += expf(v[s] - lse);
    // top-k by repeated arg-max
    float top_v[MAX_K];
    int top_e[MAX_K];
#pragma unroll
    for (int j = 0; j < MAX_K; ++j) {
      if (j < k) {
        float bv = -INFINITY;
        int be = 0x7fffffff;
#pragma unroll
        for (int s = 0; s < EPL; ++s) {
          const int e = s * 32 + lane;
          if (e < Er && (v[s] > bv || (v[s] == bv && e < be))) { bv = v[s]; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
          const int oe = __shfl_xor_sync(0xffffffffu, be, o);
          if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        top_v[j] = bv;
        top_e[j] = be;
#pragma unroll
        for (int s = 0; s < EPL; ++s)
          if (s * 32 + lane == be) v[s] = -INFINITY;
      }
    }
    // softmax over the selected logits (top_v[0] is their maximum)
    float den = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_K; ++j)
      if (j < k) den += expf(top_v[j] - top_v[0]);
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < MAX_K; ++j) {
        if (j < k) {
          idx[(long long)f * k + j] = top_e[j];
          scores[(long long)f * k + j] = expf(top_v[j] - top_v[0]) / den;
          sel_s[r * MAX_K + j] = top_e[j];
        }
      }
    }
  }
#pragma unroll
  for (int s = 0; s < EPL; ++s) colsum_s[warp][s * 32 + lane] = colsum[s];
  if (lane == 0) z_s[warp] = zsum;
  __syncthreads();
  // one thread per expert: fixed-order sums over the warps, then the block's assignments in token order
  for (int e = threadIdx.x; e < Er; e += blockDim.x) {
    float c = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) c += colsum_s[w][e];
    part_colsum[(long long)blockIdx.x * Er + e] = c;
    int n = 0;
    for (int r = 0; r < ROWS_PER_BLOCK; ++r) {
      for (int j = 0; j < k; ++j) {
        if (sel_s[r * MAX_K + j] == e) {
          local_rank[(long long)(row0 + r) * k + j] = n;
          ++n;
        }
      }
    }
    block_counts[(long long)blockIdx.x * Er + e] = n;
  }
  if (threadIdx.x == 0) {
    float z = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) z += z_s[w];
    part_z[blockIdx.x] = z;
  }
}

// One block. block_base[b][e] = assignments to expert e in blocks before b; counts[e]; starts[e] exclusive prefix over experts
// (starts[Er] = F * k); aux loss.
__global__ void route_finish_kernel(const float* __restrict__ part_colsum, const float* __restrict__ part_z, int* __restrict__ block_counts,
                                    int n_blocks, int F, int Er, int k, float lb_weight, float z_weight, int* __restrict__ counts,
                                    int* __restrict__ starts, float* __restrict__ aux) {
  __shared__ float lb_s[MAX_EXPERTS];
  __shared__ int cnt_s[MAX_EXPERTS];
  for (int e = threadIdx.x; e < Er; e += blockDim.x) {
    float c = 0.f;
    int run = 0;
    for (int b = 0; b < n_blocks; ++b) {
      c += part_colsum[(long long)b * Er + e];
      const int n = block_counts[(long long)b * Er + e];
      block_counts[(long long)b * Er + e] = run;   // becomes the exclusive prefix over blocks
      run += n;
    }
    counts[e] = run;
    cnt_s[e] = run;
    lb_s[e] = (c / F) * (float(run) / (float(F) * k));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    float lb = 0.f;
    for (int e = 0; e < Er; ++e) {
      starts[e] = run;
      run += cnt_s[e];
      lb += lb_s[e];
    }
    starts[Er] = run;
    float z = 0.f;
    for (int b = 0; b < n_blocks; ++b) z += part_z[b];
    aux[0] = lb_weight * Er * lb + z_weight * (z / F);
  }
}

__global__ void route_scatter_kernel(const long long* __restrict__ idx, const int* __restrict__ local_rank, const int* __restrict__ block_base,
                                     const int* __restrict__ starts, int A, int Er, int k, int* __restrict__ order, int* __restrict__ rank_in_expert) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= A) return;
  const int e = int(idx[a]);
  const int b = (a / k) / ROWS_PER_BLOCK;
  const int r = block_base[(long long)b * Er + e] + local_rank[a];
  rank_in_expert[a] = r;
  order[starts[e] + r] = a;
}

// d_logits[f, e] = d_aux * (lb_weight * E / F * p_e * (c_e - sum_e' c_e' p_e') + z_weight * 2 lse / F * p_e)
//                  + [e selected as j] s_j (ds_j - sum_i s_i ds_i),     p = softmax(logits + bias), c_e = counts_e / (F k)
template <int EPL>
__global__ void __launch_bounds__(WARPS * 32) route_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                               const float* __restrict__ lse, const long long* __restrict__ idx,
                                                               const float* __restrict__ scores, const float* __restrict__ dscores,
                                                               const int* __restrict__ counts, const float* __restrict__ d_aux, int F, int Er, int k,
                                                               float lb_weight, float z_weight, float* __restrict__ d_logits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f = blockIdx.x * WARPS + warp;
  if (f >= F) return;
  const float ga = d_aux ? d_aux[0] : 0.f;
  const float l = lse[f];
  float p[EPL], c[EPL];
  float dot = 0.f;
#pragma unroll
  for (int s = 0; s < EPL; ++s) {
    const int e = s * 32 + lane;
    p[s] = e < Er ? expf(logits[(long long)f * Er + e] + (bias ? bias[e] : 0.f) - l) : 0.f;
    c[s] = e < Er ? float(counts[e]) / (float(F) * k) : 0.f;
    dot += c[s] * p[s];
  }
  dot = warp_sum(dot);
  float t = 0.f;
  for (int j = 0; j < k; ++j) t += scores[(long long)f * k + j] * (dscores ? dscores[(long long)f * k + j] : 0.f);
#pragma unroll
  for (int s = 0; s < EPL; ++s) {
    const int e = s * 32 + lane;
    if (e >= Er) continue;
    float g = ga * (lb_weight * Er / F * p[s] * (c[s] - dot) + z_weight * 2.f * l / F * p[s]);
    for (int j = 0; j < k; ++j)
      if (int(idx[(long long)f * k + j]) == e) g += scores[(long long)f * k + j] * ((dscores ? dscores[(long long)f * k + j] : 0.f) - t);
    d_logits[(long long)f * Er + e] = g;
  }
}

}  // namespace

#define ST(x) reinterpret_cast<cudaStream_t>(x)

// logits [F, Er] fp32 (bias [Er] optional, added here). Outputs: idx [F, k] int64, scores [F, k], lse [F], counts [Er], starts [Er + 1],
// order [F k] (expert-sorted assignment ids, token order inside an expert), rank_in_expert [F k], aux [1].
// Scratch: part_colsum [nb, Er] fp32, part_z [nb] fp32, block_counts [nb, Er] int32, local_rank [F k] int32 with nb = ceil(F / 32).
extern "C" int lyra_route(const float* logits, const float* bias, int F, int Er, int k, float lb_weight, float z_weight, long long* idx, float* scores,
                          float* lse, int* counts, int* starts, int* order, int* rank_in_expert, float* aux, float* part_colsum, float* part_z,
                          int* block_counts, int* local_rank, void* stream) {
  if (F <= 0) return 0;
  if (Er < 1 || Er > MAX_EXPERTS || k < 1 || k > MAX_K || k > Er) return -60;
  const int nb = (F + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
  const int epl = (Er + 31) / 32;
#define LAUNCH_ROUTE(E_)                                                                                                                   \
  route_kernel<E_><<<nb, WARPS * 32, 0, ST(stream)>>>(logits, bias, F, Er, k, idx, scores, lse, part_colsum, part_z, block_counts, local_rank)
  if (epl <= 1) LAUNCH_ROUTE(1);
  else if (epl <= 2) LAUNCH_ROUTE(2);
  else if (epl <= 4) LAUNCH_ROUTE(4);
  else LAUNCH_ROUTE(8);
#undef LAUNCH_ROUTE
  LYRA_CHECK_LAUNCH();
  route_finish_kernel<<<1, 256, 0, ST(stream)>>>(part_colsum, part_z, block_counts, nb, F, Er, k, lb_weight, z_weight, counts, starts, aux);
  LYRA_CHECK_LAUNCH();
  const int A = F * k;
  route_scatter_kernel<<<(A + 255) / 256, 256, 0, ST(stream)>>>(idx, local_rank, block_counts, starts, A, Er, k, order, rank_in_expert);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_route_bwd(const float* logits, const float* bias, const float* lse, const long long* idx, const float* scores, const float* dscores,
                              const int* counts, const float* d_aux, int F, int Er, int k, float lb_weight, float z_weight, float* d_logits,
                              void* stream) {
  if (F <= 0) return 0;
  if (Er < 1 || Er > MAX_EXPERTS || k < 1 || k > MAX_K) return -60;
  const int epl = (Er + 31) / 32;
  const int grid = (F + WARPS - 1) / WARPS;
#define LAUNCH_BWD(E_)                                                                                                                      \
  route_bwd_kernel<E_><<<grid, WARPS * 32, 0, ST(stream)>>>(logits, bias, lse, idx, scores, dscores, counts, d_aux, F, Er, k, lb_weight, z_weight, \
                                                             d_logits)
  if (epl <= 1) LAUNCH_BWD(1);
  else if (epl <= 2) LAUNCH_BWD(2);
  else if (epl <= 4) LAUNCH_BWD(4);
  else LAUNCH_BWD(8);
#undef LAUNCH_BWD
  LYRA_CHECK_LAUNCH();
  return 0;
}

// Rows of x in expert order for a handful of tokens: sorted position p takes the row of token order[p] / k, and the inverse
// permutation dest[order[p]] = p is written on the way (it is what the weighted combine gathers by). One block per position.
namespace {
__global__ void gather_by_plan_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ order, int k, int C,
                                      __nv_bfloat16* __restrict__ out, long long* __restrict__ dest) {
  const int pos = blockIdx.x;
  const int a = order[pos];
  if (threadIdx.x == 0) dest[a] = pos;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(a / k) * C);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(pos) * C);
  for (int i = threadIdx.x; i < C / 8; i += blockDim.x) dst[i] = src[i];
}
}  // namespace

// x [F, C] bf16 (C a multiple of 8), order [A] int32 with A = F k -> out [A, C] bf16, dest [A] int64
extern "C" int lyra_gather_by_plan(const void* x, const int* order, int A, int k, int C, void* out, long long* dest, void* stream) {
  if (A <= 0) return 0;
  if (C % 8 || k < 1) return -61;
  gather_by_plan_kernel<<<A, 128, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(x), order, k, C, reinterpret_cast<__nv_bfloat16*>(out), dest);
  LYRA_CHECK_LAUNCH();
  return 0;
}
