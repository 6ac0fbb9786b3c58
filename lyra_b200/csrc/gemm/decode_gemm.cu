// Small-M (decode) grouped GEMM that streams expert weights once: y[rows of group g] = x[rows] @ W[g]  (+ bias, + SwiGLU).
//
// Role of lyra/kernels/decode_gemm.py:145-365: at decode time each expert sees a handful of rows, so the product is bound
// by reading the weights. Groups without rows are skipped (their CTAs leave at once), weights may be bf16 or e4m3 with
// one fp32 scale per (bk x bn) block (dequantised on the fly: value * scale rounded to bf16, the same numbers as
// dequantise-then-matmul). Unlike the reference kernel there is no K, N % 128 restriction: 64 is enough, so the 2880-wide
// GPT-OSS layers take this path too.
//
// Design: a CTA owns one 64/128/192-column panel of one group's weight matrix (and one K range when the K axis is split so that a
// dense layer still fills 148 SMs); 64-row weight tiles and the matching activation tile arrive through a four-stage
// cp.async ring; four warps each own a quarter of the panel's columns and up to four 16-row blocks of the group (warp-level m16n8k16 MMAs: a
// tcgen05 tile would need M >= 64 rows per expert, which decode does not have; groups with more than 64 rows are covered
// by further CTAs along grid.z). fp32 partials go to a scratch buffer; a finishing kernel sums the K splits, adds the
// bias and applies the clamped SwiGLU.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int TKC = 64, MROWS = 64, NST = 4, THREADS = 128;
constexpr int XROWB = TKC * 2 + 16;        // padded bf16 activation-tile row (ldmatrix rows in distinct banks)
constexpr int XTILE_B = MROWS * XROWB;     // 9216

struct DGParams {
  const __nv_bfloat16* x;   // [R, K], rows sorted by group
  const uint8_t* w;         // [G, K, N] bf16 or e4m3
  const float* wscale;      // [G, K / bk, N / bn]
  const int* offsets;       // [G + 1] row offsets, or null: one group holding all R rows
  const int* counts;        // optional [G]: rows of group g are offsets[g] .. offsets[g] + counts[g] - 1 (padded layouts)
  float* part;              // [splits, R, N]
  int R, K, N, G, splits, k_per_split, bk, bn, zblocks;
};

__device__ __forceinline__ uint32_t s32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, int nbytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(nbytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ uint32_t fp8x2_to_bf16x2(uint16_t two, float scale) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(two, __NV_E4M3);
  float2 f = __half22float2(*reinterpret_cast<__half2*>(&h));
  return pack2(f.x * scale, f.y * scale);
}

// TN = columns per CTA (64, 128 or 192): wider panels read longer contiguous pieces of each weight row.
template <bool FP8, int TN>
struct Geo {
  static constexpr int ROWB = TN * 2 + 16;                     // padded bf16 weight-tile row
  static constexpr int TILE_B = TKC * ROWB;
  static constexpr int WRAW_B = FP8 ? TKC * TN : TILE_B;       // weight tile as it arrives
  static constexpr int STAGE_B = WRAW_B + XTILE_B;             // + activation tile [64 rows][64 k]
  static constexpr int SMEM_B = NST * STAGE_B + (FP8 ? TILE_B : 0);
};

template <bool FP8, int TN>
__global__ void __launch_bounds__(THREADS) decode_gemm_kernel(const DGParams p) {
  using G_ = Geo<FP8, TN>;
  constexpr int ROWB = G_::ROWB;
  constexpr int WN = TN / 4, NT = WN / 8;                       // columns and n8 tiles per warp
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int n0 = blockIdx.x * TN, g = blockIdx.y;
  const int split = blockIdx.z % p.splits, zb = blockIdx.z / p.splits;
  const int gbeg = p.offsets ? p.offsets[g] : 0;
  const int gend = p.offsets ? (p.counts ? gbeg + p.counts[g] : p.offsets[g + 1]) : p.R;
  const int r0 = gbeg + zb * MROWS;
  if (r0 >= gend) return;                                        // group without rows (or fewer than this block covers)
  const int cnt = min(MROWS, gend - r0);
  const int n_mt = (cnt + 15) >> 4;
  const int kbeg = split * p.k_per_split, kend = min(p.K, kbeg + p.k_per_split);
  const int nchunks = (kend - kbeg) / TKC;
  constexpr int ESZ = FP8 ? 1 : 2;
  const uint8_t* wg = p.w + (static_cast<size_t>(g) * p.K * p.N + n0) * ESZ;

  auto issue = [&](int c) {
    uint8_t* st = smem + (c % NST) * G_::STAGE_B;
    const int k0 = kbeg + c * TKC;
    constexpr int WCPR = TN * ESZ / 16;                          // 16-byte chunks per weight-tile row
    constexpr int WROW = FP8 ? TN : ROWB;
#pragma unroll
    for (int j = 0; j < TKC * WCPR / THREADS; ++j) {
      const int ch = tid + THREADS * j, row = ch / WCPR, col = ch % WCPR;
      cp16(s32(st + row * WROW + col * 16), wg + static_cast<size_t>(k0 + row) * p.N * ESZ + col * 16, 16);
    }
    uint8_t* xt = st + G_::WRAW_B;
#pragma unroll
    for (int j = 0; j < MROWS * 8 / THREADS; ++j) {
      const int ch = tid + THREADS * j, row = ch >> 3, col = ch & 7;
      const bool ok = row < cnt;
      cp16(s32(xt + row * XROWB + col * 16), p.x + static_cast<size_t>(r0 + (ok ? row : 0)) * p.K + k0 + col * 8, ok ? 16 : 0);
    }
  };

  float acc[4][NT][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < NT; ++b) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.f;

#pragma unroll
  for (int s = 0; s < NST - 1; ++s) {
    if (s < nchunks) issue(s);
    cp_commit();
  }
  for (int c = 0; c < nchunks; ++c) {
    cp_wait<NST - 2>();
    __syncthreads();                       // chunk c has landed for everyone, and everyone is done with chunk c - 1
    if (c + NST - 1 < nchunks) issue(c + NST - 1);
    cp_commit();
    uint8_t* st = smem + (c % NST) * G_::STAGE_B;
    uint8_t* wt = st;
    const uint8_t* xt = st + G_::WRAW_B;
    if (FP8) {
      wt = smem + NST * G_::STAGE_B;
      const int k0 = kbeg + c * TKC;
      const float* srow = p.wscale + (static_cast<size_t>(g) * (p.K / p.bk) + k0 / p.bk) * (p.N / p.bn);
      constexpr int CPR = TN / 16;
#pragma unroll
      for (int j = 0; j < TKC * CPR / THREADS; ++j) {
        const int ch = tid + THREADS * j, row = ch / CPR, col = ch % CPR;
        const float sc = srow[(n0 + col * 16) / p.bn];
        const uint4 raw = *reinterpret_cast<const uint4*>(st + row * TN + col * 16);
        const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t o[8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          o[2 * u] = fp8x2_to_bf16x2(static_cast<uint16_t>(w4[u] & 0xffffu), sc);
          o[2 * u + 1] = fp8x2_to_bf16x2(static_cast<uint16_t>(w4[u] >> 16), sc);
        }
        uint8_t* dst = wt + row * ROWB + col * 32;
        *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      __syncthreads();
    }
    const uint32_t waddr = s32(wt) + (((lane >> 3) & 1) * 8 + (lane & 7)) * ROWB + (warp * WN + (lane >> 4) * 8) * 2;
    const uint32_t xaddr = s32(xt) + (((lane >> 3) & 1) * 8 + (lane & 7)) * XROWB + (lane >> 4) * 16;
#pragma unroll
    for (int ks = 0; ks < TKC / 16; ++ks) {
      uint32_t b[NT / 2][4];
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) ldsm4t(b[np], waddr + ks * 16 * ROWB + np * 32);
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        if (mt < n_mt) {
          uint32_t a[4];
          ldsm4(a, xaddr + mt * 16 * XROWB + ks * 32);
#pragma unroll
          for (int np = 0; np < NT / 2; ++np) {
            mma16816(acc[mt][2 * np], a, b[np][0], b[np][1]);
            mma16816(acc[mt][2 * np + 1], a, b[np][2], b[np][3]);
          }
        }
      }
    }
  }
  cp_wait<0>();
  float* out = p.part + static_cast<size_t>(split) * p.R * p.N;
  const int col = n0 + warp * WN + (lane & 3) * 2;
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
    const int ra = mt * 16 + (lane >> 2), rb = ra + 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (ra < cnt) *reinterpret_cast<float2*>(out + static_cast<size_t>(r0 + ra) * p.N + col + nt * 8) = make_float2(acc[mt][nt][0], acc[mt][nt][1]);
      if (rb < cnt) *reinterpret_cast<float2*>(out + static_cast<size_t>(r0 + rb) * p.N + col + nt * 8) = make_float2(acc[mt][nt][2], acc[mt][nt][3]);
    }
  }
}

// out[r, c] = act(sum over splits of part[s, r, c] + bias[group(r), c]); with SwiGLU the N = 2H columns are gate | linear.
// Without SwiGLU an optional residual is added after scaling: out = residual + alpha * (sum + bias).
__global__ void decode_gemm_finish_kernel(const float* __restrict__ part, const float* __restrict__ bias, const int* __restrict__ offsets,
                                          __nv_bfloat16* __restrict__ out, int R, int N, int G, int splits, int swiglu, float beta, float limit,
                                          const __nv_bfloat16* __restrict__ residual, float alpha) {
  const int r = blockIdx.x;
  int g = 0;
  if (offsets && bias) {
    int lo = 0, hi = G;                                          // last g with offsets[g] <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offsets[mid] <= r) lo = mid; else hi = mid;
    }
    g = lo;
  }
  const int H = swiglu ? N / 2 : N;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float a = bias ? bias[static_cast<size_t>(g) * N + c] : 0.f;
    float l = (swiglu && bias) ? bias[static_cast<size_t>(g) * N + H + c] : 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* row = part + (static_cast<size_t>(s) * R + r) * N;
      a += row[c];
      if (swiglu) l += row[H + c];
    }
    if (swiglu) {
      const float gc = fminf(a, limit), lc = fminf(fmaxf(l, -limit), limit);
      a = (lc + 1.f) * gc / (1.f + __expf(-beta * gc));
    } else {
      a *= alpha;
      if (residual) a += __bfloat162float(residual[static_cast<size_t>(r) * N + c]);
    }
    out[static_cast<size_t>(r) * H + c] = __float2bfloat16(a);
  }
}

template <bool FP8, int TN>
int launch(const DGParams& p, cudaStream_t stream) {
  constexpr int smem = Geo<FP8, TN>::SMEM_B;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(decode_gemm_kernel<FP8, TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -91;
    configured[dev] = true;
  }
  dim3 grid(p.N / TN, p.G, p.splits * p.zblocks);
  decode_gemm_kernel<FP8, TN><<<grid, THREADS, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -92;
}

template <bool FP8>
int launch_tn(const DGParams& p, int tn, cudaStream_t stream) {
  if (tn == 192) return launch<FP8, 192>(p, stream);
  if (tn == 128) return launch<FP8, 128>(p, stream);
  return launch<FP8, 64>(p, stream);
}

}  // namespace

// x [R, K] bf16 (rows sorted by group); w [G, K, N] bf16 (quant = 0) or e4m3 with wscale [G, K/bk, N/bn] (quant = 1);
// offsets [G+1] int32 on the device (null: a single group), counts [G] optional real row counts when the offsets are padded; part: fp32 scratch [splits, R, N]; out bf16 [R, N] or, with
// swiglu, [R, N/2]. bias fp32 [G, N] or null. Without swiglu: out = residual (bf16 [R, N], optional) + alpha * (x @ w + bias). K and N must be multiples of 64, K / splits a multiple of 64.
// `max_group_rows` = upper bound of the rows of one group (sizes grid.z; R when unknown).
// `panel` = columns per CTA: 64, 128 or 192, a divisor of N (0: 128 if it divides N, else 64).
extern "C" int lyra_decode_gemm(const void* x, const void* w, const float* wscale, int quant, int bk, int bn, const int* offsets, const int* counts,
                                const float* bias,
                                float* part, void* out, int R, int K, int N, int G, int splits, int swiglu, float swiglu_beta, float swiglu_limit,
                                int panel, int max_group_rows, const void* residual, float alpha, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (panel == 0) panel = N % 128 == 0 ? 128 : 64;
  if ((panel != 64 && panel != 128 && panel != 192) || N % panel) return -90;
  if (K % TKC || splits < 1 || (K / TKC) % splits || G < 1 || (!offsets && G != 1)) return -90;
  if (quant && (!wscale || bk % TKC || bn % 16 || K % bk || N % bn)) return -90;
  if (swiglu && (N / 2) % 2) return -90;
  DGParams p;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.w = static_cast<const uint8_t*>(w);
  p.wscale = wscale;
  p.offsets = offsets;
  p.counts = offsets ? counts : nullptr;
  p.part = part;
  p.R = R;
  p.K = K;
  p.N = N;
  p.G = G;
  p.splits = splits;
  p.k_per_split = K / splits;
  p.bk = bk;
  p.bn = bn;
  if (max_group_rows <= 0 || max_group_rows > R) max_group_rows = R;
  p.zblocks = (max_group_rows + MROWS - 1) / MROWS;   // 64-row blocks that the largest possible group needs
  const int rc = quant ? launch_tn<true>(p, panel, stream) : launch_tn<false>(p, panel, stream);
  if (rc) return rc;
  if (swiglu && (residual || alpha != 1.f)) return -90;
  decode_gemm_finish_kernel<<<R, 256, 0, stream>>>(part, bias, offsets, static_cast<__nv_bfloat16*>(out), R, N, G, splits, swiglu, swiglu_beta,
                                                   swiglu_limit, static_cast<const __nv_bfloat16*>(residual), alpha);
  return cudaGetLastError() == cudaSuccess ? 0 : -93;
}
