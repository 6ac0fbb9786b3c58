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

//
// Block-scaled e4m3 on the tensor cores (`decode_gemm_f8_kernel`, role of the quantised paths of lyra/kernels/decode_gemm.py:234-244
// and lyra/kernels/gemm.py:557-589): tcgen05 tiles need 128 rows, which a decode step's tokens cannot fill - but the weights
// can. The operand roles are swapped: the accumulator tile is D^T[128 weight columns x NTOK tokens] = W^T x^T, with the
// e4m3 weight panel as the 128-row A operand (TMA, [K, N] storage = MN-major) and the tokens, quantised to e4m3 with one
// scale per (row, K block) like the reference's `quantize(lhs, (1, scale_k))`, as the narrow B operand. Scales are applied
// in software: every K block of `bk` values accumulates into its own TMEM accumulator of a ring of four or eight
// (kind::f8f6f4, fp32), the four epilogue warps read it back (tcgen05.ld), multiply by w_scale[k block, column block] *
// x_scale[token, k block] and add into fp32 registers while the tensor core already works on the following K blocks.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/sm100.cuh"
#include "../common/tmap.h"

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
// One CTA per (row, run of 1024 output columns), four columns per thread: the pass is a few megabytes, so it is all latency -
// every thread has its loads in flight at once instead of walking the row.
__global__ void __launch_bounds__(256) decode_gemm_finish_kernel(const float* __restrict__ part, const float* __restrict__ bias,
                                                                 const int* __restrict__ offsets, __nv_bfloat16* __restrict__ out, int R, int N, int G,
                                                                 int splits, int swiglu, float beta, float limit,
                                                                 const __nv_bfloat16* __restrict__ residual, float alpha) {
  const int r = blockIdx.x;
  const int H = swiglu ? N / 2 : N;
  const int c0 = (blockIdx.y * 256 + threadIdx.x) * 4;
  if (c0 >= H) return;
  int g = 0;
  if (offsets && bias) {
    int lo = 0, hi = G;                                          // last g with offsets[g] <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offsets[mid] <= r) lo = mid; else hi = mid;
    }
    g = lo;
  }
  float a[4] = {0.f, 0.f, 0.f, 0.f}, l[4] = {0.f, 0.f, 0.f, 0.f};
  const int n = min(4, H - c0);
  if (n == 4 && (N & 3) == 0 && (H & 3) == 0) {
    for (int s = 0; s < splits; ++s) {
      const float* row = part + (static_cast<size_t>(s) * R + r) * N;
      const float4 v = *reinterpret_cast<const float4*>(row + c0);
      a[0] += v.x; a[1] += v.y; a[2] += v.z; a[3] += v.w;
      if (swiglu) {
        const float4 w = *reinterpret_cast<const float4*>(row + H + c0);
        l[0] += w.x; l[1] += w.y; l[2] += w.z; l[3] += w.w;
      }
    }
  } else {
    for (int s = 0; s < splits; ++s) {
      const float* row = part + (static_cast<size_t>(s) * R + r) * N;
      for (int i = 0; i < n; ++i) {
        a[i] += row[c0 + i];
        if (swiglu) l[i] += row[H + c0 + i];
      }
    }
  }
  for (int i = 0; i < n; ++i) {
    float av = a[i], lv = l[i];
    if (bias) {
      av += bias[static_cast<size_t>(g) * N + c0 + i];
      if (swiglu) lv += bias[static_cast<size_t>(g) * N + H + c0 + i];
    }
    if (swiglu) {
      const float gc = fminf(av, limit), lc = fminf(fmaxf(lv, -limit), limit);
      av = (lc + 1.f) * gc / (1.f + __expf(-beta * gc));
    } else {
      av *= alpha;
      if (residual) av += __bfloat162float(residual[static_cast<size_t>(r) * N + c0 + i]);
    }
    out[static_cast<size_t>(r) * H + c0 + i] = __float2bfloat16(av);
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


// ------------------------------------------------------------------------------------------------ e4m3 x e4m3 on tcgen05
constexpr int F8_KSTAGE = 128;               // K values per shared-memory stage: 128 rows of 128 weight bytes, 128 bytes per token row
constexpr int F8_THREADS = 192;              // warp 0: TMA, warp 1: MMA issue + TMEM, warps 2..5: scale-and-accumulate
constexpr int F8_MAX_KBLOCKS = 64;           // K blocks (scale rows) one CTA can hold
constexpr int F8_MAX_UNITS = 1024;           // (group, block of token rows) pairs with at least one row that one launch can hold

constexpr int f8_stages(int ntok) { return ntok >= 64 ? 3 : 4; }   // sized so that two CTAs fit one SM (two weight streams in flight)
// TMEM accumulators per CTA. One K block's round trip (MMA retires -> commit -> epilogue wakes -> tcgen05.ld -> release -> issuer
// wakes) measured about 2 us, against 0.2 us of HBM time for the block's weights: the issuer must be able to run several K
// blocks ahead of the epilogue, so the ring is as deep as the shared-memory stages hold K blocks.
constexpr int f8_accs(int ntok) { return ntok >= 64 ? 4 : 8; }

struct F8Params {
  const float* xs;          // [R, K / bk] activation scales
  const float* ws;          // [G, K / bk, N / bn] weight scales
  const int* offsets;
  const int* counts;
  float* part;              // [splits, R, N]
  int R, K, N, G, splits, k_per_split, bk, bn, zblocks;
  int* status;
};

// One pass = one (128-column weight panel, group, K split, block of NTOK rows). A CTA walks its passes in a fixed order that all
// of its roles derive independently; barriers, shared-memory stages and the accumulator ring run on across passes.
struct F8Pass {
  int n0, g, split, r0, cnt;
};
struct F8Unit {    // a group's block of token rows
  int r0;
  short g, cnt;
};

template <int NTOK>
__global__ void __launch_bounds__(F8_THREADS) decode_gemm_f8_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                                                                   const F8Params p) {
  using namespace lyra;
  constexpr int A_BYTES = F8_KSTAGE * 128;                 // 128 k rows x 128 weight columns (one byte each)
  constexpr int B_BYTES = NTOK * 128;                      // NTOK token rows x 128 k values
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int F8_STAGES = f8_stages(NTOK);
  constexpr int NACC = f8_accs(NTOK);
  constexpr uint32_t TMEM_COLS = NACC * NTOK;              // 128 or 256: a power of two
  constexpr uint32_t IDESC = make_idesc(128, NTOK, 0, 0, 1, 0);   // e4m3 x e4m3, A (weights) MN-major, B (tokens) K-major

  // Persistent: the grid is a couple of CTAs per SM and each takes passes round-robin. A pass is one 128-column weight panel
  // times one unit (a group's block of up to NTOK token rows) times one K split; every pass streams the same number of weight
  // bytes, and units exist only for groups that received rows, so the CTAs finish together however the rows are spread over the
  // groups (with a static walk over all groups, a decode step that touches 28 of 128 experts left most CTAs idle while a few
  // streamed ten panels). Panels run fastest, so CTAs working side by side read neighbouring 128-byte pieces of the same rows.
  // (One CTA per pass spent most of its life on TMEM allocation, barrier set-up and pipeline fill.)
  const int n_panels = (p.N + 127) / 128;
  const int n_steps = p.k_per_split / 32;                  // MMAs (K = 32 each) per pass
  const int n_kb = p.k_per_split / p.bk;                   // K blocks = read-backs per pass
  const int steps_per_kb = p.bk / 32;
  const int n_stage_loads = (p.k_per_split + F8_KSTAGE - 1) / F8_KSTAGE;
  const int ws_n = p.bn >= 128 ? 1 : 128 / p.bn;           // weight-scale columns a panel touches (it starts on a block boundary)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* xs_s = reinterpret_cast<float*>(smem + F8_STAGES * STAGE_BYTES);        // [n_kb][NTOK]
  float* ws_s = xs_s + F8_MAX_KBLOCKS * NTOK;                                    // [n_kb][ws_n]
  __shared__ uint64_t full_bar[F8_STAGES], empty_bar[F8_STAGES], tfull_bar[NACC], tempty_bar[NACC];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag, n_units_s;
  __shared__ F8Unit units[F8_MAX_UNITS];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < NACC; ++a) {
      mbar_init(smem_u32(&tfull_bar[a]), 1);
      mbar_init(smem_u32(&tempty_bar[a]), 4);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_holder), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_holder;
  volatile int* abortp = &abort_flag;

  // the units of this launch, built by every CTA for itself: warp 2 scans the groups' row counts
  if (warp == 2) {
    const int per = (p.G + 31) / 32;                       // consecutive groups per lane
    int mine = 0;
    for (int g = lane * per; g < min(p.G, (lane + 1) * per); ++g) {
      const int beg = p.offsets ? p.offsets[g] : 0;
      const int end = p.offsets ? (p.counts ? beg + p.counts[g] : p.offsets[g + 1]) : p.R;
      mine += (max(end - beg, 0) + NTOK - 1) / NTOK;
    }
    int at = mine;                                          // inclusive scan over the lanes
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, at, d);
      if (lane >= d) at += up;
    }
    if (lane == 31) n_units_s = min(at, F8_MAX_UNITS);
    at -= mine;
    for (int g = lane * per; g < min(p.G, (lane + 1) * per); ++g) {
      const int beg = p.offsets ? p.offsets[g] : 0;
      const int end = p.offsets ? (p.counts ? beg + p.counts[g] : p.offsets[g + 1]) : p.R;
      for (int r0 = beg; r0 < end && at < F8_MAX_UNITS; r0 += NTOK, ++at) {
        units[at].r0 = r0;
        units[at].g = static_cast<short>(g);
        units[at].cnt = static_cast<short>(min(NTOK, end - r0));
      }
    }
  }
  __syncthreads();
  const int n_units = n_units_s;
  const int n_passes = n_panels * n_units * p.splits;

  // the pass sequence of this CTA: `next` fills `ps`; every role runs the same code
  int pass = int(blockIdx.x) - int(gridDim.x);
  F8Pass ps;
  auto next = [&]() -> bool {
    pass += gridDim.x;
    if (pass >= n_passes) return false;
    const int panel = pass % n_panels, rest = pass / n_panels;
    const F8Unit u = units[rest % n_units];
    ps.split = rest / n_units;
    ps.n0 = panel * 128;
    ps.g = u.g;
    ps.r0 = u.r0;
    ps.cnt = u.cnt;
    return true;
  };

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tma_w);
      tma_prefetch_desc(&tma_x);
      uint32_t it = 0;
      bool ok = true;
      while (ok && next()) {
        const int kbeg = ps.split * p.k_per_split;
        for (int st = 0; st < n_stage_loads; ++st, ++it) {
          const int s = it % F8_STAGES;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / F8_STAGES) & 1) ^ 1, abortp)) {
            atomicCAS(p.status, 0, STATUS_TIMEOUT_EMPTY);
            abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          mbar_expect_tx(bar, STAGE_BYTES);
          const int k0 = kbeg + st * F8_KSTAGE;            // rows past K (and token rows past R) read as zeros
          tma_load_3d(sa, &tma_w, bar, ps.n0, k0, ps.g);
          tma_load_2d(sa + A_BYTES, &tma_x, bar, k0, ps.r0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it0 = 0, kc0 = 0;                           // running stage / K-block numbers at the start of the pass
      bool ok = true;
      while (ok && next()) {
        int j = 0, in_kb = 0;                              // position inside the stage / inside the K block
        uint32_t it = it0, kc = kc0;
        for (int q = 0; q < n_steps; ++q) {
          const int s = it % F8_STAGES, acc = kc % NACC;
          if (j == 0) {
            if (!mbar_wait(smem_u32(&full_bar[s]), (it / F8_STAGES) & 1, abortp)) {
              atomicCAS(p.status, 0, STATUS_TIMEOUT_FULL);
              abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after();
          }
          if (in_kb == 0) {
            if (!mbar_wait(smem_u32(&tempty_bar[acc]), ((kc / NACC) & 1) ^ 1, abortp)) {
              atomicCAS(p.status, 0, STATUS_TIMEOUT_TMEM);
              abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after();
          }
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = make_smem_desc(sa + j * 4096, 128 * 128, 1024);          // 32 k rows of 128 bytes, 8-row groups 1024 bytes apart
          const uint64_t db = make_smem_desc(sa + A_BYTES + j * 32, 16, 1024);         // 32 bytes along each token row
          tc_mma_ss_f8(tmem_base + acc * NTOK, da, db, IDESC, in_kb == 0 ? 0u : 1u);
          if (++j == F8_KSTAGE / 32 || q == n_steps - 1) {   // a pass ends its last stage, full or not
            tc_commit(smem_u32(&empty_bar[s]));
            j = 0;
            ++it;
          }
          if (++in_kb == steps_per_kb) {
            tc_commit(smem_u32(&tfull_bar[acc]));
            in_kb = 0;
            ++kc;
          }
        }
        it0 += n_stage_loads;
        kc0 += n_kb;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int te = threadIdx.x - 64;                        // 0..127 among the four epilogue warps
    uint32_t kc0 = 0;
    bool ok = true;
    int table_g = -1, table_n0 = -1, table_split = -1;
    while (ok && next()) {
      const int col = ps.n0 + quarter * 32 + lane;          // this thread's weight column = TMEM lane
      const int wsel = p.bn >= 128 ? 0 : (quarter * 32 + lane) / p.bn;
      const int kb0 = ps.split * n_kb;
      // scale tables of this pass (only these four warps touch them): tokens x K blocks, and K blocks x column blocks
      for (int i = te; i < n_kb * NTOK; i += 128) {
        const int kb = i / NTOK, t = i - kb * NTOK;
        xs_s[i] = t < ps.cnt ? p.xs[static_cast<size_t>(ps.r0 + t) * (p.K / p.bk) + kb0 + kb] : 0.f;
      }
      if (table_g != ps.g || table_n0 != ps.n0 || table_split != ps.split) {
        for (int i = te; i < n_kb * ws_n; i += 128) {
          const int kb = i / ws_n, jj = i - kb * ws_n;
          const int nb = ps.n0 / p.bn + jj;
          ws_s[i] = nb < p.N / p.bn ? p.ws[(static_cast<size_t>(ps.g) * (p.K / p.bk) + kb0 + kb) * (p.N / p.bn) + nb] : 0.f;
        }
        table_g = ps.g;
        table_n0 = ps.n0;
        table_split = ps.split;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float racc[NTOK];
#pragma unroll
      for (int t = 0; t < NTOK; ++t) racc[t] = 0.f;
      // A TMEM read is a long round trip: the accumulators of U consecutive K blocks are read back with one wait.
      constexpr int U = 64 / NTOK;
      for (int kb = 0; kb < n_kb && ok; kb += U) {
        const int nu = min(U, n_kb - kb);
        uint32_t r[U][NTOK / 16][16];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (u < nu && ok) {
            const uint32_t kc = kc0 + kb + u;
            if (!mbar_wait(smem_u32(&tfull_bar[kc % NACC]), (kc / NACC) & 1, abortp)) {
              if (lane == 0) atomicCAS(p.status, 0, STATUS_TIMEOUT_TMEM);
              abort_flag = 1;
              ok = false;
            }
          }
        }
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (u < nu) {
            const uint32_t taddr = tmem_base + ((kc0 + kb + u) % NACC) * NTOK + (uint32_t(quarter * 32) << 16);
#pragma unroll
            for (int c = 0; c < NTOK / 16; ++c) tmem_ld16(taddr + c * 16, r[u][c]);
          }
        }
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (u < nu) mbar_arrive(smem_u32(&tempty_bar[(kc0 + kb + u) % NACC]));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (u < nu) {
            const float wsv = ws_s[(kb + u) * ws_n + wsel];
            const float* xrow = xs_s + (kb + u) * NTOK;
#pragma unroll
            for (int c = 0; c < NTOK / 16; ++c)
#pragma unroll
              for (int i = 0; i < 16; ++i) racc[c * 16 + i] = fmaf(__uint_as_float(r[u][c][i]), wsv * xrow[c * 16 + i], racc[c * 16 + i]);
          }
        }
      }
      if (ok && col < p.N) {
        float* out = p.part + static_cast<size_t>(ps.split) * p.R * p.N + col;
#pragma unroll
        for (int t = 0; t < NTOK; ++t)
          if (t < ps.cnt) out[static_cast<size_t>(ps.r0 + t) * p.N] = racc[t];
      }
      kc0 += n_kb;
      asm volatile("bar.sync 1, 128;" ::: "memory");       // everyone is done with this pass's scale tables
    }
  }
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);        // let copies still in flight land before the shared memory is released
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int NTOK>
int launch_f8(const CUtensorMap& tw, const CUtensorMap& tx, const F8Params& p, cudaStream_t stream) {
  constexpr int smem = f8_stages(NTOK) * (F8_KSTAGE * 128 + NTOK * 128) + F8_MAX_KBLOCKS * (NTOK + 2) * 4 + 1024;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(decode_gemm_f8_kernel<NTOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -91;
    configured[dev] = true;
  }
  if (p.G + (p.R + NTOK - 1) / NTOK > F8_MAX_UNITS) return -93;   // more (group, row block) units than a CTA's table holds
  const long long most = (long long)((p.N + 127) / 128) * p.splits * (p.G + (p.R + NTOK - 1) / NTOK);   // upper bound of the passes
  const int resident = 2 * lyra::sm_count();               // two CTAs per SM: two weight streams in flight
  decode_gemm_f8_kernel<NTOK><<<most < resident ? int(most) : resident, F8_THREADS, smem, stream>>>(tw, tx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -92;
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
  decode_gemm_finish_kernel<<<dim3(R, ((swiglu ? N / 2 : N) + 1023) / 1024), 256, 0, stream>>>(part, bias, offsets, static_cast<__nv_bfloat16*>(out), R, N, G,
                                                                                                splits, swiglu, swiglu_beta, swiglu_limit,
                                                                                                static_cast<const __nv_bfloat16*>(residual), alpha);
  return cudaGetLastError() == cudaSuccess ? 0 : -93;
}


// The same product with e4m3 activations on the tensor cores: xq [R, K] e4m3 with xs [R, K / bk] fp32 (one scale per row and K
// block: `lyra_fp8_quantize_2d` with a (1 x bk) block), w [G, K, N] e4m3 with ws [G, K / bk, N / bn]. `ntok` = token columns
// per tile (16, 32 or 64: the smallest that holds the largest group keeps the epilogue short; larger groups take more
// blocks along grid.z). bk must be a multiple of 32 that divides or is a multiple of 128; bn 64 or a multiple of 128; K a
// multiple of bk; N a multiple of 16 and of bn.
extern "C" int lyra_decode_gemm_f8(const void* xq, const float* xs, const void* w, const float* ws, int bk, int bn, const int* offsets,
                                   const int* counts, const float* bias, float* part, void* out, int R, int K, int N, int G, int splits, int swiglu,
                                   float swiglu_beta, float swiglu_limit, int ntok, int max_group_rows, const void* residual, float alpha,
                                   int* status, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (ntok != 16 && ntok != 32 && ntok != 64) return -90;
  if (bk < 32 || bk % 32 || (128 % bk && bk % 128) || K % bk || (bn != 64 && bn % 128) || N % bn || N % 16 || K % 16) return -90;
  if (splits < 1 || (K / bk) % splits || ((K / splits) % 128 && splits > 1) || (K / splits) / bk > F8_MAX_KBLOCKS) return -90;
  if (G < 1 || (!offsets && G != 1) || (swiglu && (residual || alpha != 1.f))) return -90;
  F8Params p;
  p.xs = xs; p.ws = ws; p.offsets = offsets; p.counts = offsets ? counts : nullptr; p.part = part;
  p.R = R; p.K = K; p.N = N; p.G = G; p.splits = splits; p.k_per_split = K / splits; p.bk = bk; p.bn = bn; p.status = status;
  if (max_group_rows <= 0 || max_group_rows > R) max_group_rows = R;
  p.zblocks = (max_group_rows + ntok - 1) / ntok;
  CUtensorMap tw, tx;
  {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)G}, strides[2] = {(uint64_t)N, (uint64_t)K * N};
    uint32_t box[3] = {128, F8_KSTAGE, 1};
    if (lyra::make_tmap(&tw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -94;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)R}, strides[1] = {(uint64_t)K};
    uint32_t box[2] = {128, (uint32_t)ntok};
    if (lyra::make_tmap(&tx, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -95;
  }
  const int rc = ntok == 64 ? launch_f8<64>(tw, tx, p, stream) : ntok == 32 ? launch_f8<32>(tw, tx, p, stream) : launch_f8<16>(tw, tx, p, stream);
  if (rc) return rc;
  decode_gemm_finish_kernel<<<dim3(R, ((swiglu ? N / 2 : N) + 1023) / 1024), 256, 0, stream>>>(part, bias, offsets, static_cast<__nv_bfloat16*>(out), R, N, G,
                                                                                                splits, swiglu, swiglu_beta, swiglu_limit,
                                                                                                static_cast<const __nv_bfloat16*>(residual), alpha);
  return cudaGetLastError() == cudaSuccess ? 0 : -93;
}
