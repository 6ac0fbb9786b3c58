// Single-query (decode) attention over a dense bf16 or fp8 KV cache, split over the key axis.
//
// Role of lyra/kernels/decode_attention.py:72-260: one new token per sequence, the query heads that share a KV head form
// the M dimension of the products, online softmax seeded by the sink logit, keys visible when col <= pos (and
// col > pos - window on sliding layers, so those layers read only `window` positions), fp8 caches dequantised inside the
// kernel with one scale per (sequence, kv head, position).
//
// This op is bound by HBM reads of the cache (about 4-16 FLOP per byte), so the design is about bytes in flight, not
// tensor throughput: a grid of (key splits, kv heads, sequences); four warps per CTA, each with its own three-stage
// cp.async ring of 32-key tiles (up to 200 KB of loads in flight per SM), no CTA-wide barrier inside the key loop.
// The products use warp-level m16n8k16 bf16 MMAs with the (<= 16) query heads of the group as M: a tcgen05 tile needs
// M >= 64, which a decode step does not have. Partials of the splits are merged by a second tiny kernel.

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int WARPS = 4, TK = 32, NSTAGE = 3;
constexpr float LOG2E = 1.4426950408889634f;

struct DecParams {
  const __nv_bfloat16* q;   // [B, Nq, D]
  const uint8_t* k;         // [B, Nkv, S, D] bf16 or e4m3
  const uint8_t* v;
  const float* kscale;      // [B, Nkv, S] (fp8 only)
  const float* vscale;
  const float* sinks;       // [Nq] or null
  __nv_bfloat16* out;       // [B, Nq, D]
  float* part_o;            // [B, Nq, splits, D]   (splits > 1)
  float* part_ml;           // [B, Nq, splits, 2]
  const int* pos_dev;       // optional device-resident position (for replayed launches)
  int pos, B, Nq, Nkv, S, window, splits;
  float scale_log2;
};

__device__ __forceinline__ uint32_t s32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp16(uint32_t dst, const void* src, int nbytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(nbytes) : "memory");
}
__device__ __forceinline__ void cp4(uint32_t dst, const void* src, int nbytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(nbytes) : "memory");
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

template <int D, bool FP8>
struct Geo {
  static constexpr int ROWB = D * 2 + 16;                       // padded bf16 row: ldmatrix rows fall in distinct banks
  static constexpr int TILE_B = TK * ROWB;                      // one bf16 work tile
  static constexpr int RAW_B = FP8 ? TK * D : TILE_B;           // one K or V tile as it arrives
  static constexpr int STAGE_B = 2 * RAW_B + (FP8 ? 2 * TK * 4 : 0);
  static constexpr int WARP_B = NSTAGE * STAGE_B + (FP8 ? 2 * TILE_B : 0);
  static constexpr int SMEM_B = WARPS * WARP_B;
};

template <int D, bool FP8>
__global__ void __launch_bounds__(WARPS * 32) decode_attn_kernel(const DecParams p) {
  using G_ = Geo<D, FP8>;
  constexpr int ROWB = G_::ROWB, TILE_B = G_::TILE_B, RAW_B = G_::RAW_B, STAGE_B = G_::STAGE_B;
  constexpr int ESZ = FP8 ? 1 : 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = p.Nq / p.Nkv;
  const int pos = p.pos_dev ? *p.pos_dev : p.pos;
  const int hi = min(pos, p.S - 1);
  const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int n_keys = hi - lo + 1;
  const int chunk = ((n_keys + p.splits - 1) / p.splits + TK - 1) / TK * TK;
  const int kbeg = lo + split * chunk;
  const int kend = min(kbeg + chunk, hi + 1);
  const int n_tiles = kend > kbeg ? (kend - kbeg + TK - 1) / TK : 0;
  const int nt_w = n_tiles > warp ? (n_tiles - warp + WARPS - 1) / WARPS : 0;   // this warp's tiles: warp, warp+4, ...

  uint8_t* wsm = smem + warp * G_::WARP_B;
  const size_t head_row0 = (static_cast<size_t>(b) * p.Nkv + kvh) * p.S;
  const uint8_t* kbase = p.k + head_row0 * D * ESZ;
  const uint8_t* vbase = p.v + head_row0 * D * ESZ;

  // ---- query fragments: rows = heads of the group (rows >= G are zero)
  uint32_t qa[D / 16][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
    const __nv_bfloat16* q0 = p.q + (static_cast<size_t>(b) * p.Nq + kvh * G + r0) * D;
    const __nv_bfloat16* q1 = p.q + (static_cast<size_t>(b) * p.Nq + kvh * G + r1) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c) : 0u;
      qa[ks][1] = r1 < G ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c) : 0u;
      qa[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c + 8) : 0u;
      qa[ks][3] = r1 < G ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c + 8) : 0u;
    }
  }

  auto issue = [&](int i) {   // i-th tile of this warp -> stage i % NSTAGE
    const int key0 = kbeg + (warp + i * WARPS) * TK;
    uint8_t* st = wsm + (i % NSTAGE) * STAGE_B;
    constexpr int CPR = D * ESZ / 16;                            // 16-byte chunks per row
    constexpr int DROW = FP8 ? D : ROWB;
#pragma unroll
    for (int j = 0; j < TK * CPR / 32; ++j) {
      const int c = lane + 32 * j, row = c / CPR, col = c % CPR;
      const int key = key0 + row;
      const bool ok = key < kend;
      const size_t off = static_cast<size_t>(ok ? key : kbeg) * D * ESZ + col * 16;
      cp16(s32(st + row * DROW + col * 16), kbase + off, ok ? 16 : 0);
      cp16(s32(st + RAW_B + row * DROW + col * 16), vbase + off, ok ? 16 : 0);
    }
    if (FP8) {
      const int key = key0 + lane;
      const bool ok = key < kend;
      const size_t off = head_row0 + (ok ? key : kbeg);
      cp4(s32(st + 2 * RAW_B + lane * 4), p.kscale + off, ok ? 4 : 0);
      cp4(s32(st + 2 * RAW_B + TK * 4 + lane * 4), p.vscale + off, ok ? 4 : 0);
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
  for (int s = 0; s < NSTAGE - 1; ++s) {
    if (s < nt_w) issue(s);
    cp_commit();
  }
  for (int i = 0; i < nt_w; ++i) {
    if (i + NSTAGE - 1 < nt_w) issue(i + NSTAGE - 1);
    cp_commit();
    cp_wait<NSTAGE - 1>();
    __syncwarp();
    uint8_t* st = wsm + (i % NSTAGE) * STAGE_B;
    uint8_t *kt = st, *vt = st + RAW_B;
    if (FP8) {   // raw e4m3 rows -> scaled bf16 work tiles (same values as dequantise-then-cast)
      kt = wsm + NSTAGE * STAGE_B;
      vt = kt + TILE_B;
      const float* ksc = reinterpret_cast<const float*>(st + 2 * RAW_B);
      const float* vsc = ksc + TK;
      constexpr int CPR = D / 16;
#pragma unroll
      for (int j = 0; j < TK * CPR / 32; ++j) {
        const int c = lane + 32 * j, row = c / CPR, col = c % CPR;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint4 raw = *reinterpret_cast<const uint4*>(st + which * RAW_B + row * D + col * 16);
          const float sc = which ? vsc[row] : ksc[row];
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
          uint32_t outw[8];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            outw[2 * u] = fp8x2_to_bf16x2(static_cast<uint16_t>(w[u] & 0xffffu), sc);
            outw[2 * u + 1] = fp8x2_to_bf16x2(static_cast<uint16_t>(w[u] >> 16), sc);
          }
          uint8_t* dst = (which ? vt : kt) + row * ROWB + col * 32;
          *reinterpret_cast<uint4*>(dst) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
          *reinterpret_cast<uint4*>(dst + 16) = make_uint4(outw[4], outw[5], outw[6], outw[7]);
        }
      }
      __syncwarp();
    }

    // ---- S = Q K^T for 32 keys: four 8-key column tiles
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const uint32_t kaddr = s32(kt) + ((lane >> 4) * 8 + (lane & 7)) * ROWB + ((lane >> 3) & 1) * 16;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        uint32_t r[4];
        ldsm4(r, kaddr + jp * 16 * ROWB + ks * 32);
        mma16816(s[jp * 2], qa[ks], r[0], r[1]);
        mma16816(s[jp * 2 + 1], qa[ks], r[2], r[3]);
      }
    }
    // ---- mask, online softmax (exp2 domain)
    const int key0 = kbeg + (warp + i * WARPS) * TK + (lane & 3) * 2;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + j * 8 + (e & 1);
        s[j][e] = key < kend ? s[j][e] * p.scale_log2 : -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float a0 = mn0 == -INFINITY ? 1.f : exp2f(m0 - mn0), a1 = mn1 == -INFINITY ? 1.f : exp2f(m1 - mn1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
    m0 = mn0;
    m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = exp2f(s[j][0] - ms0);
      s[j][1] = exp2f(s[j][1] - ms0);
      s[j][2] = exp2f(s[j][2] - ms1);
      s[j][3] = exp2f(s[j][3] - ms1);
      sum0 += s[j][0] + s[j][1];
      sum1 += s[j][2] + s[j][3];
    }
    l0 = l0 * a0 + sum0;
    l1 = l1 * a1 + sum1;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      o[dt][0] *= a0;
      o[dt][1] *= a0;
      o[dt][2] *= a1;
      o[dt][3] *= a1;
    }
    // ---- O += P V: P's accumulator layout is the A-operand layout of the next product
    const uint32_t vaddr = s32(vt) + (((lane >> 3) & 1) * 8 + (lane & 7)) * ROWB + (lane >> 4) * 16;
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const uint32_t pa[4] = {pack2(s[2 * kk][0], s[2 * kk][1]), pack2(s[2 * kk][2], s[2 * kk][3]),
                              pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack2(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t r[4];
        ldsm4t(r, vaddr + kk * 16 * ROWB + dp * 32);
        mma16816(o[dp * 2], pa, r[0], r[1]);
        mma16816(o[dp * 2 + 1], pa, r[2], r[3]);
      }
    }
    __syncwarp();
  }
  cp_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();   // every warp is done with its ring: the space is reused for the merge

  float* red_o = reinterpret_cast<float*>(smem);                 // [WARPS][16][D]
  float* red_m = red_o + WARPS * 16 * D;                         // [WARPS][16]
  float* red_l = red_m + WARPS * 16;
  {
    const int r0 = lane >> 2, c = (lane & 3) * 2;
    float* base = red_o + warp * 16 * D;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      *reinterpret_cast<float2*>(base + r0 * D + dt * 8 + c) = make_float2(o[dt][0], o[dt][1]);
      *reinterpret_cast<float2*>(base + (r0 + 8) * D + dt * 8 + c) = make_float2(o[dt][2], o[dt][3]);
    }
    if ((lane & 3) == 0) {
      red_m[warp * 16 + r0] = m0;
      red_m[warp * 16 + r0 + 8] = m1;
      red_l[warp * 16 + r0] = l0;
      red_l[warp * 16 + r0 + 8] = l1;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += WARPS * 32) {
    const int g = idx / D, d = idx - g * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, red_m[w * 16 + g]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = red_m[w * 16 + g];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += red_l[w * 16 + g] * f;
      O += red_o[(w * 16 + g) * D + d] * f;
    }
    const int h = kvh * G + g;
    const size_t row = static_cast<size_t>(b) * p.Nq + h;
    if (p.splits == 1) {
      const float sk = p.sinks ? p.sinks[h] * LOG2E : -INFINITY;
      const float M2 = fmaxf(M, sk);
      const float f = M == -INFINITY ? 0.f : exp2f(M - M2);
      const float L2 = L * f + (p.sinks ? exp2f(sk - M2) : 0.f);
      p.out[row * D + d] = __float2bfloat16(L2 > 0.f ? O * f / L2 : 0.f);
    } else {
      p.part_o[(row * p.splits + split) * D + d] = O;
      if (d == 0) {
        p.part_ml[(row * p.splits + split) * 2] = M;
        p.part_ml[(row * p.splits + split) * 2 + 1] = L;
      }
    }
  }
}

// Merges the splits of one (sequence, head): block = D threads.
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const float* __restrict__ sinks,
                                    __nv_bfloat16* __restrict__ out, int Nq, int splits, int D) {
  const size_t row = blockIdx.x;
  const int h = static_cast<int>(row % Nq), d = threadIdx.x;
  const float sk = sinks ? sinks[h] * LOG2E : -INFINITY;
  float M = sk;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(row * splits + s) * 2]);
  float L = sinks ? exp2f(sk - M) : 0.f, O = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(row * splits + s) * 2];
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
    L += part_ml[(row * splits + s) * 2 + 1] * f;
    O += part_o[(row * splits + s) * D + d] * f;
  }
  out[row * D + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
}

template <int D, bool FP8>
int launch(const DecParams& p, cudaStream_t stream) {
  constexpr int smem = Geo<D, FP8>::SMEM_B;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(decode_attn_kernel<D, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -81;
    configured[dev] = true;
  }
  dim3 grid(p.splits, p.Nkv, p.B);
  decode_attn_kernel<D, FP8><<<grid, WARPS * 32, smem, stream>>>(p);
  if (cudaGetLastError() != cudaSuccess) return -82;
  if (p.splits > 1) {
    decode_merge_kernel<<<p.B * p.Nq, D, 0, stream>>>(p.part_o, p.part_ml, p.sinks, p.out, p.Nq, p.splits, D);
    if (cudaGetLastError() != cudaSuccess) return -83;
  }
  return 0;
}

}  // namespace

// q/out [B, Nq, D] bf16; k/v [B, Nkv, S, D] bf16 (quant = 0) or e4m3 with fp32 scales [B, Nkv, S] (quant = 1).
// Visible keys: max(0, pos - window + 1) (0 when window == 0) .. pos. `pos_dev`, when given, overrides `pos` at run time
// (the launch geometry then comes from `splits` alone). `part_o` / `part_ml` are needed when splits > 1.
extern "C" int lyra_decode_attention(const void* q, const void* k, const void* v, const float* kscale, const float* vscale, int quant,
                                     const float* sinks, void* out, float* part_o, float* part_ml, int splits, const int* pos_dev,
                                     int B, int Nq, int Nkv, int S, int D, float scale, int window, int pos, cudaStream_t stream) {
  if (Nq % Nkv != 0 || Nq / Nkv > 16 || (D != 64 && D != 128) || splits < 1 || B < 1 || pos < 0) return -80;
  if (splits > 1 && (!part_o || !part_ml)) return -80;
  if (quant && (!kscale || !vscale)) return -80;
  DecParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const uint8_t*>(k);
  p.v = static_cast<const uint8_t*>(v);
  p.kscale = kscale;
  p.vscale = vscale;
  p.sinks = sinks;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.pos_dev = pos_dev;
  p.pos = pos;
  p.B = B;
  p.Nq = Nq;
  p.Nkv = Nkv;
  p.S = S;
  p.window = window;
  p.splits = splits;
  p.scale_log2 = scale * LOG2E;
  if (D == 64) return quant ? launch<64, true>(p, stream) : launch<64, false>(p, stream);
  return quant ? launch<128, true>(p, stream) : launch<128, false>(p, stream);
}
