// Flash attention forward for sm_100a: causal / sliding-window GQA attention with a learned sink per
// query head (semantics of the reference's FLASH_ATTENTION kernels, lyra/kernels/flash_attention.py:208-374):
//   out = softmax([q k^T * scale | sink_h]) restricted to the key columns, LSE in natural-log units.
// The running max starts at the sink logit and the normaliser at 1, so the sink is an extra softmax column
// without a value. Only key tiles that intersect the causal / window band are visited.
//
// One CTA per (128-query tile, query head, batch). Tensors are token-major [B, T, N, D] (the layout the
// projection GEMMs produce), addressed by 4-D TMA maps, so no transposes are needed around the kernel.
//   warp 0      : TMA producer (Q once; K and V tiles double-buffered)
//   warp 1      : tcgen05 issuer:  S = Q K^T (fp32 in TMEM, two buffers)  and  O += P V (TMEM)
//   warps 2..5  : softmax - one query row per thread via tcgen05.ld, exp2-domain online softmax with lazy
//                 rescaling of O, P written as bf16 into 128B-swizzled shared memory for the second MMA
#include "../common/sm100.cuh"
#include "../common/tmap.h"

namespace lyra {

constexpr int FA_THREADS = 320;   // TMA warp, MMA warp, two groups of four softmax warps (64 of a tile's 128 key columns each)
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct FwdParams {
  int B, T, S, Nq, Nkv, window, q_start;
  float scale_log2;       // softmax scale * log2(e)
  const float* sinks;     // [Nq]
  __nv_bfloat16* out;     // [B, T, Nq, D]
  float* lse;             // [B, Nq, T]
  int* status;
};

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const FwdParams p) {
  constexpr int BQ = 128, BKV = 128;
  constexpr int TILE = BQ * D * 2;         // bytes of a 128 x D bf16 tile
  constexpr int HALF = BQ * 128;           // bytes of one 64-column swizzle atom column block (128 rows x 128 B)
  constexpr int P_BYTES = BQ * BKV * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL0 = 0, O_COL = 256;
  constexpr uint32_t IDESC_S = make_idesc(BQ, BKV, 1, 1, 0, 0);   // Q K-major, K K-major
  constexpr uint32_t IDESC_O = make_idesc(BQ, D, 1, 1, 0, 1);     // P K-major, V MN-major

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;           // 2 stages
  uint8_t* sV = sK + 2 * TILE;       // 2 stages
  uint8_t* sP = sV + 2 * TILE;
  __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full, p_empty, o_full;
  __shared__ uint64_t x_full[2], l_full;          // row-maximum / row-sum exchange between the two softmax groups
  __shared__ float xmax[2][2][BQ], xl[2][BQ];
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ, head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (p.Nq / p.Nkv);

  // key tiles that intersect the band of this query tile
  const int qlo = p.q_start + q0;
  const int qhi = min(p.q_start + min(q0 + BQ, p.T) - 1, p.S - 1);
  int klo = p.window > 0 ? max(0, qlo - p.window + 1) : 0;
  const int jt_begin = klo / BKV;
  const int jt_end = qhi < 0 ? jt_begin : qhi / BKV + 1;
  const int n_tiles = max(jt_end - jt_begin, 0);

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 256);
      mbar_init(smem_u32(&x_full[s]), 256);
    }
    mbar_init(smem_u32(&l_full), 256);
    mbar_init(smem_u32(&p_full), 256);
    mbar_init(smem_u32(&p_empty), 1);
    mbar_init(smem_u32(&o_full), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_holder), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_holder;
  volatile int* abortp = &abort_flag;
#define FA_FAIL(code)                      \
  {                                        \
    atomicExch(p.status, code);            \
    abort_flag = 1;                        \
    break;                                 \
  }

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      tma_prefetch_desc(&tq);
      tma_prefetch_desc(&tk);
      tma_prefetch_desc(&tv);
      mbar_expect_tx(smem_u32(&q_full), TILE);
      for (int h = 0; h < D / 64; ++h) tma_load_4d(smem_u32(sQ + h * HALF), &tq, smem_u32(&q_full), h * 64, q0, head, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int k0 = (jt_begin + j) * BKV;
        if (!mbar_wait(smem_u32(&k_empty[s]), ph ^ 1, abortp)) FA_FAIL(STATUS_TIMEOUT_EMPTY);
        mbar_expect_tx(smem_u32(&k_full[s]), TILE);
        for (int h = 0; h < D / 64; ++h) tma_load_4d(smem_u32(sK + s * TILE + h * HALF), &tk, smem_u32(&k_full[s]), h * 64, k0, kvh, b);
        if (!mbar_wait(smem_u32(&v_empty[s]), ph ^ 1, abortp)) FA_FAIL(STATUS_TIMEOUT_EMPTY);
        mbar_expect_tx(smem_u32(&v_full[s]), TILE);
        for (int h = 0; h < D / 64; ++h) tma_load_4d(smem_u32(sV + s * TILE + h * HALF), &tv, smem_u32(&v_full[s]), h * 64, k0, kvh, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&k_full[s]), ph, abortp)) return false;
        if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1, abortp)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + s * TILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * HALF + (k % 4) * 32;
          tc_mma_ss(tmem + S_COL0 + s * BKV, make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), IDESC_S, k > 0);
        }
        tc_commit(smem_u32(&s_full[s]));
        tc_commit(smem_u32(&k_empty[s]));
        return true;
      };
      bool ok = mbar_wait(smem_u32(&q_full), 0, abortp);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&v_full[s]), ph, abortp)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&p_full), j & 1, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + s * TILE);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t da = make_smem_desc(pa + (k / 4) * HALF + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(va + k * 2048, HALF, 1024);
          tc_mma_ss(tmem + O_COL, da, db, IDESC_O, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&v_empty[s]));
        tc_commit(smem_u32(&p_empty));
        if (j == n_tiles - 1) tc_commit(smem_u32(&o_full));
      }
      if (!ok) {
        atomicExch(p.status, STATUS_TIMEOUT_FULL);
        abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // row of the query tile == TMEM lane
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const int qpos = p.q_start + q0 + row;                // absolute position of this query
    const bool row_valid = (q0 + row) < p.T;
    const int wg = (warp - 2) >> 2;                       // group 0: key columns 0..63 of every tile, group 1: 64..127
    const float sink2 = p.sinks[head] * LOG2E;
    float m = sink2, l = wg == 0 ? 1.0f : 0.0f;           // the sink's unit weight is counted once; the groups' sums are added at the end
    bool failed = false;

    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int k0 = (jt_begin + j) * BKV;
      if (!mbar_wait(smem_u32(&s_full[s]), ph, abortp)) { failed = true; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_addr + S_COL0 + s * BKV;
      const bool need_mask = (k0 + BKV - 1 > qlo) || (p.window > 0 && k0 < qlo + BQ - p.window + 1) || (k0 + BKV > p.S);
      const int hi = min(qpos, p.S - 1);                               // last visible key
      const int lo = p.window > 0 ? qpos - p.window + 1 : 0;           // first visible key

      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = wg * (BKV / 64); c < (wg + 1) * (BKV / 64); ++c) {
        uint32_t r[32];
        tmem_ld32(s_addr + c * 32, r);
        tmem_ld_wait();
        if (!need_mask) {   // interior tile: the maximum of the raw scores, scaled once below (the scale is positive)
#pragma unroll
          for (int i = 0; i < 32; i += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kk = k0 + c * 32 + i;
            if (kk <= hi && kk >= lo) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        }
      }
      mx *= p.scale_log2;
      // the row maximum over all 128 columns: exchange the two halves (bounded wait, like every other wait here)
      xmax[s][wg][row] = mx;
      mbar_arrive(smem_u32(&x_full[s]));
      if (!mbar_wait(smem_u32(&x_full[s]), ph, abortp)) { failed = true; break; }
      mx = fmaxf(mx, xmax[s][wg ^ 1][row]);
      // lazy rescale: keep the old reference max unless the new one exceeds it by more than 2^8
      float factor = 1.0f;
      if (mx > m + 8.0f) {
        factor = exp2f(m - mx);
        m = mx;
      }
      l *= factor;
      // P(j-1) and the O accumulator must be retired before P is overwritten / O is rescaled
      if (j > 0) {
        if (!mbar_wait(smem_u32(&p_empty), (j - 1) & 1, abortp)) { failed = true; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, factor != 1.0f)) {
#pragma unroll 1
          for (int c = wg; c < D / 32; c += 2) {           // each group rescales half of the accumulator's columns
            uint32_t r[32];
            tmem_ld32(tmem + lane_addr + O_COL + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
            tmem_st32(tmem + lane_addr + O_COL + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      // pass 2: probabilities -> shared memory (bf16, K-major 128B swizzle), row sum
      float sum = 0.0f;
#pragma unroll 1
      for (int c = wg * (BKV / 64); c < (wg + 1) * (BKV / 64); ++c) {
        uint32_t r[32];
        tmem_ld32(s_addr + c * 32, r);
        tmem_ld_wait();
        float pv[32];
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            pv[i] = exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, -m));
            sum += pv[i];
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kk = k0 + c * 32 + i;
            pv[i] = (kk > hi || kk < lo) ? 0.f : exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, -m));
            sum += pv[i];
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c16 = c * 4 + q;
          uint4 o;
          o.x = pack_bf16(pv[q * 8 + 0], pv[q * 8 + 1]);
          o.y = pack_bf16(pv[q * 8 + 2], pv[q * 8 + 3]);
          o.z = pack_bf16(pv[q * 8 + 4], pv[q * 8 + 5]);
          o.w = pack_bf16(pv[q * 8 + 6], pv[q * 8 + 7]);
          *reinterpret_cast<uint4*>(sP + (c16 >> 3) * HALF + swz128(row, c16 & 7)) = o;
        }
      }
      l += sum;
      tc_fence_before();
      mbar_arrive(smem_u32(&s_empty[s]));
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&p_full));
    }

    // epilogue: O / l -> bf16, LSE
    if (!failed && n_tiles > 0) {
      if (!mbar_wait(smem_u32(&o_full), 0, abortp)) failed = true;
    }
    if (failed) {
      if (lane == 0) atomicExch(p.status, STATUS_TIMEOUT_TMEM);
      abort_flag = 1;
    } else {
      tc_fence_after();
      xl[wg][row] = l;                                      // add the two groups' partial row sums
      mbar_arrive(smem_u32(&l_full));
      if (!mbar_wait(smem_u32(&l_full), 0, abortp)) {
        if (lane == 0) atomicExch(p.status, STATUS_TIMEOUT_TMEM);
        abort_flag = 1;
      }
      l = xl[0][row] + xl[1][row];
      const float inv = 1.0f / l;
      __nv_bfloat16* orow = p.out + (((long long)b * p.T + (q0 + row)) * p.Nq + head) * D;
#pragma unroll 1
      for (int c = wg; c < D / 32; c += 2) {
        uint32_t r[32];
        if (n_tiles > 0) {
          tmem_ld32(tmem + lane_addr + O_COL + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * inv, __uint_as_float(r[q * 8 + 1]) * inv);
            o.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * inv, __uint_as_float(r[q * 8 + 3]) * inv);
            o.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * inv, __uint_as_float(r[q * 8 + 5]) * inv);
            o.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * inv, __uint_as_float(r[q * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
          }
        }
      }
      if (row_valid && wg == 0) p.lse[((long long)b * p.Nq + head) * p.T + q0 + row] = (m + log2f(l)) * LN2;
    }
  }
#undef FA_FAIL

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// 4-D map over a token-major [B, T, N, D] bf16 tensor with arbitrary (element) strides; box = 64 x 128 rows.
static int make_btnd_map(CUtensorMap* m, const void* ptr, int B, int T, int N, int D, long long sb, long long st, long long sn, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)T, (uint64_t)N, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)st * 2, (uint64_t)sn * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tmap(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace lyra

using namespace lyra;

// q [B,T,Nq,D], k/v [B,S,Nkv,D] given by (batch, token, head) element strides; the innermost stride is 1.
extern "C" int lyra_flash_fwd(const void* q, long long q_sb, long long q_st, long long q_sn,
                              const void* k, long long k_sb, long long k_st, long long k_sn,
                              const void* v, long long v_sb, long long v_st, long long v_sn,
                              const float* sinks, void* out, float* lse,
                              int B, int T, int S, int Nq, int Nkv, int D, float scale, int window, int q_start,
                              int* status, void* stream) {
  if (D != 64 && D != 128) return -20;
  CUtensorMap tq, tk, tv;
  if (make_btnd_map(&tq, q, B, T, Nq, D, q_sb, q_st, q_sn, 128)) return -21;
  if (make_btnd_map(&tk, k, B, S, Nkv, D, k_sb, k_st, k_sn, 128)) return -22;
  if (make_btnd_map(&tv, v, B, S, Nkv, D, v_sb, v_st, v_sn, 128)) return -23;
  FwdParams p;
  p.B = B; p.T = T; p.S = S; p.Nq = Nq; p.Nkv = Nkv; p.window = window; p.q_start = q_start;
  p.scale_log2 = scale * LOG2E; p.sinks = sinks; p.out = reinterpret_cast<__nv_bfloat16*>(out); p.lse = lse; p.status = status;
  dim3 grid((T + 127) / 128, Nq, B);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) {
    constexpr int smem = 6 * 128 * 128 * 2 + 1024;  // Q + 2K + 2V + P
    static bool once = false;
    if (!once) { if (cudaFuncSetAttribute(flash_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -24; once = true; }
    flash_fwd_kernel<128><<<grid, FA_THREADS, smem, s>>>(tq, tk, tv, p);
  } else {
    constexpr int smem = 5 * 128 * 64 * 2 + 128 * 128 * 2 + 1024;
    static bool once = false;
    if (!once) { if (cudaFuncSetAttribute(flash_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -24; once = true; }
    flash_fwd_kernel<64><<<grid, FA_THREADS, smem, s>>>(tq, tk, tv, p);
  }
  LYRA_CHECK_LAUNCH();
  return 0;
}
