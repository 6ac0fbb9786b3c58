// Flash attention backward for sm_100a (semantics of the reference's FLASH_ATTENTION_BWD_DQ / _DKV kernels
// and its dsinks reduction, lyra/kernels/flash_attention.py:377-659). Probabilities are recomputed from the
// stored LSE; dS = P o (dP - delta) with delta = rowsum(O o dO). Two deterministic kernels (no atomics):
//
//   dq  kernel: one CTA per (128-query tile, head, batch); per 64-key tile  S = Q K^T, dP = dO V^T (TMEM),
//               dS written in place over dP as bf16 and taken from TMEM by dQ += dS K (accumulator across key tiles);
//               two elementwise groups work on alternate key tiles.
//   dkv kernel: one CTA per (128-key tile, kv head, batch); loops over the GQA group's query heads and the
//               64-query tiles inside the band, working in the transposed orientation (keys on TMEM lanes):
//               S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q. Two elementwise groups take alternate
//               iterations, each with its own S^T / dP^T buffers in TMEM, which it turns in place into the bf16
//               P^T / dS^T operands of the accumulating products (no shared-memory staging).
// The same shared-memory tile serves as a K-major operand in one product and an MN-major operand in the other
// (e.g. K in S = Q K^T and in dQ = dS K), so every tile is loaded once per use by TMA.
#include "../common/sm100.cuh"
#include "../common/tmap.h"

namespace lyra {

constexpr int FB_THREADS = 320;   // dQ kernel: TMA warp, MMA warp and two groups of four elementwise warps (alternate key tiles)
constexpr int DKV_THREADS = 320;  // dK/dV kernel: the same roles, alternate iterations per group
constexpr float B_LOG2E = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------------- delta
// delta[b, h, t] = sum_d O[b,t,h,d] * dO[b,t,h,d]; one warp per (b, t, h) row.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                  int B, int T, int N, int D, long long do_sb, long long do_st, long long do_sn) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (long long)B * T * N) return;
  const int h = int(row % N);
  const long long bt = row / N;
  const int t = int(bt % T);
  const int b = int(bt / T);
  const __nv_bfloat16* po = o + row * D;
  const __nv_bfloat16* pd = d_o + b * do_sb + t * do_st + h * do_sn;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po + i));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd + i));
    acc += a.x * c.x + a.y * c.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[((long long)b * N + h) * T + t] = acc;
}

struct BwdParams {
  int B, T, S, Nq, Nkv, window, q_start;
  float scale, scale_log2;
  const float* lse;     // [B, Nq, T] natural log
  const float* delta;   // [B, Nq, T]
  __nv_bfloat16* dq;    // [B, T, Nq, D]
  __nv_bfloat16* dk;    // [B, S, Nkv, D]
  __nv_bfloat16* dv;    // [B, S, Nkv, D]
  int* status;
};

// ---------------------------------------------------------------------------------------------- dQ
constexpr int DQ_STAGES = 4;      // (K, V) tiles of 64 keys in flight

template <int D>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo, const BwdParams p) {
  constexpr int BQ = 128, BKV = 64;
  constexpr int TILE = BQ * D * 2;         // Q or dO tile
  constexpr int KTILE = BKV * D * 2;       // K or V tile of 64 keys
  constexpr int HALF = 128 * 128;          // one 64-column block of a 128-row tile
  constexpr int KHALF = 64 * 128;          // one 64-column block of a 64-row tile
  constexpr uint32_t TMEM_COLS = 512, S_COL = 0, DP_COL = 128, DQ_COL = 256;   // S of group 0 / 1 at 0 / 64, dP at 128 / 192
  constexpr uint32_t QA_COL = 384, DOA_COL = 384 + D / 2;                      // Q and dO as packed bf16 TMEM operands (D / 2 columns each)
  constexpr uint32_t IDESC_S = make_idesc(BQ, BKV, 1, 1, 0, 0);
  constexpr uint32_t IDESC_DQ = make_idesc(BQ, D, 1, 1, 0, 1);                 // dS (TMEM) x K (MN-major)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + TILE;
  uint8_t* sKV = sDO + TILE;          // DQ_STAGES x (K, V)
  __shared__ uint64_t q_full, a_full, kv_full[DQ_STAGES], kv_empty[DQ_STAGES], sdp_full[2], ds_full[2], dq_full;
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // late query tiles see the most keys: they come first in launch order
  const int per_qt = p.Nq * p.B, n_qt = (p.T + BQ - 1) / BQ;
  const int q0 = (n_qt - 1 - int(blockIdx.x) / per_qt) * BQ, head = (int(blockIdx.x) % per_qt) % p.Nq, b = (int(blockIdx.x) % per_qt) / p.Nq;
  const int kvh = head / (p.Nq / p.Nkv);
  const int qlo = p.q_start + q0;
  const int qhi = min(p.q_start + min(q0 + BQ, p.T) - 1, p.S - 1);
  const int klo = p.window > 0 ? max(0, qlo - p.window + 1) : 0;
  const int jt_begin = klo / BKV;
  const int n_tiles = qhi < 0 ? 0 : max(qhi / BKV + 1 - jt_begin, 0);

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < DQ_STAGES; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&sdp_full[g]), 1);
      mbar_init(smem_u32(&ds_full[g]), 128);
    }
    mbar_init(smem_u32(&dq_full), 1);
    mbar_init(smem_u32(&a_full), 256);
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

  // Q and dO are the fixed operands of every S = Q K^T and dP = dO V^T of this CTA. They are copied once from their shared-memory
  // tiles into TMEM (group 0 copies Q, group 1 dO) and the products take them from there: an SS product of a 128-row tile with a
  // 64-column B needs 6 KB of shared-memory operands per instruction (48 clk at 128 B/clk against 32 clk of math); with A in
  // TMEM it needs 2 KB.
  // Key tile j (64 keys) belongs to elementwise group j & 1; each group has its own S / dP buffers and turns dP in place into the
  // bf16 dS operand of dQ += dS K, so the groups never wait for each other and the tensor core always has the other group's work.
  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(smem_u32(&q_full), 2 * TILE);
      for (int h = 0; h < D / 64; ++h) {
        tma_load_4d(smem_u32(sQ + h * HALF), &tq, smem_u32(&q_full), h * 64, q0, head, b);
        tma_load_4d(smem_u32(sDO + h * HALF), &tdo, smem_u32(&q_full), h * 64, q0, head, b);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % DQ_STAGES;
        const uint32_t ph = (j / DQ_STAGES) & 1;
        const int k0 = (jt_begin + j) * BKV;
        if (!mbar_wait(smem_u32(&kv_empty[s]), ph ^ 1, abortp)) {
          atomicCAS(p.status, 0, STATUS_TIMEOUT_EMPTY);
          abort_flag = 1;
          break;
        }
        mbar_expect_tx(smem_u32(&kv_full[s]), 2 * KTILE);
        for (int h = 0; h < D / 64; ++h) {
          tma_load_4d(smem_u32(sKV + (2 * s) * KTILE + h * KHALF), &tk, smem_u32(&kv_full[s]), h * 64, k0, kvh, b);
          tma_load_4d(smem_u32(sKV + (2 * s + 1) * KTILE + h * KHALF), &tv, smem_u32(&kv_full[s]), h * 64, k0, kvh, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      // MMAs of one thread retire in issue order: dP_g(j + 2) is issued after dQ += dS_g(j) K_j, so it cannot overwrite dS_g(j) early
      const uint64_t dk0 = make_smem_desc(smem_u32(sKV), 16, 1024);          // K of stage 0 as the K-major operand of S
      const uint64_t dkmn0 = make_smem_desc(smem_u32(sKV), KHALF, 1024);     // the same tile as the MN-major operand of dQ += dS K
      auto issue_s = [&](int j) -> bool {
        const int s = j % DQ_STAGES, g = j & 1;
        if (!mbar_wait(smem_u32(&kv_full[s]), (j / DQ_STAGES) & 1, abortp)) return false;
        tc_fence_after();
        const uint64_t dk = desc_advance(dk0, (2 * s) * KTILE), dv = desc_advance(dk0, (2 * s + 1) * KTILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)       // 16 values of d = 8 TMEM columns of the resident operand
          tc_mma_ts(tmem + S_COL + g * BKV, tmem + QA_COL + k * 8, desc_advance(dk, (k / 4) * KHALF + (k % 4) * 32), IDESC_S, k > 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          tc_mma_ts(tmem + DP_COL + g * BKV, tmem + DOA_COL + k * 8, desc_advance(dv, (k / 4) * KHALF + (k % 4) * 32), IDESC_S, k > 0);
        tc_commit(smem_u32(&sdp_full[g]));
        return true;
      };
      bool ok = mbar_wait(smem_u32(&a_full), 0, abortp);
      if (ok) ok = issue_s(0);
      if (ok && n_tiles > 1) ok = issue_s(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % DQ_STAGES, g = j & 1;
        if (!mbar_wait(smem_u32(&ds_full[g]), (j >> 1) & 1, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint64_t dkmn = desc_advance(dkmn0, (2 * s) * KTILE);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)     // 16 keys of dS = 8 TMEM columns of packed bf16 pairs
          tc_mma_ts(tmem + DQ_COL, tmem + DP_COL + g * BKV + k * 8, desc_advance(dkmn, k * 2048), IDESC_DQ, (j > 0 || k > 0) ? 1u : 0u);
        tc_commit(smem_u32(&kv_empty[s]));
        if (j + 2 < n_tiles) ok = issue_s(j + 2);
      }
      if (ok) tc_commit(smem_u32(&dq_full));
      if (!ok) {
        atomicCAS(p.status, 0, STATUS_TIMEOUT_FULL);
        abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int g = (warp - 2) >> 2;                        // group 0: key tiles 0, 2, 4, ...; group 1: 1, 3, 5, ...
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + S_COL + g * BKV, dp_addr = tmem + lane_addr + DP_COL + g * BKV;
    const int qpos = p.q_start + q0 + row;
    const bool row_valid = (q0 + row) < p.T;
    const long long stat_idx = ((long long)b * p.Nq + head) * p.T + q0 + row;
    const float lse2 = row_valid ? p.lse[stat_idx] * B_LOG2E : INFINITY;
    const float delta = row_valid ? p.delta[stat_idx] : 0.f;
    const int hi = min(qpos, p.S - 1);
    const int lo = p.window > 0 ? qpos - p.window + 1 : 0;
    bool failed = false;
    if (n_tiles > 0) {
      // this thread's row of Q (group 0) or dO (group 1): 128-byte-swizzled shared memory -> packed bf16 pairs in TMEM
      if (!mbar_wait(smem_u32(&q_full), 0, abortp)) failed = true;
      if (!failed) {
        const uint8_t* tile = g == 0 ? sQ : sDO;
        const uint32_t a_addr = tmem + lane_addr + (g == 0 ? QA_COL : DOA_COL);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          uint32_t v[32];
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint4 x = *reinterpret_cast<const uint4*>(tile + h * HALF + swz128(row, ch));
            v[ch * 4 + 0] = x.x; v[ch * 4 + 1] = x.y; v[ch * 4 + 2] = x.z; v[ch * 4 + 3] = x.w;
          }
          tmem_st32(a_addr + h * 32, v);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      mbar_arrive(smem_u32(&a_full));
    }
    for (int j = g; j < n_tiles && !failed; j += 2) {
      const int k0 = (jt_begin + j) * BKV;
      if (!mbar_wait(smem_u32(&sdp_full[g]), (j >> 1) & 1, abortp)) { failed = true; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t rs[32], rp[32], pd[16];
        tmem_ld32(s_addr + c * 32, rs);
        tmem_ld32(dp_addr + c * 32, rp);
        tmem_ld_wait();
        const int kfirst = k0 + c * 32;
        if (kfirst >= lo && kfirst + 31 <= hi) {           // whole chunk visible (all but the diagonal / band-edge tiles)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2));
            const float p1 = exp2f(fmaf(__uint_as_float(rs[i + 1]), p.scale_log2, -lse2));
            pd[i >> 1] = pack_bf16(p0 * (__uint_as_float(rp[i]) - delta), p1 * (__uint_as_float(rp[i + 1]) - delta));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int kk = kfirst + i;
            const float p0 = (kk > hi || kk < lo) ? 0.f : exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2));
            const float p1 = (kk + 1 > hi || kk + 1 < lo) ? 0.f : exp2f(fmaf(__uint_as_float(rs[i + 1]), p.scale_log2, -lse2));
            pd[i >> 1] = pack_bf16(p0 * (__uint_as_float(rp[i]) - delta), p1 * (__uint_as_float(rp[i + 1]) - delta));
          }
        }
        tmem_st16(dp_addr + c * 16, pd);                  // in place: column j holds keys 2j and 2j+1, both read above
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&ds_full[g]));
    }
    if (!failed && n_tiles > 0 && !mbar_wait(smem_u32(&dq_full), 0, abortp)) failed = true;
    if (failed) {
      if (lane == 0) atomicCAS(p.status, 0, STATUS_TIMEOUT_TMEM);
      abort_flag = 1;
    } else {
      tc_fence_after();
      __nv_bfloat16* orow = p.dq + (((long long)b * p.T + (q0 + row)) * p.Nq + head) * D;
#pragma unroll 1
      for (int c = g; c < D / 32; c += 2) {
        uint32_t r[32];
        if (n_tiles > 0) {
          tmem_ld32(tmem + lane_addr + DQ_COL + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * p.scale, __uint_as_float(r[q * 8 + 1]) * p.scale);
            o.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * p.scale, __uint_as_float(r[q * 8 + 3]) * p.scale);
            o.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * p.scale, __uint_as_float(r[q * 8 + 5]) * p.scale);
            o.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * p.scale, __uint_as_float(r[q * 8 + 7]) * p.scale);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
          }
        }
      }
    }
  }

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

// ---------------------------------------------------------------------------------------------- dK, dV
constexpr int DKV_STAGES = 4;     // (Q, dO) tiles in flight: the loads run two iterations ahead of the products that free a stage

template <int D>
__global__ void __launch_bounds__(DKV_THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo, const BwdParams p) {
  constexpr int BKV = 128, BQ = 64;
  constexpr int KTILE = BKV * D * 2;       // K or V tile
  constexpr int QTILE = BQ * D * 2;        // Q or dO tile
  constexpr int KHALF = 128 * 128;         // one 64-column block of a 128-row tile
  constexpr int QHALF = 64 * 128;          // one 64-column block of a 64-row tile
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t ST_COL = 0;           // S^T of group 0 / 1 at 0 / 64; dP^T at 128 / 192
  constexpr uint32_t DPT_COL = 128, DK_COL = 256, DV_COL = 384;
  constexpr uint32_t IDESC_ST = make_idesc(BKV, BQ, 1, 1, 0, 0);   // K (K-major) x Q (K-major) -> [keys, q]
  constexpr uint32_t IDESC_ACC = make_idesc(BKV, D, 1, 1, 0, 1);   // P^T (TMEM) x dO/Q (MN-major) -> [keys, d]

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + KTILE;
  uint8_t* sQD = sV + KTILE;               // DKV_STAGES x (Q, dO)
  __shared__ uint64_t kv_full, qd_full[DKV_STAGES], qd_empty[DKV_STAGES], st_full[2], stat_full[2], pt_full[2], acc_full;
  __shared__ __align__(16) float s_lse2[2][2][BQ], s_delta[2][2][BQ];     // [group][iteration parity][query]
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // early key tiles are seen by the most queries: they come first in launch order, so the long CTAs start first
  const int per_kt = p.Nkv * p.B;
  const int k0 = (int(blockIdx.x) / per_kt) * BKV, kvh = (int(blockIdx.x) % per_kt) % p.Nkv, b = (int(blockIdx.x) % per_kt) / p.Nkv;
  const int rep = p.Nq / p.Nkv;
  // queries (indices into T) whose band touches keys [k0, k0 + 127]
  const int khi = min(k0 + BKV, p.S) - 1;
  int qi_lo = max(k0 - p.q_start, 0);
  int qi_hi = p.T - 1;
  if (p.window > 0) qi_hi = min(qi_hi, khi + p.window - 1 - p.q_start);
  const int it_begin = qi_lo / BQ;
  const int tiles_per_head = (qi_hi >= qi_lo) ? (qi_hi / BQ + 1 - it_begin) : 0;
  const int n_iter = tiles_per_head * rep;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&kv_full), 1);
    for (int s = 0; s < DKV_STAGES; ++s) {
      mbar_init(smem_u32(&qd_full[s]), 1);
      mbar_init(smem_u32(&qd_empty[s]), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&st_full[g]), 1);
      mbar_init(smem_u32(&stat_full[g]), 128);
      mbar_init(smem_u32(&pt_full[g]), 128);
    }
    mbar_init(smem_u32(&acc_full), 1);
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

  // Iteration `it` (one 64-query tile of one head of the GQA group) belongs to elementwise group it & 1. The groups never meet:
  // each has its own S^T / dP^T buffers, turns them in place into bf16 P^T / dS^T (two values per 32-bit column), and the two
  // accumulating products take those as their TMEM operand. While a group exponentiates, the tensor core works for the other one.
  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(smem_u32(&kv_full), 2 * KTILE);
      for (int h = 0; h < D / 64; ++h) {
        tma_load_4d(smem_u32(sK + h * KHALF), &tk, smem_u32(&kv_full), h * 64, k0, kvh, b);
        tma_load_4d(smem_u32(sV + h * KHALF), &tv, smem_u32(&kv_full), h * 64, k0, kvh, b);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % DKV_STAGES;
        const uint32_t ph = (it / DKV_STAGES) & 1;
        const int head = kvh * rep + it / tiles_per_head;
        const int qi0 = (it_begin + it % tiles_per_head) * BQ;
        if (!mbar_wait(smem_u32(&qd_empty[s]), ph ^ 1, abortp)) {
          atomicCAS(p.status, 0, STATUS_TIMEOUT_EMPTY);
          abort_flag = 1;
          break;
        }
        mbar_expect_tx(smem_u32(&qd_full[s]), 2 * QTILE);
        for (int h = 0; h < D / 64; ++h) {
          tma_load_4d(smem_u32(sQD + (2 * s) * QTILE + h * QHALF), &tq, smem_u32(&qd_full[s]), h * 64, qi0, head, b);
          tma_load_4d(smem_u32(sQD + (2 * s + 1) * QTILE + h * QHALF), &tdo, smem_u32(&qd_full[s]), h * 64, qi0, head, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      // MMAs of one thread retire in issue order: S^T_g(it + 2) is issued after the products that read P^T_g(it) / dS^T_g(it),
      // so the in-place operands cannot be overwritten early.
      const uint64_t dk0 = make_smem_desc(smem_u32(sK), 16, 1024), dv0 = make_smem_desc(smem_u32(sV), 16, 1024);
      const uint64_t dq0 = make_smem_desc(smem_u32(sQD), 16, 1024);          // Q of stage 0 as the K-major operand of S^T
      const uint64_t dqmn0 = make_smem_desc(smem_u32(sQD), QHALF, 1024);     // the same tile as the MN-major operand of dK += dS^T Q
      auto issue_st = [&](int it) -> bool {
        const int s = it % DKV_STAGES, g = it & 1;
        if (!mbar_wait(smem_u32(&qd_full[s]), (it / DKV_STAGES) & 1, abortp)) return false;
        tc_fence_after();
        const uint64_t dq = desc_advance(dq0, (2 * s) * QTILE), ddo = desc_advance(dq0, (2 * s + 1) * QTILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          tc_mma_ss(tmem + ST_COL + g * BQ, desc_advance(dk0, (k / 4) * KHALF + (k % 4) * 32), desc_advance(dq, (k / 4) * QHALF + (k % 4) * 32), IDESC_ST, k > 0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          tc_mma_ss(tmem + DPT_COL + g * BQ, desc_advance(dv0, (k / 4) * KHALF + (k % 4) * 32), desc_advance(ddo, (k / 4) * QHALF + (k % 4) * 32), IDESC_ST, k > 0);
        tc_commit(smem_u32(&st_full[g]));
        return true;
      };
      bool ok = mbar_wait(smem_u32(&kv_full), 0, abortp);
      if (ok) ok = issue_st(0);
      if (ok && n_iter > 1) ok = issue_st(1);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % DKV_STAGES, g = it & 1;
        if (!mbar_wait(smem_u32(&pt_full[g]), (it >> 1) & 1, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint64_t dqmn = desc_advance(dqmn0, (2 * s) * QTILE), ddomn = desc_advance(dqmn0, (2 * s + 1) * QTILE);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)    // dV += P^T dO   (16 queries of P^T = 8 TMEM columns)
          tc_mma_ts(tmem + DV_COL, tmem + ST_COL + g * BQ + k * 8, desc_advance(ddomn, k * 2048), IDESC_ACC, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k)    // dK += dS^T Q
          tc_mma_ts(tmem + DK_COL, tmem + DPT_COL + g * BQ + k * 8, desc_advance(dqmn, k * 2048), IDESC_ACC, (it > 0 || k > 0) ? 1u : 0u);
        tc_commit(smem_u32(&qd_empty[s]));
        if (it + 2 < n_iter) ok = issue_st(it + 2);
      }
      if (ok) tc_commit(smem_u32(&acc_full));
      if (!ok) {
        atomicCAS(p.status, 0, STATUS_TIMEOUT_FULL);
        abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // key row == TMEM lane
    const int g = (warp - 2) >> 2;                        // group 0: iterations 0, 2, 4, ...; group 1: 1, 3, 5, ...
    const int gt = (threadIdx.x - 64) & 127;              // 0..127 inside the group
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const uint32_t st_addr = tmem + lane_addr + ST_COL + g * BQ, dpt_addr = tmem + lane_addr + DPT_COL + g * BQ;
    const int kk = k0 + row;
    const bool key_valid = kk < p.S;
    bool failed = false;
    // per-query statistics of iteration `it`: the first 64 threads of the group fetch the log-sum-exp, the others delta, one of
    // the group's iterations ahead, so that the global-load latency is off the critical path
    auto load_stat = [&](int it) -> float {
      const int head = kvh * rep + it / tiles_per_head;
      const int qi = (it_begin + it % tiles_per_head) * BQ + (gt & 63);
      const long long idx = ((long long)b * p.Nq + head) * p.T + qi;
      if (gt < 64) return qi < p.T ? p.lse[idx] * B_LOG2E : INFINITY;
      return qi < p.T ? p.delta[idx] : 0.f;
    };
    float stat = g < n_iter ? load_stat(g) : 0.f;
    for (int it = g; it < n_iter; it += 2) {
      const int par = (it >> 1) & 1;
      const int qi0 = (it_begin + it % tiles_per_head) * BQ;
      // publish this iteration's statistics (buffer `par`: its readers of two iterations ago passed pt_full since)
      if (gt < 64) s_lse2[g][par][gt] = stat;
      else s_delta[g][par][gt - 64] = stat;
      mbar_arrive(smem_u32(&stat_full[g]));
      if (it + 2 < n_iter) stat = load_stat(it + 2);
      if (!mbar_wait(smem_u32(&stat_full[g]), par, abortp)) { failed = true; break; }
      if (!mbar_wait(smem_u32(&st_full[g]), par, abortp)) { failed = true; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < BQ / 32; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld32(st_addr + c * 32, rs);
        tmem_ld32(dpt_addr + c * 32, rp);
        tmem_ld_wait();
        const float* lse_c = &s_lse2[g][par][c * 32];
        const float* del_c = &s_delta[g][par][c * 32];
        uint32_t pp[16], pd[16];
        const int qfirst = p.q_start + qi0 + c * 32;
        if (key_valid && kk <= qfirst && (p.window == 0 || kk > qfirst + 31 - p.window)) {   // whole chunk visible
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse_c[i]));
            const float p1 = exp2f(fmaf(__uint_as_float(rs[i + 1]), p.scale_log2, -lse_c[i + 1]));
            pp[i >> 1] = pack_bf16(p0, p1);
            pd[i >> 1] = pack_bf16(p0 * (__uint_as_float(rp[i]) - del_c[i]), p1 * (__uint_as_float(rp[i + 1]) - del_c[i + 1]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int qpos = qfirst + i;
            const bool v0 = key_valid && kk <= qpos && (p.window == 0 || kk > qpos - p.window);
            const bool v1 = key_valid && kk <= qpos + 1 && (p.window == 0 || kk > qpos + 1 - p.window);
            const float p0 = v0 ? exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse_c[i])) : 0.f;
            const float p1 = v1 ? exp2f(fmaf(__uint_as_float(rs[i + 1]), p.scale_log2, -lse_c[i + 1])) : 0.f;
            pp[i >> 1] = pack_bf16(p0, p1);
            pd[i >> 1] = pack_bf16(p0 * (__uint_as_float(rp[i]) - del_c[i]), p1 * (__uint_as_float(rp[i + 1]) - del_c[i + 1]));
          }
        }
        // in place: column j of the bf16 operand holds queries 2j and 2j+1, whose fp32 columns were read above
        tmem_st16(st_addr + c * 16, pp);
        tmem_st16(dpt_addr + c * 16, pd);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&pt_full[g]));
    }
    if (!failed && n_iter > 0 && !mbar_wait(smem_u32(&acc_full), 0, abortp)) failed = true;
    if (failed) {
      if (lane == 0) atomicCAS(p.status, 0, STATUS_TIMEOUT_TMEM);
      abort_flag = 1;
    } else {
      tc_fence_after();
      const long long o_off = (((long long)b * p.S + kk) * p.Nkv + kvh) * D;
      {
        const int which = g;                              // group 0 writes dK, group 1 writes dV
        __nv_bfloat16* orow = (which == 0 ? p.dk : p.dv) + o_off;
        const float mul = which == 0 ? p.scale : 1.0f;
        const uint32_t col0 = which == 0 ? DK_COL : DV_COL;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          if (n_iter > 0) {
            tmem_ld32(tmem + lane_addr + col0 + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          if (key_valid) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(r[q * 8 + 0]) * mul, __uint_as_float(r[q * 8 + 1]) * mul);
              o.y = pack_bf16(__uint_as_float(r[q * 8 + 2]) * mul, __uint_as_float(r[q * 8 + 3]) * mul);
              o.z = pack_bf16(__uint_as_float(r[q * 8 + 4]) * mul, __uint_as_float(r[q * 8 + 5]) * mul);
              o.w = pack_bf16(__uint_as_float(r[q * 8 + 6]) * mul, __uint_as_float(r[q * 8 + 7]) * mul);
              *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o;
            }
          }
        }
      }
    }
  }

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

static int bwd_map(CUtensorMap* m, const void* ptr, int B, int T, int N, int D, long long sb, long long st, long long sn, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)T, (uint64_t)N, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)st * 2, (uint64_t)sn * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tmap(m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int D>
static int launch_bwd(const void* q, const long long* qs, const void* k, const long long* ks, const void* v, const long long* vs,
                      const void* d_o, const long long* dos, const BwdParams& p, cudaStream_t s) {
  CUtensorMap tq, tk, tv, tdo, tq64, tdo64, tk64, tv64;
  if (bwd_map(&tq, q, p.B, p.T, p.Nq, D, qs[0], qs[1], qs[2], 128)) return -31;
  if (bwd_map(&tk, k, p.B, p.S, p.Nkv, D, ks[0], ks[1], ks[2], 128)) return -32;
  if (bwd_map(&tv, v, p.B, p.S, p.Nkv, D, vs[0], vs[1], vs[2], 128)) return -33;
  if (bwd_map(&tdo, d_o, p.B, p.T, p.Nq, D, dos[0], dos[1], dos[2], 128)) return -34;
  if (bwd_map(&tq64, q, p.B, p.T, p.Nq, D, qs[0], qs[1], qs[2], 64)) return -35;
  if (bwd_map(&tdo64, d_o, p.B, p.T, p.Nq, D, dos[0], dos[1], dos[2], 64)) return -36;
  if (bwd_map(&tk64, k, p.B, p.S, p.Nkv, D, ks[0], ks[1], ks[2], 64)) return -32;
  if (bwd_map(&tv64, v, p.B, p.S, p.Nkv, D, vs[0], vs[1], vs[2], 64)) return -33;
  constexpr int smem_dq = 2 * 128 * D * 2 + DQ_STAGES * 2 * 64 * D * 2 + 1024;          // Q, dO, stages of (K, V)
  constexpr int smem_dkv = 2 * 128 * D * 2 + DKV_STAGES * 2 * 64 * D * 2 + 1024;      // K, V, stages of (Q, dO)
  static bool once = false;
  if (!once) {
    if (cudaFuncSetAttribute(flash_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq) != cudaSuccess) return -37;
    if (cudaFuncSetAttribute(flash_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkv) != cudaSuccess) return -38;
    once = true;
  }
  flash_bwd_dq_kernel<D><<<dim3(((p.T + 127) / 128) * p.Nq * p.B), FB_THREADS, smem_dq, s>>>(tq, tk64, tv64, tdo, p);
  flash_bwd_dkv_kernel<D><<<dim3(((p.S + 127) / 128) * p.Nkv * p.B), DKV_THREADS, smem_dkv, s>>>(tq64, tk, tv, tdo64, p);
  return 0;
}

}  // namespace lyra

using namespace lyra;

// strides arrays: {batch, token, head} element strides of q / k / v / dO (token-major, unit inner stride).
// out [B,T,Nq,D] contiguous; dq/dk/dv contiguous token-major outputs; delta is a [B,Nq,T] fp32 workspace.
extern "C" int lyra_flash_bwd(const void* q, const long long* qs, const void* k, const long long* ks, const void* v, const long long* vs,
                              const void* out, const void* d_o, const long long* dos, const float* lse, float* delta,
                              void* dq, void* dk, void* dv,
                              int B, int T, int S, int Nq, int Nkv, int D, float scale, int window, int q_start,
                              int* status, void* stream) {
  if (D != 64 && D != 128) return -30;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * T * Nq;
  attn_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                                                reinterpret_cast<const __nv_bfloat16*>(d_o), delta, B, T, Nq, D, dos[0], dos[1], dos[2]);
  BwdParams p;
  p.B = B; p.T = T; p.S = S; p.Nq = Nq; p.Nkv = Nkv; p.window = window; p.q_start = q_start;
  p.scale = scale; p.scale_log2 = scale * B_LOG2E; p.lse = lse; p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq); p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.status = status;
  int rc = D == 128 ? launch_bwd<128>(q, qs, k, ks, v, vs, d_o, dos, p, s) : launch_bwd<64>(q, qs, k, ks, v, vs, d_o, dos, p, s);
  if (rc) return rc;
  LYRA_CHECK_LAUNCH();
  return 0;
}
