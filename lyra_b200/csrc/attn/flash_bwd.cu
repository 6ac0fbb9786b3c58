// Flash attention backward for sm_100a (semantics of the reference's FLASH_ATTENTION_BWD_DQ / _DKV kernels
// and its dsinks reduction, lyra/kernels/flash_attention.py:377-659). Probabilities are recomputed from the
// stored LSE; dS = P o (dP - delta) with delta = rowsum(O o dO). Two deterministic kernels (no atomics):
//
//   dq  kernel: one CTA per (128-query tile, head, batch); per key tile  S = Q K^T, dP = dO V^T (TMEM),
//               dS -> bf16 shared memory, dQ += dS K (TMEM accumulator across key tiles).
//   dkv kernel: one CTA per (128-key tile, kv head, batch); loops over the GQA group's query heads and the
//               64-query tiles inside the band, working in the transposed orientation (keys on TMEM lanes):
//               S^T = K Q^T, dP^T = V dO^T, dV += P^T dO, dK += dS^T Q. S^T/dP^T are double-buffered in TMEM.
// The same shared-memory tile serves as a K-major operand in one product and an MN-major operand in the other
// (e.g. K in S = Q K^T and in dQ = dS K), so every tile is loaded once per use by TMA.
#include "../common/sm100.cuh"
#include "../common/tmap.h"

namespace lyra {

constexpr int FB_THREADS = 320;   // dQ kernel: TMA warp, MMA warp and two groups of four elementwise warps (two 32-key chunks of a tile each)
constexpr int DKV_THREADS = 320;  // dK/dV kernel: the same roles, one 32-query chunk of a tile per group
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
template <int D>
__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo, const BwdParams p) {
  constexpr int BQ = 128, BKV = 128;
  constexpr int TILE = BQ * D * 2;
  constexpr int HALF = 128 * 128;
  constexpr uint32_t TMEM_COLS = 512, S_COL = 0, DP_COL = 128, DQ_COL = 256;
  constexpr uint32_t IDESC_S = make_idesc(BQ, BKV, 1, 1, 0, 0);
  constexpr uint32_t IDESC_DQ = make_idesc(BQ, D, 1, 1, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + TILE;
  uint8_t* sKV = sDO + TILE;          // 2 stages x (K, V)
  uint8_t* sDS = sKV + 4 * TILE;
  __shared__ uint64_t q_full, kv_full[2], kv_empty[2], sdp_full, sdp_empty, ds_full, ds_empty, dq_full;
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ, head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / (p.Nq / p.Nkv);
  const int qlo = p.q_start + q0;
  const int qhi = min(p.q_start + min(q0 + BQ, p.T) - 1, p.S - 1);
  const int klo = p.window > 0 ? max(0, qlo - p.window + 1) : 0;
  const int jt_begin = klo / BKV;
  const int n_tiles = qhi < 0 ? 0 : max(qhi / BKV + 1 - jt_begin, 0);

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    mbar_init(smem_u32(&sdp_full), 1);
    mbar_init(smem_u32(&sdp_empty), 256);
    mbar_init(smem_u32(&ds_full), 256);
    mbar_init(smem_u32(&ds_empty), 1);
    mbar_init(smem_u32(&dq_full), 1);
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

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(smem_u32(&q_full), 2 * TILE);
      for (int h = 0; h < D / 64; ++h) {
        tma_load_4d(smem_u32(sQ + h * HALF), &tq, smem_u32(&q_full), h * 64, q0, head, b);
        tma_load_4d(smem_u32(sDO + h * HALF), &tdo, smem_u32(&q_full), h * 64, q0, head, b);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int k0 = (jt_begin + j) * BKV;
        if (!mbar_wait(smem_u32(&kv_empty[s]), ph ^ 1, abortp)) {
          atomicExch(p.status, STATUS_TIMEOUT_EMPTY);
          abort_flag = 1;
          break;
        }
        mbar_expect_tx(smem_u32(&kv_full[s]), 2 * TILE);
        for (int h = 0; h < D / 64; ++h) {
          tma_load_4d(smem_u32(sKV + (2 * s) * TILE + h * HALF), &tk, smem_u32(&kv_full[s]), h * 64, k0, kvh, b);
          tma_load_4d(smem_u32(sKV + (2 * s + 1) * TILE + h * HALF), &tv, smem_u32(&kv_full[s]), h * 64, k0, kvh, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      bool ok = mbar_wait(smem_u32(&q_full), 0, abortp);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&kv_full[s]), ph, abortp)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&sdp_empty), (j & 1) ^ 1, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), doa = smem_u32(sDO);
        const uint32_t ka = smem_u32(sKV + (2 * s) * TILE), va = smem_u32(sKV + (2 * s + 1) * TILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * HALF + (k % 4) * 32;
          tc_mma_ss(tmem + S_COL, make_smem_desc(qa + off, 16, 1024), make_smem_desc(ka + off, 16, 1024), IDESC_S, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * HALF + (k % 4) * 32;
          tc_mma_ss(tmem + DP_COL, make_smem_desc(doa + off, 16, 1024), make_smem_desc(va + off, 16, 1024), IDESC_S, k > 0);
        }
        tc_commit(smem_u32(&sdp_full));
        // dQ += dS K once the softmax threads have written dS
        if (!mbar_wait(smem_u32(&ds_full), j & 1, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint32_t dsa = smem_u32(sDS);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t da = make_smem_desc(dsa + (k / 4) * HALF + (k % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(ka + k * 2048, HALF, 1024);
          tc_mma_ss(tmem + DQ_COL, da, db, IDESC_DQ, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&kv_empty[s]));
        tc_commit(smem_u32(&ds_empty));
        if (j == n_tiles - 1) tc_commit(smem_u32(&dq_full));
      }
      if (!ok) {
        atomicExch(p.status, STATUS_TIMEOUT_FULL);
        abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int wg = (warp - 2) >> 2;                       // two groups of four warps share each tile's key columns
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const int qpos = p.q_start + q0 + row;
    const bool row_valid = (q0 + row) < p.T;
    const long long stat_idx = ((long long)b * p.Nq + head) * p.T + q0 + row;
    const float lse2 = row_valid ? p.lse[stat_idx] * B_LOG2E : INFINITY;
    const float delta = row_valid ? p.delta[stat_idx] : 0.f;
    bool failed = false;
    for (int j = 0; j < n_tiles; ++j) {
      const int k0 = (jt_begin + j) * BKV;
      if (!mbar_wait(smem_u32(&sdp_full), j & 1, abortp)) { failed = true; break; }
      if (j > 0 && !mbar_wait(smem_u32(&ds_empty), (j - 1) & 1, abortp)) { failed = true; break; }
      tc_fence_after();
      const int hi = min(qpos, p.S - 1);
      const int lo = p.window > 0 ? qpos - p.window + 1 : 0;
#pragma unroll 1
      for (int c = wg * (BKV / 64); c < (wg + 1) * (BKV / 64); ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld32(tmem + lane_addr + S_COL + c * 32, rs);
        tmem_ld32(tmem + lane_addr + DP_COL + c * 32, rp);
        tmem_ld_wait();
        float ds[32];
        const int kfirst = k0 + c * 32;
        if (kfirst >= lo && kfirst + 31 <= hi) {           // whole chunk visible (all but the diagonal / band-edge tiles)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float pr = exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2));
            ds[i] = pr * (__uint_as_float(rp[i]) - delta);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kk = kfirst + i;
            const float pr = (kk > hi || kk < lo) ? 0.f : exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2));
            ds[i] = pr * (__uint_as_float(rp[i]) - delta);
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c16 = c * 4 + q;
          uint4 o;
          o.x = pack_bf16(ds[q * 8 + 0], ds[q * 8 + 1]);
          o.y = pack_bf16(ds[q * 8 + 2], ds[q * 8 + 3]);
          o.z = pack_bf16(ds[q * 8 + 4], ds[q * 8 + 5]);
          o.w = pack_bf16(ds[q * 8 + 6], ds[q * 8 + 7]);
          *reinterpret_cast<uint4*>(sDS + (c16 >> 3) * HALF + swz128(row, c16 & 7)) = o;
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&sdp_empty));
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&ds_full));
    }
    if (!failed && n_tiles > 0 && !mbar_wait(smem_u32(&dq_full), 0, abortp)) failed = true;
    if (failed) {
      if (lane == 0) atomicExch(p.status, STATUS_TIMEOUT_TMEM);
      abort_flag = 1;
    } else {
      tc_fence_after();
      __nv_bfloat16* orow = p.dq + (((long long)b * p.T + (q0 + row)) * p.Nq + head) * D;
#pragma unroll 1
      for (int c = wg; c < D / 32; c += 2) {
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
template <int D>
__global__ void __launch_bounds__(DKV_THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo, const BwdParams p) {
  constexpr int BKV = 128, BQ = 64;
  constexpr int KTILE = BKV * D * 2;       // K or V tile
  constexpr int QTILE = BQ * D * 2;        // Q or dO tile
  constexpr int KHALF = 128 * 128;         // one 64-column block of a 128-row tile
  constexpr int QHALF = 64 * 128;          // one 64-column block of a 64-row tile
  constexpr int PT_BYTES = BKV * BQ * 2;   // P^T / dS^T tile: 128 rows x 128 B
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t ST_COL = 0;           // S^T buffers at 0, 64; dP^T buffers at 128, 192
  constexpr uint32_t DPT_COL = 128, DK_COL = 256, DV_COL = 384;
  constexpr uint32_t IDESC_ST = make_idesc(BKV, BQ, 1, 1, 0, 0);   // K (K-major) x Q (K-major) -> [keys, q]
  constexpr uint32_t IDESC_ACC = make_idesc(BKV, D, 1, 1, 0, 1);   // P^T (K-major) x dO/Q (MN-major) -> [keys, d]

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + KTILE;
  uint8_t* sQD = sV + KTILE;               // 2 stages x (Q, dO)
  uint8_t* sPT = sQD + 4 * QTILE;
  uint8_t* sDST = sPT + PT_BYTES;
  __shared__ uint64_t kv_full, qd_full[2], qd_empty[2], st_full[2], st_empty[2], stat_full[2], pt_full, pt_empty, acc_full;
  __shared__ __align__(16) float s_lse2[2][BQ], s_delta[2][BQ];
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * BKV, kvh = blockIdx.y, b = blockIdx.z;
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
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&qd_full[s]), 1);
      mbar_init(smem_u32(&qd_empty[s]), 1);
      mbar_init(smem_u32(&st_full[s]), 1);
      mbar_init(smem_u32(&st_empty[s]), 256);
      mbar_init(smem_u32(&stat_full[s]), 256);
    }
    mbar_init(smem_u32(&pt_full), 256);
    mbar_init(smem_u32(&pt_empty), 1);
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

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(smem_u32(&kv_full), 2 * KTILE);
      for (int h = 0; h < D / 64; ++h) {
        tma_load_4d(smem_u32(sK + h * KHALF), &tk, smem_u32(&kv_full), h * 64, k0, kvh, b);
        tma_load_4d(smem_u32(sV + h * KHALF), &tv, smem_u32(&kv_full), h * 64, k0, kvh, b);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int head = kvh * rep + it / tiles_per_head;
        const int qi0 = (it_begin + it % tiles_per_head) * BQ;
        if (!mbar_wait(smem_u32(&qd_empty[s]), ph ^ 1, abortp)) {
          atomicExch(p.status, STATUS_TIMEOUT_EMPTY);
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
      auto issue_st = [&](int it) -> bool {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(smem_u32(&qd_full[s]), ph, abortp)) return false;
        if (!mbar_wait(smem_u32(&st_empty[s]), ph ^ 1, abortp)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
        const uint32_t qa = smem_u32(sQD + (2 * s) * QTILE), doa = smem_u32(sQD + (2 * s + 1) * QTILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t offk = (k / 4) * KHALF + (k % 4) * 32, offq = (k / 4) * QHALF + (k % 4) * 32;
          tc_mma_ss(tmem + ST_COL + s * BQ, make_smem_desc(ka + offk, 16, 1024), make_smem_desc(qa + offq, 16, 1024), IDESC_ST, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t offk = (k / 4) * KHALF + (k % 4) * 32, offq = (k / 4) * QHALF + (k % 4) * 32;
          tc_mma_ss(tmem + DPT_COL + s * BQ, make_smem_desc(va + offk, 16, 1024), make_smem_desc(doa + offq, 16, 1024), IDESC_ST, k > 0);
        }
        tc_commit(smem_u32(&st_full[s]));
        return true;
      };
      bool ok = mbar_wait(smem_u32(&kv_full), 0, abortp);
      if (ok) ok = issue_st(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it + 1 < n_iter) ok = issue_st(it + 1);
        if (!ok) break;
        const int s = it & 1;
        if (!mbar_wait(smem_u32(&pt_full), it & 1, abortp)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pta = smem_u32(sPT), dsta = smem_u32(sDST);
        const uint32_t qa = smem_u32(sQD + (2 * s) * QTILE), doa = smem_u32(sQD + (2 * s + 1) * QTILE);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {  // dV += P^T dO
          tc_mma_ss(tmem + DV_COL, make_smem_desc(pta + k * 32, 16, 1024), make_smem_desc(doa + k * 2048, QHALF, 1024), IDESC_ACC,
                    (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {  // dK += dS^T Q
          tc_mma_ss(tmem + DK_COL, make_smem_desc(dsta + k * 32, 16, 1024), make_smem_desc(qa + k * 2048, QHALF, 1024), IDESC_ACC,
                    (it > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&qd_empty[s]));
        tc_commit(smem_u32(&pt_empty));
        if (it == n_iter - 1) tc_commit(smem_u32(&acc_full));
      }
      if (!ok) {
        atomicExch(p.status, STATUS_TIMEOUT_FULL);
        abort_flag = 1;
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // key row
    const int tid = threadIdx.x - 64;                     // 0..255 among the elementwise threads
    const int wg = tid >> 7;                              // group 0 takes query columns 0..31 of a tile, group 1 columns 32..63
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const int kk = k0 + row;
    const bool key_valid = kk < p.S;
    bool failed = false;
    // per-query statistics (log-sum-exp, delta) of tile `it`, one value per thread of the first group; they are fetched one
    // iteration ahead so that the global-load latency is off the per-iteration critical path
    auto load_stat = [&](int it) -> float {
      const int head = kvh * rep + it / tiles_per_head;
      const int qi = (it_begin + it % tiles_per_head) * BQ + (tid & 63);
      const long long idx = ((long long)b * p.Nq + head) * p.T + qi;
      if (tid < 64) return qi < p.T ? p.lse[idx] * B_LOG2E : INFINITY;
      if (tid < 128) return qi < p.T ? p.delta[idx] : 0.f;
      return 0.f;
    };
    auto publish_stat = [&](int buf, float v) {
      if (tid < 64) s_lse2[buf][tid] = v;
      else if (tid < 128) s_delta[buf][tid - 64] = v;
      mbar_arrive(smem_u32(&stat_full[buf]));
    };
    if (n_iter > 0) publish_stat(0, load_stat(0));
    for (int it = 0; it < n_iter; ++it) {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int qi0 = (it_begin + it % tiles_per_head) * BQ;
      const float next_stat = it + 1 < n_iter ? load_stat(it + 1) : 0.f;
      if (!mbar_wait(smem_u32(&stat_full[s]), ph, abortp)) { failed = true; break; }
      if (!mbar_wait(smem_u32(&st_full[s]), ph, abortp)) { failed = true; break; }
      tc_fence_after();
      {
        const int c = wg;                                 // BQ / 32 = 2 column chunks, one per group
        uint32_t rs[32], rp[32];
        tmem_ld32(tmem + lane_addr + ST_COL + s * BQ + c * 32, rs);
        tmem_ld32(tmem + lane_addr + DPT_COL + s * BQ + c * 32, rp);
        tmem_ld_wait();
        float pr[32], ds[32];
        float lse_c[32], del_c[32];                         // this chunk's statistics, fetched 16 bytes at a time
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 a = reinterpret_cast<const float4*>(&s_lse2[s][c * 32])[i];
          const float4 d = reinterpret_cast<const float4*>(&s_delta[s][c * 32])[i];
          lse_c[4 * i] = a.x; lse_c[4 * i + 1] = a.y; lse_c[4 * i + 2] = a.z; lse_c[4 * i + 3] = a.w;
          del_c[4 * i] = d.x; del_c[4 * i + 1] = d.y; del_c[4 * i + 2] = d.z; del_c[4 * i + 3] = d.w;
        }
        const int qfirst = p.q_start + qi0 + c * 32;
        if (key_valid && kk <= qfirst && (p.window == 0 || kk > qfirst + 31 - p.window)) {   // whole chunk visible
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            pr[i] = exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse_c[i]));
            ds[i] = pr[i] * (__uint_as_float(rp[i]) - del_c[i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int qpos = qfirst + i;
            const bool vis = key_valid && kk <= qpos && (p.window == 0 || kk > qpos - p.window);
            pr[i] = vis ? exp2f(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse_c[i])) : 0.f;
            ds[i] = pr[i] * (__uint_as_float(rp[i]) - del_c[i]);
          }
        }
        // the previous tile's dV / dK products must have consumed P^T and dS^T before they are overwritten
        if (it > 0 && !mbar_wait(smem_u32(&pt_empty), (it - 1) & 1, abortp)) failed = true;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c16 = c * 4 + q;
          uint4 o;
          o.x = pack_bf16(pr[q * 8 + 0], pr[q * 8 + 1]);
          o.y = pack_bf16(pr[q * 8 + 2], pr[q * 8 + 3]);
          o.z = pack_bf16(pr[q * 8 + 4], pr[q * 8 + 5]);
          o.w = pack_bf16(pr[q * 8 + 6], pr[q * 8 + 7]);
          *reinterpret_cast<uint4*>(sPT + swz128(row, c16)) = o;
          o.x = pack_bf16(ds[q * 8 + 0], ds[q * 8 + 1]);
          o.y = pack_bf16(ds[q * 8 + 2], ds[q * 8 + 3]);
          o.z = pack_bf16(ds[q * 8 + 4], ds[q * 8 + 5]);
          o.w = pack_bf16(ds[q * 8 + 6], ds[q * 8 + 7]);
          *reinterpret_cast<uint4*>(sDST + swz128(row, c16)) = o;
        }
      }
      if (failed) break;
      tc_fence_before();
      mbar_arrive(smem_u32(&st_empty[s]));
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&pt_full));
      // everyone who passed this iteration's stat_full wait has finished iteration it - 1, the last reader of the other buffer
      if (it + 1 < n_iter) publish_stat(s ^ 1, next_stat);
    }
    if (!failed && n_iter > 0 && !mbar_wait(smem_u32(&acc_full), 0, abortp)) failed = true;
    if (failed) {
      if (lane == 0) atomicExch(p.status, STATUS_TIMEOUT_TMEM);
      abort_flag = 1;
    } else {
      tc_fence_after();
      const long long o_off = (((long long)b * p.S + kk) * p.Nkv + kvh) * D;
      {
        const int which = wg;                             // group 0 writes dK, group 1 writes dV
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
  CUtensorMap tq, tk, tv, tdo, tq64, tdo64;
  if (bwd_map(&tq, q, p.B, p.T, p.Nq, D, qs[0], qs[1], qs[2], 128)) return -31;
  if (bwd_map(&tk, k, p.B, p.S, p.Nkv, D, ks[0], ks[1], ks[2], 128)) return -32;
  if (bwd_map(&tv, v, p.B, p.S, p.Nkv, D, vs[0], vs[1], vs[2], 128)) return -33;
  if (bwd_map(&tdo, d_o, p.B, p.T, p.Nq, D, dos[0], dos[1], dos[2], 128)) return -34;
  if (bwd_map(&tq64, q, p.B, p.T, p.Nq, D, qs[0], qs[1], qs[2], 64)) return -35;
  if (bwd_map(&tdo64, d_o, p.B, p.T, p.Nq, D, dos[0], dos[1], dos[2], 64)) return -36;
  constexpr int smem_dq = 7 * 128 * D * 2 + 1024 + (D == 64 ? 128 * 128 * 2 - 128 * 64 * 2 : 0);  // Q, dO, 2x(K,V), dS(32 KB)
  constexpr int smem_dkv = 2 * 128 * D * 2 + 4 * 64 * D * 2 + 2 * 128 * 64 * 2 + 1024;
  static bool once = false;
  if (!once) {
    if (cudaFuncSetAttribute(flash_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq) != cudaSuccess) return -37;
    if (cudaFuncSetAttribute(flash_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkv) != cudaSuccess) return -38;
    once = true;
  }
  flash_bwd_dq_kernel<D><<<dim3((p.T + 127) / 128, p.Nq, p.B), FB_THREADS, smem_dq, s>>>(tq, tk, tv, tdo, p);
  flash_bwd_dkv_kernel<D><<<dim3((p.S + 127) / 128, p.Nkv, p.B), DKV_THREADS, smem_dkv, s>>>(tq64, tk, tv, tdo64, p);
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
