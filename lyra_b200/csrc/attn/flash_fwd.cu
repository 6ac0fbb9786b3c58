// Flash attention forward for sm_100a: causal / sliding-window GQA attention with a learned sink per
// query head (semantics of the reference's FLASH_ATTENTION kernels, lyra/kernels/flash_attention.py:208-374):
//   out = softmax([q k^T * scale | sink_h]) restricted to the key columns, LSE in natural-log units.
// The running max starts at the sink logit and the normaliser at 1, so the sink is an extra softmax column
// without a value. Only key tiles that intersect the causal / window band are visited.
//
// A work item is a (128-query tile, query head, batch); one persistent CTA per SM walks its share of the items.
// Tensors are token-major [B, T, N, D] (the layout the projection GEMMs produce), addressed by 4-D TMA maps,
// so no transposes are needed around the kernel.
//
// The key tiles of a query tile are dealt alternately to two softmax groups that never talk to each other
// until the end: each group has its own score buffer, its own running (max, sum) per row and its own output
// accumulator in TMEM (2 x 128 score columns + 2 x D output columns), as if the keys were split in two
// interleaved sequences; the two partial results are merged once, in the epilogue. While one group
// exponentiates tile j, the tensor core runs the other group's P V and Q K^T, so the two pipes overlap
// without any per-tile exchange between the groups.
//   warp 0      : TMA producer (Q once; K and V tiles double-buffered)
//   warp 1      : tcgen05 issuer:  S_g = Q K_j^T  and  O_g += P_g V_j   (g = j mod 2)
//   warps 2..5  : softmax group 0, warps 6..9 : softmax group 1 - one query row per thread: the row's 128 scores
//                 come out of TMEM once, exp2-domain online softmax with lazy rescaling of O_g, and P goes back
//                 as packed bf16 into the first 64 columns of the same score buffer, from where the second MMA
//                 takes it as its TMEM operand (no shared-memory staging of P)
#include "../common/sm100.cuh"
#include "../common/tmap.h"

namespace lyra {

constexpr int FA_THREADS = 320;   // TMA warp, MMA warp, two groups of four softmax warps (alternate key tiles)
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

// One work item: a 128-query tile of one (batch, head) and the key tiles inside its band.
struct FwdItem {
  int q0, head, b, kvh, jt_begin, n_tiles, qlo;
};

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const FwdParams p) {
  constexpr int BQ = 128, BKV = 128;
  constexpr int TILE = BQ * D * 2;         // bytes of a 128 x D bf16 tile
  constexpr int HALF = BQ * 128;           // bytes of one 64-column swizzle atom column block (128 rows x 128 B)
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, O_COL = 256, GROUP_COLS = 128;    // group g: scores at S_COL + 128 g, output at O_COL + 128 g
  constexpr uint32_t IDESC_S = make_idesc(BQ, BKV, 1, 1, 0, 0);   // Q K-major, K K-major
  constexpr uint32_t IDESC_O = make_idesc(BQ, D, 1, 1, 0, 1);     // P K-major (TMEM), V MN-major

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;           // 2 stages
  uint8_t* sV = sK + 2 * TILE;       // 2 stages
  __shared__ uint64_t q_full, q_empty, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_full, o_empty, l_full;
  __shared__ float xm[2][2][BQ], xl[2][2][BQ];      // [item parity][group][row]: the groups' row maxima and sums, merged in the epilogue
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Persistent: one CTA per SM walks the work items, so TMEM allocation, barrier set-up and the first loads are paid once and
  // the output pass of one item overlaps the first products of the next. Items are ordered by falling key-tile count (late
  // query tiles first) and dealt to the CTAs in a serpentine, which evens out the sums without a shared counter.
  const int n_qt = (p.T + BQ - 1) / BQ;
  const int per_qt = p.Nq * p.B;
  const int n_items = n_qt * per_qt;
  auto item_at = [&](int round, FwdItem& it) -> bool {
    const int idx = round * int(gridDim.x) + ((round & 1) ? int(gridDim.x) - 1 - int(blockIdx.x) : int(blockIdx.x));
    if (idx >= n_items) return false;
    const int rest = idx % per_qt;
    it.q0 = (n_qt - 1 - idx / per_qt) * BQ;
    it.head = rest % p.Nq;
    it.b = rest / p.Nq;
    it.kvh = it.head / (p.Nq / p.Nkv);
    it.qlo = p.q_start + it.q0;
    const int qhi = min(p.q_start + min(it.q0 + BQ, p.T) - 1, p.S - 1);
    const int klo = p.window > 0 ? max(0, it.qlo - p.window + 1) : 0;
    it.jt_begin = klo / BKV;
    const int jt_end = qhi < 0 ? it.jt_begin : qhi / BKV + 1;
    it.n_tiles = max(jt_end - it.jt_begin, 0);
    return true;
  };

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&q_full), 1);
    mbar_init(smem_u32(&q_empty), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&p_full[s]), 128);
    }
    mbar_init(smem_u32(&l_full), 256);
    mbar_init(smem_u32(&o_full), 1);
    mbar_init(smem_u32(&o_empty), 256);
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
  FwdItem w;

  // Counters that run across the items of this CTA (every role keeps its own copies and advances them the same way):
  //   t    key tiles so far: stage t & 1 of the K and V rings, parity (t >> 1) & 1
  //   n    items with at least one key tile so far: parity of q_full / q_empty / o_full / o_empty / l_full
  //   c_g  tiles given to softmax group g so far: parity of s_full[g] / p_full[g]
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tq);
      tma_prefetch_desc(&tk);
      tma_prefetch_desc(&tv);
      uint32_t t = 0, n = 0;
      bool ok = true;
      for (int round = 0; ok && item_at(round, w); ++round) {
        if (w.n_tiles == 0) continue;
        if (!mbar_wait(smem_u32(&q_empty), (n & 1) ^ 1, abortp)) { ok = false; break; }   // the last Q K^T of the previous item retired
        mbar_expect_tx(smem_u32(&q_full), TILE);
        for (int h = 0; h < D / 64; ++h) tma_load_4d(smem_u32(sQ + h * HALF), &tq, smem_u32(&q_full), h * 64, w.q0, w.head, w.b);
        ++n;
        for (int j = 0; j < w.n_tiles; ++j, ++t) {
          const int s = t & 1;
          const uint32_t ph = (t >> 1) & 1;
          const int k0 = (w.jt_begin + j) * BKV;
          if (!mbar_wait(smem_u32(&k_empty[s]), ph ^ 1, abortp)) { ok = false; break; }
          mbar_expect_tx(smem_u32(&k_full[s]), TILE);
          for (int h = 0; h < D / 64; ++h) tma_load_4d(smem_u32(sK + s * TILE + h * HALF), &tk, smem_u32(&k_full[s]), h * 64, k0, w.kvh, w.b);
          if (!mbar_wait(smem_u32(&v_empty[s]), ph ^ 1, abortp)) { ok = false; break; }
          mbar_expect_tx(smem_u32(&v_full[s]), TILE);
          for (int h = 0; h < D / 64; ++h) tma_load_4d(smem_u32(sV + s * TILE + h * HALF), &tv, smem_u32(&v_full[s]), h * 64, k0, w.kvh, w.b);
        }
      }
      if (!ok) {
        atomicCAS(p.status, 0, STATUS_TIMEOUT_EMPTY);
        abort_flag = 1;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // Tile j of an item belongs to group g = j & 1. MMAs of one thread retire in issue order, so S_g(j + 2) (issued after
      // P_g(j) V_j) can never overwrite P_g(j) before it was read, and s_full[g] of tile j + 2 tells the group that O_g is quiet
      // (P_g(j) V_j retired) until the group itself releases the next P.
      uint32_t t = 0, n = 0, c[2] = {0, 0};
      bool ok = true;
      const uint64_t dq0 = make_smem_desc(smem_u32(sQ), 16, 1024), dk0 = make_smem_desc(smem_u32(sK), 16, 1024);
      const uint64_t dv0 = make_smem_desc(smem_u32(sV), HALF, 1024);         // V as the MN-major operand of O += P V
      for (int round = 0; ok && item_at(round, w); ++round) {
        if (w.n_tiles == 0) continue;
        const uint32_t t0 = t;
        auto issue_s = [&](int j) -> bool {
          const int g = j & 1, s = (t0 + j) & 1;
          if (!mbar_wait(smem_u32(&k_full[s]), ((t0 + j) >> 1) & 1, abortp)) return false;
          tc_fence_after();
          const uint64_t dk = desc_advance(dk0, s * TILE);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            tc_mma_ss(tmem + S_COL + g * GROUP_COLS, desc_advance(dq0, (k / 4) * HALF + (k % 4) * 32), desc_advance(dk, (k / 4) * HALF + (k % 4) * 32), IDESC_S, k > 0);
          tc_commit(smem_u32(&s_full[g]));
          tc_commit(smem_u32(&k_empty[s]));
          if (j == w.n_tiles - 1) tc_commit(smem_u32(&q_empty));
          return true;
        };
        ok = mbar_wait(smem_u32(&q_full), n & 1, abortp);
        if (ok) ok = issue_s(0);
        if (ok && w.n_tiles > 1) ok = issue_s(1);
        // the previous item's output must have been read before the first P V of this one overwrites the accumulators
        if (ok) ok = mbar_wait(smem_u32(&o_empty), (n & 1) ^ 1, abortp);
        for (int j = 0; j < w.n_tiles && ok; ++j) {
          const int g = j & 1, s = (t0 + j) & 1;
          if (!mbar_wait(smem_u32(&v_full[s]), ((t0 + j) >> 1) & 1, abortp)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&p_full[g]), c[g] & 1, abortp)) { ok = false; break; }
          ++c[g];
          tc_fence_after();
          const uint64_t dv = desc_advance(dv0, s * TILE);
#pragma unroll
          for (int k = 0; k < BKV / 16; ++k)      // 16 keys of P = 8 TMEM columns of packed bf16 pairs
            tc_mma_ts(tmem + O_COL + g * GROUP_COLS, tmem + S_COL + g * GROUP_COLS + k * 8, desc_advance(dv, k * 2048), IDESC_O, (j >= 2 || k > 0) ? 1u : 0u);
          tc_commit(smem_u32(&v_empty[s]));
          if (j + 2 < w.n_tiles) ok = issue_s(j + 2);
        }
        if (ok) tc_commit(smem_u32(&o_full));
        t += w.n_tiles;
        ++n;
      }
      if (!ok) {
        atomicCAS(p.status, 0, STATUS_TIMEOUT_FULL);
        abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // row of the query tile == TMEM lane
    const uint32_t lane_addr = uint32_t(quarter * 32) << 16;
    const int g = (warp - 2) >> 2;                        // group 0: key tiles 0, 2, 4, ... of an item; group 1: 1, 3, 5, ...
    const uint32_t s_addr = tmem + lane_addr + S_COL + g * GROUP_COLS;
    const uint32_t o_addr = tmem + lane_addr + O_COL + g * GROUP_COLS;
    const float sc = p.scale_log2;
    uint32_t n = 0, cg = 0;
    bool failed = false;

    for (int round = 0; !failed && item_at(round, w); ++round) {
      const int qpos = p.q_start + w.q0 + row;              // absolute position of this query
      const bool row_valid = (w.q0 + row) < p.T;
      const float sink2 = p.sinks[w.head] * LOG2E;
      float m = sink2, l = g == 0 ? 1.0f : 0.0f;            // the sink's unit weight is counted once, by group 0
      const int hi = min(qpos, p.S - 1);                    // last visible key
      const int lo = p.window > 0 ? qpos - p.window + 1 : 0;   // first visible key

      for (int j = g; j < w.n_tiles; j += 2, ++cg) {
        const int k0 = (w.jt_begin + j) * BKV;
        if (!mbar_wait(smem_u32(&s_full[g]), cg & 1, abortp)) { failed = true; break; }
        tc_fence_after();
        const bool need_mask = (k0 + BKV - 1 > w.qlo) || (p.window > 0 && k0 < w.qlo + BQ - p.window + 1) || (k0 + BKV > p.S);
        auto mask = [&](uint32_t (&r)[32], int c) {
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int kk = k0 + c * 32 + i;
              if (kk > hi || kk < lo) r[i] = 0xff800000u;        // -inf: never the maximum, weight 0
            }
          }
        };
        // One pass in the common case: the probabilities are formed against the current reference maximum while the tile's own
        // maximum is tracked, and stay in registers (packed) until it is known that no row of the warp has to move its
        // reference (lazy rescale: only when the new maximum exceeds the reference by more than 2^8). Otherwise the warp reads
        // the scores again - they are still in TMEM - and redoes the tile with the new references; rows that keep theirs get the
        // same values again.
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[2][32];
        auto quarter_pass = [&](int c, bool track) {
          uint32_t r[32];
          tmem_ld32(s_addr + c * 32, r);
          tmem_ld_wait();
          mask(r, c);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            if (track) mx4[c] = fmaxf(mx4[c], fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
            const float p0 = exp2f(fmaf(__uint_as_float(r[i]), sc, -m));
            const float p1 = exp2f(fmaf(__uint_as_float(r[i + 1]), sc, -m));
            sum4[c] += p0 + p1;
            pk[c >> 1][(c & 1) * 16 + (i >> 1)] = pack_bf16(p0, p1);
          }
        };
#pragma unroll
        for (int c = 0; c < 4; ++c) quarter_pass(c, true);
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc;    // the scale is positive
        if (__any_sync(0xffffffffu, mx > m + 8.0f)) {
          float factor = 1.0f;
          if (mx > m + 8.0f) {
            factor = exp2f(m - mx);
            m = mx;
          }
          l *= factor;
          if (j >= 2) {                                       // O_g holds tiles j-2, j-4, ...: all retired (see the issuer)
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(o_addr + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
              tmem_st32(o_addr + c * 32, o);
            }
          }
          sum4[0] = sum4[1] = sum4[2] = sum4[3] = 0.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) quarter_pass(c, false);
        }
        // bf16 pairs back into columns 0..63 of the same buffer (column c holds keys 2c and 2c+1)
        tmem_st32(s_addr, pk[0]);
        tmem_st32(s_addr + 32, pk[1]);
        tmem_st_wait();
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        tc_fence_before();
        mbar_arrive(smem_u32(&p_full[g]));
      }
      if (failed) break;

      // epilogue of the item: merge the two groups, O / l -> bf16, LSE
      __nv_bfloat16* orow = p.out + (((long long)w.b * p.T + (w.q0 + row)) * p.Nq + w.head) * D;
      if (w.n_tiles == 0) {                                   // no visible key at all: the sink takes all the weight
        if (row_valid) {
          for (int c = g * (D / 2); c < (g + 1) * (D / 2); c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0u, 0u, 0u, 0u);
          if (g == 0) p.lse[((long long)w.b * p.Nq + w.head) * p.T + w.q0 + row] = sink2 * LN2;
        }
        continue;
      }
      const int par = n & 1;
      xm[par][g][row] = m;
      xl[par][g][row] = l;
      mbar_arrive(smem_u32(&l_full));
      if (!mbar_wait(smem_u32(&o_full), par, abortp)) { failed = true; break; }
      if (!mbar_wait(smem_u32(&l_full), par, abortp)) { failed = true; break; }
      tc_fence_after();
      const bool two = w.n_tiles > 1;                         // group 1 saw at least one tile
      const float m0 = xm[par][0][row], m1 = xm[par][1][row];
      const float mt = two ? fmaxf(m0, m1) : m0;
      const float a0 = exp2f(m0 - mt), a1 = two ? exp2f(m1 - mt) : 0.0f;
      const float lt = a0 * xl[par][0][row] + a1 * xl[par][1][row];
      const float w0 = a0 / lt, w1 = a1 / lt;
#pragma unroll 1
      for (int c = g; c < D / 32; c += 2) {                   // each group writes half of the columns
        uint32_t r0[32], r1[32];
        tmem_ld32(tmem + lane_addr + O_COL + c * 32, r0);
        if (two) tmem_ld32(tmem + lane_addr + O_COL + GROUP_COLS + c * 32, r1);
        tmem_ld_wait();
        float o[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          o[i] = __uint_as_float(r0[i]) * w0;
          if (two) o[i] = fmaf(__uint_as_float(r1[i]), w1, o[i]);
        }
        if (row_valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16(o[q * 8 + 0], o[q * 8 + 1]);
            v.y = pack_bf16(o[q * 8 + 2], o[q * 8 + 3]);
            v.z = pack_bf16(o[q * 8 + 4], o[q * 8 + 5]);
            v.w = pack_bf16(o[q * 8 + 6], o[q * 8 + 7]);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = v;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&o_empty));                        // the accumulators may be overwritten by the next item
      if (row_valid && g == 0) p.lse[((long long)w.b * p.Nq + w.head) * p.T + w.q0 + row] = (mt + log2f(lt)) * LN2;
      ++n;
    }
    if (failed) {
      if (lane == 0) atomicCAS(p.status, 0, STATUS_TIMEOUT_TMEM);
      abort_flag = 1;
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
  const long long n_items = (long long)((T + 127) / 128) * Nq * B;
  const int sms = lyra::sm_count();
  dim3 grid(n_items < sms ? (unsigned)n_items : (unsigned)sms);          // persistent: one CTA per SM
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) {
    constexpr int smem = 5 * 128 * 128 * 2 + 1024;  // Q + 2K + 2V
    static bool once = false;
    if (!once) { if (cudaFuncSetAttribute(flash_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -24; once = true; }
    flash_fwd_kernel<128><<<grid, FA_THREADS, smem, s>>>(tq, tk, tv, p);
  } else {
    constexpr int smem = 5 * 128 * 64 * 2 + 1024;
    static bool once = false;
    if (!once) { if (cudaFuncSetAttribute(flash_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -24; once = true; }
    flash_fwd_kernel<64><<<grid, FA_THREADS, smem, s>>>(tq, tk, tv, p);
  }
  LYRA_CHECK_LAUNCH();
  return 0;
}
