// Persistent warp-specialised bf16 GEMM for sm_100a: TMA (local memory) -> 128B-swizzled shared
// memory -> tcgen05.mma with fp32 accumulators in TMEM -> tcgen05.ld epilogue.
//
//   D[M,N] = alpha * A[M,K] x B[N,K]^T + beta * Cin        (dense)
//   grouped-M : rows of A/D are sorted by group, each 128-row tile belongs to one group and uses
//               that group's B (ragged grouped GEMM of a mixture-of-experts layer; the reference's
//               `GEMM` / `GEMM_DLHS`, lyra/kernels/gemm.py:512-1120)
//   grouped-K : per group g, D[g] = A[:, rows_g]^T-style contraction over the group's rows
//               (expert weight gradients; the reference's `TGEMM`, lyra/kernels/gemm.py:1175-1445)
//   batched   : independent problems of the same shape (Newton-Schulz over stacked expert matrices)
//
// Either operand may be K-major (contraction dim contiguous) or MN-major (its own dim contiguous), so
// forward, data-gradient and weight-gradient products of an [in,out]-layout weight run without transposes.
// Epilogues: plain store (bf16 or fp32, optional bias, optional alpha/beta with a second input), and the
// fused clamped SwiGLU of the reference (lyra/kernels/common.py:98-114) where each 256-wide accumulator
// tile holds 128 gate columns and their 128 linear columns.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 = epilogue.
// Two 256-column accumulators (all 512 TMEM columns) let the epilogue of tile i overlap tile i+1.
#include "../common/sm100.cuh"
#include "../common/tmap.h"

namespace lyra {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int MIRROR_LD = 136;           // row length (elements) of the 32 x 128 staging tile used to mirror symmetric results
constexpr int MIRROR_BYTES = 32 * MIRROR_LD * 2;
constexpr int SCATTER_LD = 72;           // row length (elements) of the 128 x 64 staging tile of the scattered (peer) store
constexpr int EPI_STAGE_BYTES = 128 * SCATTER_LD * 2 + 128 * 4 + 512;   // staging tile + one destination per row (>= MIRROR_BYTES)
constexpr int GEMM_THREADS_AG = 320;   // + four warps that pull the B operand from peer GPUs (all-gather fused GEMM)
constexpr int AG_MAX_RANKS = 16;

enum GroupMode : int { GROUP_NONE = 0, GROUP_M = 1, GROUP_K = 2, GROUP_BATCH = 3 };
enum Epilogue : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_CE_FWD = 2, EPI_CE_DZ = 3 };

struct GemmParams {
  int M, N, K;              // per-problem extents (N = accumulator columns; SwiGLU output has N/2)
  int m_tiles, n_tiles, total_tiles;
  void* C;                  // output
  const void* Cin;          // optional second input of the epilogue (same dtype / ld as C)
  long long ldc;
  long long c_group_stride; // elements between per-group outputs (grouped-K / batched)
  int out_fp32;
  float alpha, beta;
  const float* bias;        // [groups, N] or [N] or null
  long long bias_group_stride;
  int group_mode;
  const int* tile_group;    // grouped-M: group of each 128-row tile, -1 = unused tile
  const int* group_offsets; // grouped-K: [G+1] row offsets, multiples of 64
  int num_groups;
  int n_split;              // SwiGLU: column where the linear half starts in B (= hidden size)
  float swiglu_beta, swiglu_limit;
  // scattered output (expert-parallel return fused into the GEMM): row r of the result is stored to row (row_dest[r] & 0xFFFFFF)
  // of the buffer peer_out[row_dest[r] >> 24] (another GPU's memory, plain 16-byte stores); rows with row_dest < 0 are dropped
  const int* row_dest;
  void* peer_out[AG_MAX_RANKS];
  const float* row_scale;   // scattered output: optional per-row factor (the routing score of the row's assignment) applied after the bias
  int* peer_count[AG_MAX_RANKS];  // scattered output: per destination rank, a counter in that rank's memory to which every tile adds the
                            // number of rows it has stored there (release, system scope); null = no counting
  // tile-granular dispatch (grouped-M): the rows of A are stored into this GPU's memory by other GPUs while the kernel runs
  const int* tile_perm;     // logical -> physical 128-row tile, -1 = no more tiles; null = identity
  const int* arrive;        // per physical tile: rows that have landed so far (running total, bumped by the senders)
  const int* expect;        // per physical tile: running total that means "this tile is complete"
  int sym_tiles;            // tiles per matrix that are enumerated when sym_upper is set
  int sym_upper;            // 1: the result is symmetric (A A^T): tiles wholly below the diagonal are not enumerated; bf16 outputs are mirrored by
                            //    the epilogue of the upper tiles, fp32 outputs by `lyra_symmetrize`
  int raster_group;         // > 0: grouped raster with bands of this many M-tiles (takes precedence over raster_n_major)
  int raster_n_major;       // 1: consecutive tiles walk M first (the B operand is streamed once; used by the vocabulary GEMMs)
  // fused linear cross-entropy epilogues (B = the [V, C] head, N = real vocabulary size)
  const int* ce_y;          // [M] target ids
  float* ce_part_m;         // [n_tiles, M] per-tile row maxima          (EPI_CE_FWD)
  float* ce_part_l;         // [n_tiles, M] per-tile sum exp(z - max)    (EPI_CE_FWD)
  float* ce_tgt;            // [M] target logit                          (EPI_CE_FWD)
  const float* ce_lse;      // [M] log-sum-exp                           (EPI_CE_DZ)
  const float* ce_gscale;   // device scalar multiplying dZ              (EPI_CE_DZ)
  // all-gather fused mode (ag_world > 0): B's K-rows live in peer GPUs' memory; four extra warps per CTA copy them,
  // one 256-column panel after the other, into the local B buffer (the one the TMA map points at) and count the
  // finished pieces per panel; the TMA producer waits for a tile's panel before loading it. TMA only ever reads
  // local memory.
  int ag_world;                      // 0 = off
  int ag_rows_per_rank;              // K-rows held by each rank (K for a single owner, K / world for row shards)
  int ag_my_rank;
  long long ag_row_bytes;            // bytes per K-row (ldb * 2)
  const void* ag_src[AG_MAX_RANKS];  // per-rank base of its rows (row index local to the rank)
  void* ag_dst;                      // local B buffer base
  int* ag_flags;                     // [ceil(N / 256)] local counters, one per column panel of B
  int ag_epoch;                      // number of this call on these counters (1, 2, ...)
  int* status;
};

struct TileInfo {
  int m0, n0, ga, gb, gc, krow0, num_kb;
  bool valid;
};

template <int BN, int EPI>
__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int tile) {
  TileInfo t;
  constexpr int NSTEP = (EPI == EPI_SWIGLU) ? BN / 2 : BN;
  t.valid = true;
  t.ga = t.gb = t.gc = 0;
  t.krow0 = 0;
  t.num_kb = (p.K + BK - 1) / BK;
  int local = tile;
  if (p.group_mode == GROUP_K || p.group_mode == GROUP_BATCH) {
    const int per = p.sym_upper ? p.sym_tiles : p.m_tiles * p.n_tiles;
    const int g = tile / per;
    local = tile - g * per;
    t.gc = g;
    if (p.group_mode == GROUP_K) {
      const int b = p.group_offsets[g], e = p.group_offsets[g + 1];
      t.krow0 = b;
      t.num_kb = (e - b + BK - 1) / BK;
    } else {
      t.ga = t.gb = g;
    }
  }
  int m_blk, n_blk;
  if (p.sym_upper) {
    // symmetric result: only tiles that reach the diagonal or lie above it are enumerated (row m starts at column tile
    // m * BM / NSTEP), so the persistent CTAs share the real work evenly instead of drawing skipped tiles
    int m = 0, acc = 0;
    for (;;) {
      const int cnt = p.n_tiles - min(p.n_tiles, m * BM / NSTEP);
      if (local < acc + cnt || m + 1 >= p.m_tiles) break;
      acc += cnt;
      ++m;
    }
    m_blk = m;
    n_blk = m * BM / NSTEP + (local - acc);
  } else if (p.raster_group > 0) {
    // grouped raster: tiles walk N inside a band of `raster_group` M-tiles, so a wave of CTAs shares a small set of A row
    // panels and a run of B column panels (both stay in L2) instead of one operand in full
    const int band = p.raster_group * p.n_tiles;
    const int grp = local / band, within = local - grp * band;
    const int gm = min(p.raster_group, p.m_tiles - grp * p.raster_group);
    n_blk = within / gm;
    m_blk = grp * p.raster_group + (within - n_blk * gm);
  } else if (p.raster_n_major) {
    n_blk = local / p.m_tiles;
    m_blk = local - n_blk * p.m_tiles;
  } else {
    m_blk = local / p.n_tiles;
    n_blk = local - m_blk * p.n_tiles;
  }
  if (p.group_mode == GROUP_M) {
    if (p.tile_perm) m_blk = p.tile_perm[m_blk];
    const int g = m_blk >= 0 ? p.tile_group[m_blk] : -1;
    t.valid = g >= 0;
    t.gb = g < 0 ? 0 : g;
    if (m_blk < 0) m_blk = 0;
  }
  t.m0 = m_blk * BM;
  t.n0 = n_blk * NSTEP;
  return t;
}

__device__ __forceinline__ float swiglu_act(float g, float l, float beta, float limit) {
  g = fminf(g, limit);
  l = fminf(fmaxf(l, -limit), limit);
  return (l + 1.0f) * g * (1.0f / (1.0f + __expf(-beta * g)));
}

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS_AG, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmParams p) {
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int STAGES = (BN == 256) ? 4 : 6;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 512 or 256: a power of two
  constexpr uint32_t IDESC = make_idesc(BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      uint32_t it = 0;
      bool ok = true;
      int ready_tile = -1;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const TileInfo t = decode_tile<BN, EPI>(p, tile);
        if (!t.valid) continue;
        if (p.arrive) {  // rows of this 128-row tile are being stored by other GPUs: wait until all of them have landed
          const int mt = t.m0 / BM;
          if (mt != ready_tile) {
            const int want = p.expect[mt];
            const long long t0 = clock64();
            int v;
            do {
              asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.arrive + mt) : "memory");
              // give up after the time limit - or after 2 ms if an earlier kernel has already reported a failure (rows dropped on
              // overflow never arrive; a healthy exchange delivers a tile within microseconds of its neighbours)
              const long long waited = clock64() - t0;
              if (v - want < 0 && (waited > PEER_WAIT_LIMIT_CYCLES || *abortp || (waited > 4000000 && *reinterpret_cast<volatile int*>(p.status) != 0))) {
                atomicCAS(p.status, 0, STATUS_TIMEOUT_TILE);
                abort_flag = 1;
                ok = false;
                break;
              }
            } while (v - want < 0);
            if (!ok) break;
            asm volatile("fence.proxy.async.global;" ::: "memory");
            ready_tile = mt;
          }
        }
        if (p.ag_world > 0) {  // this tile's 256-column panel of B must have landed in local memory before TMA reads it
          const int* flag = p.ag_flags + t.n0 / BN;
          const int want = p.ag_epoch * ((p.K + BK - 1) / BK);
          const long long t0 = clock64();
          int v;
          do {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v < want && (clock64() - t0 > WAIT_LIMIT_CYCLES || *abortp)) {
              atomicCAS(p.status, 0, STATUS_TIMEOUT_PEER);
              abort_flag = 1;
              ok = false;
              break;
            }
          } while (v < want);
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abortp)) {
            atomicCAS(p.status, 0, STATUS_TIMEOUT_EMPTY);
            abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          mbar_expect_tx(bar, STAGE_BYTES);
          const int k0 = t.krow0 + kb * BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d(sa + j * (BK * 128), &tma_a, bar, t.m0 + j * 64, k0, t.ga);
          } else {
            tma_load_3d(sa, &tma_a, bar, k0, t.m0, t.ga);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
              int col = t.n0 + j * 64;
              if (EPI == EPI_SWIGLU && j >= BN / 128) col = p.n_split + t.n0 + (j - BN / 128) * 64;
              tma_load_3d(sb + j * (BK * 128), &tma_b, bar, col, k0, t.gb);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) {
              int row = t.n0 + j * 128;
              if (EPI == EPI_SWIGLU && j >= 1) row = p.n_split + t.n0;
              tma_load_3d(sb + j * (128 * 128), &tma_b, bar, k0, row, t.gb);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const TileInfo t = decode_tile<BN, EPI>(p, tile);
        if (!t.valid) continue;
        if (t.num_kb == 0) continue;  // empty group: epilogue writes zeros without an accumulator
        const int acc = tile_it & 1;
        const uint32_t aph = (tile_it >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), aph ^ 1, abortp)) {
          atomicCAS(p.status, 0, STATUS_TIMEOUT_TMEM);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < t.num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, abortp)) {
            atomicCAS(p.status, 0, STATUS_TIMEOUT_FULL);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            tc_mma_ss(tmem_d, da, db, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(smem_u32(&empty_bar[s]));  // frees the stage when these MMAs retire
        }
        if (ok) tc_commit(smem_u32(&tfull_bar[acc]));
        ++tile_it;
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ peer copy warps (all-gather fused mode only)
    if (p.ag_world > 0) {
      // Work unit: a piece = 64 K-rows x one 256-column panel (32 KB: one 16-byte load per thread and unrolled step).
      // Pieces are numbered panel by panel and dealt round-robin over the CTAs, so B lands in the order in which the
      // (column-panel-major) tile raster consumes it: the first tiles start after a few MB, the rest of the transfer
      // hides behind the MMAs. Each finished piece bumps its panel's counter; a panel is ready at epoch * slabs.
      const int n_slabs = (p.K + BK - 1) / BK;
      const int row_elems = int(p.ag_row_bytes / 2);
      const int n_panels = (p.N + BN - 1) / BN;
      const int t = threadIdx.x - 6 * 32;  // 0..127
      for (int piece = blockIdx.x; piece < n_slabs * n_panels; piece += gridDim.x) {
        const int panel = piece / n_slabs, slab = piece - panel * n_slabs;
        const int row0 = slab * BK;
        const int owner = row0 / p.ag_rows_per_rank;
        const int rows = min(BK, p.K - row0);
        if (owner != p.ag_my_rank || p.ag_src[owner] != p.ag_dst) {
          const int col0 = panel * BN;
          const int v_per_row = min(BN, row_elems - col0) / 8;      // uint4 per row of this piece
          const uint8_t* sbase = static_cast<const uint8_t*>(p.ag_src[owner]) + (long long)(row0 - owner * p.ag_rows_per_rank) * p.ag_row_bytes + col0 * 2;
          uint8_t* dbase = static_cast<uint8_t*>(p.ag_dst) + (long long)row0 * p.ag_row_bytes + col0 * 2;
          const int total = rows * v_per_row;
          // NVLink round trips are microseconds: 16 loads of 16 bytes in flight per thread (32 KB per CTA) hide them
          for (int i0 = t; i0 < total; i0 += 128 * 16) {
            uint4 v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
              const int i = i0 + u * 128;
              if (i < total) v[u] = *reinterpret_cast<const uint4*>(sbase + (long long)(i / v_per_row) * p.ag_row_bytes + (i % v_per_row) * 16);
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
              const int i = i0 + u * 128;
              if (i < total) *reinterpret_cast<uint4*>(dbase + (long long)(i / v_per_row) * p.ag_row_bytes + (i % v_per_row) * 16) = v[u];
            }
          }
        }
        __threadfence();
        asm volatile("fence.proxy.async.global;" ::: "memory");
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (t == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.ag_flags + panel) : "memory");
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, one TMEM lane quarter each)
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t tile_it = 0;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      const TileInfo t = decode_tile<BN, EPI>(p, tile);
      if (!t.valid) continue;
      const bool have_acc = t.num_kb > 0;
      const int acc = tile_it & 1;
      if (have_acc) {
        const uint32_t aph = (tile_it >> 1) & 1;
        if (!mbar_wait(smem_u32(&tfull_bar[acc]), aph, abortp)) {
          if (lane == 0) atomicCAS(p.status, 0, STATUS_TIMEOUT_TMEM);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
      }
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(quarter * 32) << 16);
      const int row = t.m0 + row_in_tile;
      const bool row_ok = row < p.M;
      const long long c_off = (long long)t.gc * p.c_group_stride + (long long)row * p.ldc;
      const int rdest = (p.row_dest && row < p.M) ? p.row_dest[row] : -1;   // scattered-output mode only
      const float* bias = p.bias ? p.bias + (long long)(p.group_mode == GROUP_M ? t.gb : t.gc) * p.bias_group_stride : nullptr;

      if (EPI == EPI_STORE && p.row_dest) {
        // Scattered store to other GPUs' buffers: 16-byte stores from one row per thread would cross NVLink as 32 separate
        // small writes per instruction, so two 32-column chunks are staged in shared memory and written out as 128 contiguous
        // bytes per row (eight lanes per row, four rows per store instruction).
        __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * STAGE_BYTES);
        int* sdest = reinterpret_cast<int*>(smem + STAGES * STAGE_BYTES + 128 * SCATTER_LD * 2);
        sdest[row_in_tile] = rdest;
        const float rscale = (p.row_scale && rdest >= 0) ? p.row_scale[row] : 1.0f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          if (have_acc) {
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          const int col = t.n0 + c * 32;
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
          if (bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.N) v[i] += bias[col + i];
          }
          if (p.row_scale) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= rscale;
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16(v[q * 8 + 0], v[q * 8 + 1]);
            o.y = pack_bf16(v[q * 8 + 2], v[q * 8 + 3]);
            o.z = pack_bf16(v[q * 8 + 4], v[q * 8 + 5]);
            o.w = pack_bf16(v[q * 8 + 6], v[q * 8 + 7]);
            *reinterpret_cast<uint4*>(stg + row_in_tile * SCATTER_LD + (c & 1) * 32 + q * 8) = o;
          }
          if (c & 1) {
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int col0 = t.n0 + (c - 1) * 32;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int piece = row_in_tile + 128 * k, rr = piece >> 3, part = piece & 7;
              const int d = sdest[rr];
              const int colp = col0 + part * 8;
              if (d >= 0 && colp < p.N)
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.peer_out[d >> 24]) + (long long)(d & 0xFFFFFF) * p.ldc + colp) =
                    *reinterpret_cast<const uint4*>(stg + rr * SCATTER_LD + part * 8);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
        }
        if (p.peer_count[0]) {
          // Every store of this tile has been issued (the loop ends behind a barrier of the four warps). Thread r tells rank r how
          // many rows of this (row tile, column tile) now sit in its buffer: the receiving rank sums these until it has seen
          // rows x column tiles of everything it sent out. The fence + release make the rows visible before the count.
          if (row_in_tile < AG_MAX_RANKS && p.peer_count[row_in_tile]) {
            int n = 0;
            for (int i = 0; i < 128; ++i) {
              const int d = sdest[i];
              n += (d >= 0 && (d >> 24) == row_in_tile) ? 1 : 0;
            }
            if (n > 0) {
              __threadfence_system();
              asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p.peer_count[row_in_tile]), "r"(n) : "memory");
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      } else if (EPI == EPI_STORE) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          if (have_acc) {
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          const int col = t.n0 + c * 32;
          const bool mirror = p.sym_upper && !p.out_fp32 && col < p.N && BN * (t.m0 / BN + 1) <= BM * (col / BM);   // same for all 4 warps
          if (row_ok && col < p.N) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
            if (bias) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col + i < p.N) v[i] += bias[col + i];
            }
            if (p.out_fp32) {
              float* dst = reinterpret_cast<float*>(p.C) + c_off + col;
              const float* src = p.Cin ? reinterpret_cast<const float*>(p.Cin) + c_off + col : nullptr;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                if (col + q * 4 < p.N) {
                  float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
                  if (src) {
                    const float4 s4 = *reinterpret_cast<const float4*>(src + q * 4);
                    o.x += p.beta * s4.x; o.y += p.beta * s4.y; o.z += p.beta * s4.z; o.w += p.beta * s4.w;
                  }
                  *reinterpret_cast<float4*>(dst + q * 4) = o;
                }
              }
            } else {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + col;
              const __nv_bfloat16* src = p.Cin ? reinterpret_cast<const __nv_bfloat16*>(p.Cin) + c_off + col : nullptr;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                if (col + q * 8 < p.N) {
                  if (src) {
                    const uint4 s4 = *reinterpret_cast<const uint4*>(src + q * 8);
                    const __nv_bfloat162* sp = reinterpret_cast<const __nv_bfloat162*>(&s4);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                      const float2 f = __bfloat1622float2(sp[i]);
                      v[q * 8 + 2 * i] += p.beta * f.x;
                      v[q * 8 + 2 * i + 1] += p.beta * f.y;
                    }
                  }
                  uint4 o;
                  o.x = pack_bf16(v[q * 8 + 0], v[q * 8 + 1]);
                  o.y = pack_bf16(v[q * 8 + 2], v[q * 8 + 3]);
                  o.z = pack_bf16(v[q * 8 + 4], v[q * 8 + 5]);
                  o.w = pack_bf16(v[q * 8 + 6], v[q * 8 + 7]);
                  *reinterpret_cast<uint4*>(dst + q * 8) = o;
                }
              }
              if (mirror) {   // stage this row's 32 values column-wise: stg[j][row_in_tile]
                __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * STAGE_BYTES);
#pragma unroll
                for (int i = 0; i < 32; ++i) stg[i * MIRROR_LD + row_in_tile] = __float2bfloat16(v[i]);
              }
            }
          }
          // Symmetric result: the mirror image of this 32-column piece lies in a tile that was skipped iff that tile is
          // wholly below the diagonal. The four epilogue warps then write it from the staged copy, 16 bytes per store:
          // C[col + j][m0 .. m0 + 127] = stg[j][0 .. 127].
          if (mirror) {
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const __nv_bfloat16* stg = reinterpret_cast<const __nv_bfloat16*>(smem + STAGES * STAGE_BYTES);
            __nv_bfloat16* cbase = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)t.gc * p.c_group_stride;
#pragma unroll
            for (int pass = 0; pass < 4; ++pass) {
              const int piece = row_in_tile + 128 * pass, j = piece >> 4, part = piece & 15;
              if (col + j < p.N && t.m0 + part * 8 < p.M)
                *reinterpret_cast<uint4*>(cbase + (long long)(col + j) * p.ldc + t.m0 + part * 8) =
                    *reinterpret_cast<const uint4*>(stg + j * MIRROR_LD + part * 8);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          }
        }
      } else if (EPI == EPI_CE_FWD) {
        // one pass over the tile: online (max, sum exp) per row and the target logit if it lies in this tile
        const int y = row_ok ? p.ce_y[row] : -1;
        float mx = -INFINITY, l = 0.f, tz = 0.f;
        bool has_t = false;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col = t.n0 + c * 32;
          if (col < p.N) {
            float cm = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float z = (col + i < p.N) ? __uint_as_float(r[i]) : -INFINITY;
              r[i] = __float_as_uint(z);
              cm = fmaxf(cm, z);
              if (col + i == y) { tz = z; has_t = true; }
            }
            if (cm > mx) {
              l *= __expf(mx - cm);
              mx = cm;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) l += __expf(__uint_as_float(r[i]) - mx);
          }
        }
        if (row_ok) {
          const long long pi = (long long)(t.n0 / BN) * p.M + row;
          p.ce_part_m[pi] = mx;
          p.ce_part_l[pi] = l;
          if (has_t) p.ce_tgt[row] = tz;
        }
      } else if (EPI == EPI_CE_DZ) {
        // dZ = (softmax - onehot) * g as bf16, softmax recomputed from the stored log-sum-exp
        const int y = row_ok ? p.ce_y[row] : -1;
        const float lse = row_ok ? p.ce_lse[row] : 0.f;
        const float g = *p.ce_gscale;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col = t.n0 + c * 32;
          if (row_ok && col < p.N) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float pr = __expf(__uint_as_float(r[i]) - lse);
              if (col + i == y) pr -= 1.0f;
              v[i] = pr * g;
            }
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + col;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col + q * 8 < p.N) {
                uint4 o;
                o.x = pack_bf16(v[q * 8 + 0], v[q * 8 + 1]);
                o.y = pack_bf16(v[q * 8 + 2], v[q * 8 + 3]);
                o.z = pack_bf16(v[q * 8 + 4], v[q * 8 + 5]);
                o.w = pack_bf16(v[q * 8 + 6], v[q * 8 + 7]);
                *reinterpret_cast<uint4*>(dst + q * 8) = o;
              }
            }
          }
        }
      } else {
        // SwiGLU: accumulator columns [0,BN/2) = gate, [BN/2,BN) = linear, output columns n0 .. n0+BN/2
        const int n_out = p.n_split;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], l[32];
          tmem_ld32(taddr + c * 32, g);
          tmem_ld32(taddr + BN / 2 + c * 32, l);
          tmem_ld_wait();
          const int col = t.n0 + c * 32;
          if (row_ok && col < n_out) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float gv = __uint_as_float(g[i]), lv = __uint_as_float(l[i]);
              if (bias && col + i < n_out) {
                gv += bias[col + i];
                lv += bias[n_out + col + i];
              }
              v[i] = swiglu_act(gv, lv, p.swiglu_beta, p.swiglu_limit);
            }
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + col;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col + q * 8 < n_out) {
                uint4 o;
                o.x = pack_bf16(v[q * 8 + 0], v[q * 8 + 1]);
                o.y = pack_bf16(v[q * 8 + 2], v[q * 8 + 3]);
                o.z = pack_bf16(v[q * 8 + 4], v[q * 8 + 5]);
                o.w = pack_bf16(v[q * 8 + 6], v[q * 8 + 7]);
                *reinterpret_cast<uint4*>(dst + q * 8) = o;
              }
            }
          }
        }
      }
      if (have_acc) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
        ++tile_it;
      }
    }
  }

  // ------------------------------------------------------------ teardown
  __syncthreads();
  if (abort_flag) {
    // let any TMA copy still in flight land before the shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN>
constexpr int gemm_smem_bytes() {
  return ((BN == 256) ? 4 : 6) * (BM * BK * 2 + BN * BK * 2) + 1024 + EPI_STAGE_BYTES;
}

template <int BN, bool A_MN, bool B_MN, int EPI>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  auto kern = gemm_kernel<BN, A_MN, B_MN, EPI>;
  static bool configured = false;
  constexpr int smem = gemm_smem_bytes<BN>();
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    configured = true;
  }
  int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  if (grid <= 0) return 0;
  if (p.ag_world > 0) grid = sm_count();  // every slab needs a copier even if there are few tiles
  kern<<<grid, p.ag_world > 0 ? GEMM_THREADS_AG : GEMM_THREADS, smem, stream>>>(ta, tb, p);
  LYRA_CHECK_LAUNCH();
  return 0;
}

}  // namespace lyra

using namespace lyra;

// Operand description: a row-major 2-D (or stacked 3-D) bf16 array.
//   K-major  operand: rows = M (or N), cols = K        -> mn_major = 0
//   MN-major operand: rows = K,        cols = M (or N)  -> mn_major = 1
// `ld` = elements between rows, `group_stride` = elements between stacked matrices (0 if not stacked).
// Band height (in 128-row tiles) of the grouped tile raster. Measured on B200 (8192 x N x 4096, bf16): bands of 8 take
// N = 12288 from 1244 to 1430 TFLOP/s (forward) and from 1139 to 1305 (weight gradient) and change nothing at N = 4096, where
// a wave of 148 tiles already spans every column panel; so bands are used from 32 column panels on.
// LYRA_GEMM_RASTER_GROUP overrides the choice for every shape (0 = plain M-major).
static int default_raster_group(int n_tiles) {
  static int forced = -2;
  if (forced == -2) {
    const char* e = getenv("LYRA_GEMM_RASTER_GROUP");
    forced = e ? atoi(e) : -1;
    if (forced < -1 || forced > 1024) forced = -1;
  }
  if (forced >= 0) return forced;
  return n_tiles >= 32 ? 8 : 0;
}

extern "C" int lyra_gemm_bf16(
    const void* A, long long lda, long long a_group_stride, int a_mn,
    const void* B, long long ldb, long long b_group_stride, int b_mn,
    void* C, const void* Cin, long long ldc, long long c_group_stride, int out_fp32,
    int M, int N, int K, float alpha, float beta,
    const float* bias, long long bias_group_stride,
    int group_mode, int num_groups, const int* tile_group, const int* group_offsets, int total_rows,
    int epilogue, int n_split, float swiglu_beta, float swiglu_limit, int sym_upper,
    const int* row_dest, const long long* peer_out, int n_peers,
    const float* row_scale, const long long* peer_count, const int* tile_perm, const int* arrive, const int* expect,
    int* status, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8))) return -10;
  if (sym_upper && (M != N || epilogue != EPI_STORE || group_mode == GROUP_M || group_mode == GROUP_K)) return -14;
  if (row_dest && (epilogue != EPI_STORE || out_fp32 || Cin || !peer_out || n_peers < 1 || n_peers > AG_MAX_RANKS || sym_upper)) return -15;
  if ((row_scale || peer_count) && !row_dest) return -16;
  if ((tile_perm || arrive || expect) && group_mode != GROUP_M) return -17;
  if ((arrive != nullptr) != (expect != nullptr)) return -17;
  const int G = num_groups > 0 ? num_groups : 1;
  constexpr int BN = 256;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.Cin = Cin; p.ldc = ldc; p.c_group_stride = c_group_stride; p.out_fp32 = out_fp32;
  p.alpha = alpha; p.beta = beta; p.bias = bias; p.bias_group_stride = bias_group_stride;
  p.group_mode = group_mode; p.tile_group = tile_group; p.group_offsets = group_offsets; p.num_groups = G;
  p.n_split = n_split; p.swiglu_beta = swiglu_beta; p.swiglu_limit = swiglu_limit; p.status = status;
  p.ag_world = 0; p.raster_n_major = 0; p.raster_group = 0; p.sym_upper = sym_upper; p.row_dest = row_dest; p.ce_y = nullptr; p.ce_part_m = nullptr; p.ce_part_l = nullptr; p.ce_tgt = nullptr; p.ce_lse = nullptr; p.ce_gscale = nullptr;
  p.m_tiles = (M + BM - 1) / BM;
  if (epilogue == EPI_SWIGLU) p.n_tiles = (n_split + BN / 2 - 1) / (BN / 2);
  else p.n_tiles = (N + BN - 1) / BN;
  p.total_tiles = p.m_tiles * p.n_tiles * ((group_mode == GROUP_K || group_mode == GROUP_BATCH) ? G : 1);
  p.raster_group = default_raster_group(p.n_tiles);
  for (int r = 0; r < AG_MAX_RANKS; ++r) p.peer_out[r] = (row_dest && r < n_peers) ? reinterpret_cast<void*>(peer_out[r]) : nullptr;
  for (int r = 0; r < AG_MAX_RANKS; ++r) p.peer_count[r] = (row_dest && peer_count && r < n_peers) ? reinterpret_cast<int*>(peer_count[r]) : nullptr;
  p.row_scale = row_scale; p.tile_perm = tile_perm; p.arrive = arrive; p.expect = expect;
  p.sym_tiles = 0;
  if (sym_upper) {
    for (int m = 0; m < p.m_tiles; ++m) p.sym_tiles += p.n_tiles - (p.n_tiles < m * BM / BN ? p.n_tiles : m * BM / BN);
    p.total_tiles = p.sym_tiles * (group_mode == GROUP_BATCH ? G : 1);
  }

  // Tensor maps (3-D: inner, rows, group). Row counts seen by TMA:
  //  A K-major : dims {K, rows_a, Ga};  A MN-major: dims {M, krows, Ga}
  const bool a_grouped = group_mode == GROUP_BATCH;
  const bool b_grouped = group_mode == GROUP_BATCH || group_mode == GROUP_M;
  const uint64_t krows = (group_mode == GROUP_K) ? (uint64_t)total_rows : (uint64_t)K;
  CUtensorMap ta, tb;
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (a_mn) { dims[0] = M; dims[1] = krows; box[0] = 64; box[1] = BK; }
    else      { dims[0] = K; dims[1] = M;     box[0] = 64; box[1] = BM; }
    dims[2] = a_grouped ? G : 1; box[2] = 1;
    strides[0] = (uint64_t)lda * 2;
    strides[1] = a_grouped ? (uint64_t)a_group_stride * 2 : dims[1] * strides[0];
    if (make_tmap_cached(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -11;
  }
  {
    uint64_t dims[3], strides[2];
    uint32_t box[3];
    if (b_mn) { dims[0] = N; dims[1] = krows; box[0] = 64; box[1] = BK; }
    else      { dims[0] = K; dims[1] = N;     box[0] = 64; box[1] = 128; }
    dims[2] = b_grouped ? G : 1; box[2] = 1;
    strides[0] = (uint64_t)ldb * 2;
    strides[1] = b_grouped ? (uint64_t)b_group_stride * 2 : dims[1] * strides[0];
    if (make_tmap_cached(&tb, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -12;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int code = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  if (epilogue == EPI_SWIGLU) {
    switch (code) {
      case 0: return launch_gemm<BN, false, false, EPI_SWIGLU>(ta, tb, p, s);
      case 1: return launch_gemm<BN, false, true, EPI_SWIGLU>(ta, tb, p, s);
      default: return -13;
    }
  }
  switch (code) {
    case 0: return launch_gemm<BN, false, false, EPI_STORE>(ta, tb, p, s);
    case 1: return launch_gemm<BN, false, true, EPI_STORE>(ta, tb, p, s);
    case 2: return launch_gemm<BN, true, false, EPI_STORE>(ta, tb, p, s);
    default: return launch_gemm<BN, true, true, EPI_STORE>(ta, tb, p, s);
  }
}


// Mirrors the upper triangle of G stacked n x n matrices into the lower one: C[r][c] = C[c][r] for r > c (32 x 32 tiles through
// shared memory so that both the read and the write are row-contiguous). Completes a product launched with `sym_upper`.
template <typename T>
__global__ void symmetrize_kernel(T* __restrict__ C, long long ld, long long group_stride, int n) {
  __shared__ T tile[32][33];
  const int bi = blockIdx.y, bj = blockIdx.x;   // destination block (rows bi, columns bj), bi >= bj
  if (bj > bi) return;
  T* base = C + (long long)blockIdx.z * group_stride;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {   // source block: rows bj*32.., columns bi*32..
    const int sr = bj * 32 + r, sc = bi * 32 + threadIdx.x;
    if (sr < n && sc < n) tile[r][threadIdx.x] = base[(long long)sr * ld + sc];
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int dr = bi * 32 + r, dc = bj * 32 + threadIdx.x;
    if (dr < n && dc < n && dr > dc) base[(long long)dr * ld + dc] = tile[threadIdx.x][r];
  }
}

extern "C" int lyra_symmetrize(void* C, long long ld, long long group_stride, int n, int G, int is_fp32, void* stream) {
  if (n <= 0 || G <= 0) return 0;
  dim3 grid((n + 31) / 32, (n + 31) / 32, G), block(32, 8);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (is_fp32) symmetrize_kernel<float><<<grid, block, 0, s>>>(static_cast<float*>(C), ld, group_stride, n);
  else symmetrize_kernel<__nv_bfloat16><<<grid, block, 0, s>>>(static_cast<__nv_bfloat16*>(C), ld, group_stride, n);
  LYRA_CHECK_LAUNCH();
  return 0;
}

// Fused output head + cross entropy, forward: x [M, K] bf16, w [V, K] bf16 (first `vocab` rows used).
// Writes per-tile partial (max, sum-exp) [ceil(vocab/256), M] and the target logit [M]; `lyra_ce_merge` finishes.
// mode 0 = forward partials; mode 1 = dZ[M, vocab] (ld = ldz) = (softmax - onehot) * (*gscale).
extern "C" int lyra_ce_gemm(const void* x, long long ldx, const void* w, long long ldw, const int* y, int M, int vocab, int K, int mode,
                            float* part_m, float* part_l, float* tgt, const float* lse, const float* gscale, void* dz, long long ldz,
                            int* status, void* stream) {
  if (M <= 0) return 0;
  constexpr int BN = 256;
  GemmParams p;
  p.M = M; p.N = vocab; p.K = K;
  p.C = dz; p.Cin = nullptr; p.ldc = ldz; p.c_group_stride = 0; p.out_fp32 = 0;
  p.alpha = 1.f; p.beta = 0.f; p.bias = nullptr; p.bias_group_stride = 0;
  p.group_mode = GROUP_NONE; p.tile_group = nullptr; p.group_offsets = nullptr; p.num_groups = 1;
  p.n_split = 0; p.swiglu_beta = 0.f; p.swiglu_limit = 0.f; p.status = status;
  p.ag_world = 0;
  p.raster_n_major = 1; p.raster_group = 0; p.sym_upper = 0; p.sym_tiles = 0; p.row_dest = nullptr;
  p.row_scale = nullptr; p.tile_perm = nullptr; p.arrive = nullptr; p.expect = nullptr;
  for (int r = 0; r < AG_MAX_RANKS; ++r) p.peer_count[r] = nullptr;
  p.ce_y = y; p.ce_part_m = part_m; p.ce_part_l = part_l; p.ce_tgt = tgt; p.ce_lse = lse; p.ce_gscale = gscale;
  p.m_tiles = (M + BM - 1) / BM;
  p.n_tiles = (vocab + BN - 1) / BN;
  p.total_tiles = p.m_tiles * p.n_tiles;
  CUtensorMap ta, tb;
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, 1}, strides[2] = {(uint64_t)ldx * 2, (uint64_t)M * ldx * 2};
    uint32_t box[3] = {64, BM, 1};
    if (make_tmap_cached(&ta, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -11;
  }
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)vocab, 1}, strides[2] = {(uint64_t)ldw * 2, (uint64_t)vocab * ldw * 2};
    uint32_t box[3] = {64, 128, 1};
    if (make_tmap_cached(&tb, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -12;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return mode == 0 ? launch_gemm<BN, false, false, EPI_CE_FWD>(ta, tb, p, s) : launch_gemm<BN, false, false, EPI_CE_DZ>(ta, tb, p, s);
}

namespace lyra {
// One warp per row: merges the per-tile partials into lse and the row loss (lse - target logit).
__global__ void ce_merge_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l, const float* __restrict__ tgt,
                                float* __restrict__ lse, float* __restrict__ row_loss, int M, int n_tiles) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float m = -INFINITY, l = 0.f;
  for (int t = lane; t < n_tiles; t += 32) {
    const float pm = part_m[(long long)t * M + row], pl = part_l[(long long)t * M + row];
    if (pm > m) {
      l = l * __expf(m - pm) + pl;
      m = pm;
    } else if (pm > -INFINITY) {
      l += pl * __expf(pm - m);
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, s), ol = __shfl_xor_sync(0xffffffffu, l, s);
    const float nm = fmaxf(m, om);
    l = (m > -INFINITY ? l * __expf(m - nm) : 0.f) + (om > -INFINITY ? ol * __expf(om - nm) : 0.f);
    m = nm;
  }
  if (lane == 0) {
    const float v = m + __logf(l);
    lse[row] = v;
    row_loss[row] = v - tgt[row];
  }
}
}  // namespace lyra

extern "C" int lyra_ce_merge(const float* part_m, const float* part_l, const float* tgt, float* lse, float* row_loss, int M, int n_tiles,
                             void* stream) {
  if (M <= 0) return 0;
  lyra::ce_merge_kernel<<<(M + 7) / 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(part_m, part_l, tgt, lse, row_loss, M, n_tiles);
  LYRA_CHECK_LAUNCH();
  return 0;
}


// y[M, N] = x[M, K] @ W[K, N] where W's rows live on peer GPUs (all-gather fused into the GEMM). `w_local` is this
// rank's full-size [K, N] buffer that the kernel fills (rows owned by this rank must already be in place when
// src[my_rank] == w_local); `src[r]` is rank r's peer-mapped base of its rows. `flags` holds ceil(N/256) counters and
// `epoch` counts the calls made on them (1, 2, ...; they start at zero and each call adds ceil(K/64) to each).
extern "C" int lyra_gemm_allgather_bf16(const void* x, long long ldx, void* w_local, long long ldw, const long long* src, int world, int my_rank,
                                        int rows_per_rank, void* y, const void* c_in, long long ldy, int M, int N, int K, float alpha, float beta,
                                        const float* bias, int* flags, int epoch, int* status, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((ldx % 8) || (ldw % 8) || (ldy % 8) || world > AG_MAX_RANKS || world < 1) return -10;
  constexpr int BN = 256;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.C = y; p.Cin = c_in; p.ldc = ldy; p.c_group_stride = 0; p.out_fp32 = 0;
  p.alpha = alpha; p.beta = beta; p.bias = bias; p.bias_group_stride = 0;
  p.group_mode = GROUP_NONE; p.tile_group = nullptr; p.group_offsets = nullptr; p.num_groups = 1;
  p.n_split = 0; p.swiglu_beta = 0.f; p.swiglu_limit = 0.f; p.status = status;
  p.raster_group = 0; p.sym_upper = 0; p.sym_tiles = 0; p.row_dest = nullptr;
  p.row_scale = nullptr; p.tile_perm = nullptr; p.arrive = nullptr; p.expect = nullptr;
  for (int r = 0; r < AG_MAX_RANKS; ++r) p.peer_count[r] = nullptr;
  p.raster_n_major = 1;  // tiles walk M first, column panel by column panel: the order in which the panels of B arrive
  p.ce_y = nullptr; p.ce_part_m = nullptr; p.ce_part_l = nullptr; p.ce_tgt = nullptr; p.ce_lse = nullptr; p.ce_gscale = nullptr;
  p.ag_world = world; p.ag_rows_per_rank = rows_per_rank; p.ag_my_rank = my_rank; p.ag_row_bytes = ldw * 2;
  for (int r = 0; r < AG_MAX_RANKS; ++r) p.ag_src[r] = r < world ? reinterpret_cast<const void*>(src[r]) : nullptr;
  p.ag_dst = w_local; p.ag_flags = flags; p.ag_epoch = epoch;
  p.m_tiles = (M + BM - 1) / BM;
  p.n_tiles = (N + BN - 1) / BN;
  p.total_tiles = p.m_tiles * p.n_tiles;
  CUtensorMap ta, tb;
  {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, 1}, strides[2] = {(uint64_t)ldx * 2, (uint64_t)M * ldx * 2};
    uint32_t box[3] = {64, BM, 1};
    if (make_tmap_cached(&ta, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -11;
  }
  {
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, 1}, strides[2] = {(uint64_t)ldw * 2, (uint64_t)K * ldw * 2};
    uint32_t box[3] = {64, BK, 1};
    if (make_tmap_cached(&tb, w_local, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return -12;
  }
  return launch_gemm<BN, false, true, EPI_STORE>(ta, tb, p, reinterpret_cast<cudaStream_t>(stream));
}
