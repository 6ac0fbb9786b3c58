// NVLink / NVSwitch data movement between the GPUs of one node through peer-mapped (symmetric) memory.
// Every kernel takes raw peer pointers and uses plain 16-byte loads / stores plus system-scope release / acquire
// flags: no collective library call, and nothing that can wait forever - every wait spins for a
// bounded time, then records STATUS_TIMEOUT_PEER in a status word and returns.
//
//   p2p_copy      : pull a buffer from one peer (parameter broadcast from its owner = the all-gather leg of ZeRO-3)
//   reduce_pull   : out = sum over ranks of peer[r][...] in rank order (gradient reduce to the owning rank; deterministic)
//   signal / wait : epoch flags (a stream-ordered barrier across ranks)
//   ep_*          : expert-parallel token exchange - counts push, layout, row dispatch into the owner's expert-sorted
//                   receive buffer, and the return of expert outputs to the source rank's combine buffer
//                   (roles of lyra/kernels/ep_moe.py:9-37,94-127 in the reference)
//   ep_*_sorted / arrivals : the tile-granular form of the exchange. Senders walk their assignments in the order in which
//                   the receivers will consume them (destination rank by destination rank, starting with themselves) and
//                   bump one arrival counter per 128-row tile of the receiver's buffer; the receiver's grouped GEMM waits
//                   for a tile's counter inside its TMA producer (csrc/gemm/gemm.cu) instead of behind an all-rank barrier.
//                   Counters only ever grow: the receiver keeps the running total it expects per tile, so nothing is reset.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/tmap.h"

namespace lyra {

constexpr int MAX_RANKS = 16;
constexpr long long PEER_WAIT_NS = 10000000000LL;  // 10 s: absorbs a peer whose host is busy (first-step allocations); tests pass shorter limits
constexpr int STATUS_PEER_TIMEOUT = 4;
constexpr int STATUS_EP_OVERFLOW = 6;
constexpr int STATUS_RETURN_TIMEOUT = 8;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ long long now_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Spins until *flag >= value or the time limit passes. Returns false on timeout.
__device__ __forceinline__ bool wait_flag(const int* flag, int value, long long limit_ns = PEER_WAIT_NS) {
  const long long start = now_ns();
  while (ld_acquire_sys(flag) < value) {
    if (now_ns() - start > limit_ns) return false;
    __nanosleep(200);
  }
  return true;
}

// ------------------------------------------------------------------------------------------------ copies / reductions
__global__ void p2p_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long n16) {
  // four independent 16-byte loads per thread and step: NVLink reads take microseconds, so bytes in flight set the rate
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = c;
    dst[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) dst[i] = src[i];
}

// fp32 or bf16 inputs on every rank, fp32 (or bf16) output; 8 elements per thread per step.
template <bool IN_BF16, bool OUT_BF16>
__global__ void reduce_pull_kernel(void* __restrict__ out, PeerPtrs peers, int world, long long n) {
  const long long n8 = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      if (IN_BF16) {
        const uint4 v = reinterpret_cast<const uint4*>(peers.p[r])[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(h[k]);
          acc[2 * k] += f.x;
          acc[2 * k + 1] += f.y;
        }
      } else {
        const float4 a = reinterpret_cast<const float4*>(peers.p[r])[2 * i], b = reinterpret_cast<const float4*>(peers.p[r])[2 * i + 1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
    }
    if (OUT_BF16) {
      uint4 o;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
      reinterpret_cast<uint4*>(out)[i] = o;
    } else {
      reinterpret_cast<float4*>(out)[2 * i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

// The same rank-ordered sum, plus the sum of squares of the result on the way out (the optimizer's global-norm gate and Muon's
// per-matrix RMS clip need it; computing it here saves two more passes over every reduced gradient). A leaf may interleave
// `n_seg` (1 or 2) matrices in runs of `seg_len` elements (the gate and linear halves of a `[C, 2, H]` up-projection):
// partial[block][s] receives the block's sum for matrix s; the caller adds the blocks up in order.
template <bool IN_BF16, bool OUT_BF16>
__global__ void reduce_pull_norm_kernel(void* __restrict__ out, PeerPtrs peers, int world, long long n, long long seg_len, int n_seg,
                                        float* __restrict__ partial) {
  __shared__ float red[2][32];
  const long long n8 = n / 8;
  float sq[2] = {0.f, 0.f};
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      if (IN_BF16) {
        const uint4 v = reinterpret_cast<const uint4*>(peers.p[r])[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(h[k]);
          acc[2 * k] += f.x;
          acc[2 * k + 1] += f.y;
        }
      } else {
        const float4 a = reinterpret_cast<const float4*>(peers.p[r])[2 * i], b = reinterpret_cast<const float4*>(peers.p[r])[2 * i + 1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
    }
    float s = 0.f;
    if (OUT_BF16) {
      uint4 o;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        h[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
        const float2 f = __bfloat1622float2(h[k]);   // the norm of what is stored
        s += f.x * f.x + f.y * f.y;
      }
      reinterpret_cast<uint4*>(out)[i] = o;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) s += acc[k] * acc[k];
      reinterpret_cast<float4*>(out)[2 * i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    const int seg = n_seg > 1 ? int(((i * 8) / seg_len) % n_seg) : 0;
    sq[seg] += s;
  }
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    float v = sq[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[t][threadIdx.x >> 5] = v;
  }
  __syncthreads();
  if (threadIdx.x < 2) {
    float v = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) v += red[threadIdx.x][w];
    partial[blockIdx.x * 2 + threadIdx.x] = v;
  }
}

// In-switch all-reduce (NVLS) of a small buffer that every rank holds at the same offset of a symmetric allocation bound to an
// NVLink multicast object: `mc` is the multicast address of that buffer. Rank r owns the r-th slice: one `multimem.ld_reduce`
// returns the sum over all ranks' copies (added inside the switch: one load instead of `world` peer loads), one `multimem.st`
// writes the sum back into every rank's copy. The caller brackets the kernel with the flag barrier: every rank's copy written
// before, every slice stored before anyone reads its own copy.
__global__ void multimem_all_reduce_kernel(float* mc, long long n4, int world, int my_rank) {
  const long long per = (n4 + world - 1) / world;
  const long long lo = per * my_rank, hi = lo + per < n4 ? lo + per : n4;
  for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (long long)gridDim.x * blockDim.x) {
    float4 v;
    float* a = mc + 4 * i;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(a)
                 : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ flags
// Thread r writes `value` into slot [my_rank] of rank r's flag array (after all earlier writes of this stream).
__global__ void signal_kernel(PeerPtrs flag_arrays, int world, int my_rank, int value) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flag_arrays.p[r]) + my_rank, value);
  }
}
// Thread r waits until slot [r] of the local flag array reaches `value`.
__global__ void wait_kernel(const int* __restrict__ flags, int world, int value, int* status, long long limit_ns) {
  const int r = threadIdx.x;
  if (r < world && !wait_flag(flags + r, value, limit_ns)) atomicExch(status, STATUS_PEER_TIMEOUT);
}

// Device-resident epochs. The host-valued versions above bake the epoch into the launch, which a replayed CUDA graph cannot
// change; here the epoch lives in a counter in this GPU's memory: the signalling kernel increments it and raises the new
// value on every peer, the waiting kernel reads it. Every rank runs the same sequence, so the counters agree.
__global__ void signal_ctr_kernel(PeerPtrs flag_arrays, int world, int my_rank, int* ctr) {
  __shared__ int v;
  if (threadIdx.x == 0) {
    v = *ctr + 1;
    *ctr = v;
  }
  __syncthreads();
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flag_arrays.p[r]) + my_rank, v);
  }
}
__global__ void wait_ctr_kernel(const int* __restrict__ flags, int world, const int* __restrict__ ctr, int* status, long long limit_ns) {
  const int r = threadIdx.x;
  const int value = *ctr;
  if (r < world && !wait_flag(flags + r, value, limit_ns)) atomicExch(status, STATUS_PEER_TIMEOUT);
}
// One block: this rank's per-expert counts into row [my_rank] of every rank's counts matrix, then its flag (epoch = ++*ctr).
__global__ void ep_counts_push_ctr_kernel(const int* __restrict__ my_counts, PeerPtrs counts_mats, PeerPtrs flag_arrays, int world, int my_rank,
                                          int n_experts, int* ctr) {
  __shared__ int v;
  if (threadIdx.x == 0) {
    v = *ctr + 1;
    *ctr = v;
  }
  for (int r = 0; r < world; ++r) {
    int* dst = reinterpret_cast<int*>(counts_mats.p[r]) + (long long)my_rank * n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) dst[e] = my_counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) st_release_sys(reinterpret_cast<int*>(flag_arrays.p[threadIdx.x]) + my_rank, v);
}

// ------------------------------------------------------------------------------------------------ expert-parallel exchange
// Writes this rank's per-expert counts into row [my_rank] of every rank's counts matrix, then raises its flag there.
__global__ void ep_counts_push_kernel(const int* __restrict__ my_counts, PeerPtrs counts_mats, PeerPtrs flag_arrays, int world, int my_rank,
                                      int n_experts, int epoch) {
  const int r = blockIdx.x;  // destination rank
  int* dst = reinterpret_cast<int*>(counts_mats.p[r]) + (long long)my_rank * n_experts;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) dst[e] = my_counts[e];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) st_release_sys(reinterpret_cast<int*>(flag_arrays.p[r]) + my_rank, epoch);
}

// One block. From counts[world][E] (all ranks' routed counts):
//   send_base[e]   : row in the owner's receive buffer where this rank's rows of expert e start
//   recv_offsets   : [E_local + 1] padded (x128) row offsets of this rank's local experts
//   tile_group     : [cap_rows / 128] local expert of each 128-row tile, -1 beyond the used rows
// Receive layout is expert-major, then source-rank-major (lyra/kernels/ep_moe.py:9-37), each expert padded to 128 rows.
__global__ void ep_layout_kernel(const int* __restrict__ counts, int world, int my_rank, int n_experts, int e_local, int cap_rows,
                                 int* __restrict__ send_base, int* __restrict__ recv_offsets, int* __restrict__ tile_group,
                                 int* __restrict__ recv_total, int* __restrict__ valid, int* status) {
  extern __shared__ int sh[];  // per-expert totals [E], padded bases [E]
  int* total = sh;
  int* base = sh + n_experts;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < world; ++s) t += counts[s * n_experts + e];
    total[e] = t;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int d = 0; d < world; ++d) {
      int off = 0;
      for (int j = 0; j < e_local; ++j) {
        const int e = d * e_local + j;
        base[e] = off;
        if (d == my_rank) {
          recv_offsets[j] = off < cap_rows ? off : cap_rows;
          if (valid) valid[j] = min(total[e], max(cap_rows - off, 0));     // real rows of local expert j (its group is padded to 128)
        }
        off += (total[e] + 127) / 128 * 128;
      }
      // Too small a buffer is reported, never written past: senders drop rows beyond the capacity and every offset that later
      // kernels index with is clamped to it, so the step's numbers are wrong but no access leaves the buffers.
      if (off > cap_rows) atomicExch(status, STATUS_EP_OVERFLOW);
      if (d == my_rank) {
        recv_offsets[e_local] = off < cap_rows ? off : cap_rows;
        *recv_total = off < cap_rows ? off : cap_rows;
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < my_rank; ++s) before += counts[s * n_experts + e];
    send_base[e] = base[e] + before;
  }
  const int used = recv_offsets[e_local] < cap_rows ? recv_offsets[e_local] : cap_rows;
  for (int t = threadIdx.x; t < cap_rows / 128; t += blockDim.x) {
    const int row = t * 128;
    int g = -1;
    if (row < used) {
      for (int j = 0; j < e_local; ++j)
        if (row >= recv_offsets[j] && row < recv_offsets[j + 1]) g = j;
    }
    tile_group[t] = g;
  }
}

// One block per assignment a = f * K + k: copies the source row into the owner's receive buffer and records (rank, a).
// `src_div` = K when the source rows are tokens (forward: row a / K), 1 when they are per-assignment rows (backward).
__global__ void ep_dispatch_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ expert_of, const int* __restrict__ rank_in_expert,
                                   const int* __restrict__ send_base, PeerPtrs recv_bufs, PeerPtrs recv_meta, int my_rank, int e_local, int cap_rows,
                                   int n_assign, int src_div, int C) {
  const int a = blockIdx.x;
  if (a >= n_assign) return;
  const int e = expert_of[a];
  const int d = e / e_local;
  const int row = send_base[e] + rank_in_expert[a];
  if (row >= cap_rows) return;  // overflow was flagged by the layout kernel
  const uint4* s = reinterpret_cast<const uint4*>(src + (long long)(a / src_div) * C);
  uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recv_bufs.p[d]) + (long long)row * C);
  for (int c = threadIdx.x; c < C / 8; c += blockDim.x) o[c] = s[c];
  if (threadIdx.x == 0 && recv_meta.p[d]) reinterpret_cast<int*>(recv_meta.p[d])[row] = (my_rank << 24) | a;
}

// One block per received row: sends the row back to slot a of the source rank's return buffer.
__global__ void ep_return_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ meta, const int* __restrict__ recv_offsets,
                                 const int* __restrict__ counts, int world, int my_rank, int n_experts, int e_local, PeerPtrs ret_bufs, int C) {
  const int row = blockIdx.x;
  if (row >= recv_offsets[e_local]) return;
  // is the row a real one (not expert padding)?
  int j = 0;
  while (j + 1 < e_local && row >= recv_offsets[j + 1]) ++j;
  int valid = 0;
  for (int s = 0; s < world; ++s) valid += counts[s * n_experts + my_rank * e_local + j];
  if (row - recv_offsets[j] >= valid) return;
  const int m = meta[row];
  const int src_rank = m >> 24, a = m & 0xFFFFFF;
  const uint4* s = reinterpret_cast<const uint4*>(rows + (long long)row * C);
  uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(ret_bufs.p[src_rank]) + (long long)a * C);
  for (int c = threadIdx.x; c < C / 8; c += blockDim.x) o[c] = s[c];
}

// dest[row] = meta[row] (source rank << 24 | slot) for real rows of the receive buffer, -1 for expert padding and unused rows:
// the scatter map of the GEMM whose epilogue returns expert outputs straight into the source ranks' buffers.
__global__ void ep_row_dest_kernel(const int* __restrict__ meta, const int* __restrict__ recv_offsets, const int* __restrict__ counts, int world,
                                   int my_rank, int n_experts, int e_local, int cap_rows, int* __restrict__ dest) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= cap_rows) return;
  int out = -1;
  if (row < recv_offsets[e_local]) {
    int j = 0;
    while (j + 1 < e_local && row >= recv_offsets[j + 1]) ++j;
    int valid = 0;
    for (int s = 0; s < world; ++s) valid += counts[s * n_experts + my_rank * e_local + j];
    if (row - recv_offsets[j] < valid) out = meta[row];
  }
  dest[row] = out;
}

// Zeroes the padding rows of the receive buffer (rows of an expert beyond its real count), so they contribute nothing to dW.
__global__ void ep_zero_pad_kernel(__nv_bfloat16* __restrict__ rows, const int* __restrict__ recv_offsets, const int* __restrict__ counts, int world,
                                   int my_rank, int n_experts, int e_local, int C) {
  const int row = blockIdx.x;
  if (row >= recv_offsets[e_local]) return;
  int j = 0;
  while (j + 1 < e_local && row >= recv_offsets[j + 1]) ++j;
  int valid = 0;
  for (int s = 0; s < world; ++s) valid += counts[s * n_experts + my_rank * e_local + j];
  if (row - recv_offsets[j] < valid) return;
  uint4* o = reinterpret_cast<uint4*>(rows + (long long)row * C);
  for (int c = threadIdx.x; c < C / 8; c += blockDim.x) o[c] = make_uint4(0, 0, 0, 0);
}

// ------------------------------------------------------------------------------------------------ tile-granular exchange
// Block-wide exclusive scan of one 0/1 flag per thread (blockDim.x <= 1024); returns this thread's rank among the set
// flags and, through `total`, their number. `warp_sums` is 32 ints of shared memory.
__device__ __forceinline__ int block_rank_of_flag(bool flag, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
  const unsigned ballot = __ballot_sync(0xffffffffu, flag);
  const int in_warp = __popc(ballot & ((1u << lane) - 1u));
  if (lane == 0) warp_sums[warp] = __popc(ballot);
  __syncthreads();
  int before = 0, all = 0;
  for (int w = 0; w < n_warps; ++w) {
    const int c = warp_sums[w];
    if (w < warp) before += c;
    all += c;
  }
  __syncthreads();
  total = all;
  return before + in_warp;
}

// Layout of one exchange, one block. Everything `ep_layout_kernel` computes, plus what the tile-granular path needs:
//   starts[E + 1]      : exclusive prefix of this rank's own per-expert counts (position of expert e's run in the sender's
//                        expert-sorted assignment list); starts[E] = number of assignments
//   send_starts[E + 1] : the order in which this rank SENDS its runs: by local expert index j first, then by destination
//                        starting with itself (k = j * world + t  ->  expert ((my_rank + t) % world) * e_local + j); entry k is
//                        the number of assignments sent before run k. Every receiver thus gets all of its expert 0's rows
//                        first, then expert 1's, ... (it consumes tiles expert by expert, which keeps one expert's weights in L2),
//                        while at any moment the senders target different destinations (no incast).
//   tile_valid[t]      : real (non-padding) rows in 128-row tile t of the receive buffer, 0 for unused tiles
//   tile_perm[i]       : the used tiles in the order in which they complete under that sending order: by expert, inside an expert
//                        by the step (my_rank - source) mod world of the last source that contributes rows to the tile, then by
//                        row; -1 after the last used tile. The grouped GEMM enumerates its row tiles through this list.
__global__ void ep_layout_tiles_kernel(const int* __restrict__ counts, int world, int my_rank, int n_experts, int e_local, int cap_rows,
                                       int* __restrict__ send_base, int* __restrict__ recv_offsets, int* __restrict__ tile_group,
                                       int* __restrict__ recv_total, int* __restrict__ starts, int* __restrict__ send_starts,
                                       int* __restrict__ tile_valid, int* __restrict__ tile_perm, int* status) {
  extern __shared__ int sh[];  // totals [E], padded bases [E], warp sums [32], step of each tile [cap_rows / 128]
  int* total = sh;
  int* base = sh + n_experts;
  int* warp_sums = base + n_experts;
  int* step_of = warp_sums + 32;
  __shared__ int filled;
  const int n_tiles = cap_rows / 128;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int t = 0;
    for (int s = 0; s < world; ++s) t += counts[s * n_experts + e];
    total[e] = t;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int d = 0; d < world; ++d) {
      int off = 0;
      for (int j = 0; j < e_local; ++j) {
        const int e = d * e_local + j;
        base[e] = off;
        if (d == my_rank) recv_offsets[j] = off < cap_rows ? off : cap_rows;
        off += (total[e] + 127) / 128 * 128;
      }
      // Too small a buffer is reported, never written past: senders drop rows beyond the capacity and every offset that later
      // kernels index with is clamped to it, so the step's numbers are wrong but no access leaves the buffers.
      if (off > cap_rows) atomicExch(status, STATUS_EP_OVERFLOW);
      if (d == my_rank) {
        recv_offsets[e_local] = off < cap_rows ? off : cap_rows;
        *recv_total = off < cap_rows ? off : cap_rows;
      }
    }
    int run = 0;
    for (int e = 0; e < n_experts; ++e) {
      starts[e] = run;
      run += counts[my_rank * n_experts + e];
    }
    starts[n_experts] = run;
    run = 0;
    for (int k = 0; k < n_experts; ++k) {
      const int j = k / world, t = k - j * world;
      send_starts[k] = run;
      run += counts[my_rank * n_experts + ((my_rank + t) % world) * e_local + j];
    }
    send_starts[n_experts] = run;
    filled = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < my_rank; ++s) before += counts[s * n_experts + e];
    send_base[e] = base[e] + before;
  }
  const int used = recv_offsets[e_local] < cap_rows ? recv_offsets[e_local] : cap_rows;
  for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) {
    const int row = t * 128;
    int g = -1, valid = 0, step = -1;
    if (row < used) {
      for (int j = 0; j < e_local; ++j)
        if (row >= recv_offsets[j] && row < recv_offsets[j + 1]) g = j;
    }
    if (g >= 0) {
      const int e = my_rank * e_local + g;
      const int r0 = row - recv_offsets[g];
      const int r1 = min(r0 + 128, total[e]);
      valid = max(r1 - r0, 0);
      int lo = 0;                               // rows of sources before s in this expert
      for (int s = 0; s < world; ++s) {
        const int c = counts[s * n_experts + e];
        if (c > 0 && lo < r1 && lo + c > r0) step = max(step, (my_rank - s + world) % world);
        lo += c;
      }
    }
    tile_group[t] = g;
    tile_valid[t] = valid;
    step_of[t] = valid > 0 ? g * world + step : -1;   // sort key: expert, then arrival step
  }
  __syncthreads();
  for (int k = 0; k < e_local * world; ++k) {
    for (int t0 = 0; t0 < n_tiles; t0 += blockDim.x) {
      const int t = t0 + threadIdx.x;
      const bool mine = t < n_tiles && step_of[t] == k;
      int n_set;
      const int pos = block_rank_of_flag(mine, warp_sums, n_set);
      if (mine) tile_perm[filled + pos] = t;
      __syncthreads();
      if (threadIdx.x == 0) filled += n_set;
      __syncthreads();
    }
  }
  for (int i = filled + threadIdx.x; i < n_tiles; i += blockDim.x) tile_perm[i] = -1;
}

// expect[t] += tile_valid[t]: the receiver's running total of rows that must have arrived in tile t once the dispatch that is
// about to start has landed. Wrap-around is harmless (waits compare differences).
__global__ void ep_expect_bump_kernel(int* __restrict__ expect, const int* __restrict__ tile_valid, int n_tiles) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n_tiles) expect[t] += tile_valid[t];
}

// One block per assignment, taken in the sender's order (see ep_layout_tiles_kernel): copies the source row into the owner's
// receive buffer, records (rank, slot) and optionally the routing score beside it, then adds one to the arrival counter of the
// row's 128-row tile on the owner (release at system scope: the row is visible before the count).
__global__ void ep_dispatch_sorted_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ order, const int* __restrict__ starts,
                                          const int* __restrict__ send_base, const int* __restrict__ send_starts,
                                          const float* __restrict__ scores, PeerPtrs recv_bufs, PeerPtrs recv_meta, PeerPtrs recv_score,
                                          PeerPtrs arrive, int world, int my_rank, int n_experts, int e_local, int cap_rows, int n_assign, int src_div,
                                          int C) {
  const int i = blockIdx.x;
  if (i >= n_assign || i >= send_starts[n_experts]) return;
  int lo = 0, hi = n_experts;                    // last run k with send_starts[k] <= i
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (send_starts[mid] <= i) lo = mid; else hi = mid;
  }
  const int j = lo / world, t = lo - j * world;
  const int d = (my_rank + t) % world;
  const int e = d * e_local + j;
  const int pos = i - send_starts[lo];           // position inside expert e's run (token order)
  const int a = order[starts[e] + pos];
  const int row = send_base[e] + pos;
  if (row >= cap_rows) return;  // overflow was flagged by the layout kernel
  const uint4* s = reinterpret_cast<const uint4*>(src + (long long)(a / src_div) * C);
  uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recv_bufs.p[d]) + (long long)row * C);
  for (int c = threadIdx.x; c < C / 8; c += blockDim.x) o[c] = s[c];
  if (threadIdx.x == 0) {
    if (recv_meta.p[d]) reinterpret_cast<int*>(recv_meta.p[d])[row] = (my_rank << 24) | a;
    if (scores && recv_score.p[d]) reinterpret_cast<float*>(recv_score.p[d])[row] = scores[a];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(reinterpret_cast<int*>(arrive.p[d]) + row / 128) : "memory");
  }
}

// Stream-ordered wait for rows that other ranks store into a buffer of this rank: *expect += add (this rank's running total,
// kept on the device so that a replayed CUDA graph advances it), then spin until the arrival counter that the storing kernels
// bump has caught up. Bounded like every wait here.
__global__ void wait_arrivals_kernel(const int* __restrict__ arrived, int* __restrict__ expect, int add, int* status, long long limit_ns) {
  if (threadIdx.x != 0) return;
  const int want = *expect + add;
  *expect = want;
  const long long start = now_ns();
  while (ld_acquire_sys(arrived) - want < 0) {
    if (*reinterpret_cast<volatile int*>(status) != 0) return;   // an earlier kernel already failed (e.g. rows dropped on overflow): do not wait for them
    if (now_ns() - start > limit_ns) {
      atomicCAS(status, 0, STATUS_RETURN_TIMEOUT);
      return;
    }
    __nanosleep(200);
  }
}

static PeerPtrs make_ptrs(const long long* ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return p;
}
static inline int copy_grid(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  return int(b < cap ? (b > 0 ? b : 1) : cap);
}

}  // namespace lyra

using namespace lyra;
#define ST(x) reinterpret_cast<cudaStream_t>(x)

extern "C" int lyra_p2p_copy(void* dst, const void* src, long long nbytes, void* stream) {
  if (nbytes <= 0) return 0;
  if (nbytes % 16 || (reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) % 16) return -50;
  p2p_copy_kernel<<<copy_grid(nbytes / 16), 256, 0, ST(stream)>>>(reinterpret_cast<uint4*>(dst), reinterpret_cast<const uint4*>(src), nbytes / 16);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_reduce_pull(void* out, const long long* peer_ptrs, int world, long long n, int in_bf16, int out_bf16, void* stream) {
  if (n <= 0) return 0;
  if (n % 8 || world > MAX_RANKS) return -51;
  const PeerPtrs p = make_ptrs(peer_ptrs, world);
  const int grid = copy_grid(n / 8);
  if (in_bf16 && out_bf16) reduce_pull_kernel<true, true><<<grid, 256, 0, ST(stream)>>>(out, p, world, n);
  else if (in_bf16) reduce_pull_kernel<true, false><<<grid, 256, 0, ST(stream)>>>(out, p, world, n);
  else if (out_bf16) reduce_pull_kernel<false, true><<<grid, 256, 0, ST(stream)>>>(out, p, world, n);
  else reduce_pull_kernel<false, false><<<grid, 256, 0, ST(stream)>>>(out, p, world, n);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_signal(const long long* flag_arrays, int world, int my_rank, int value, void* stream) {
  signal_kernel<<<1, 32, 0, ST(stream)>>>(make_ptrs(flag_arrays, world), world, my_rank, value);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_wait(const int* flags, int world, int value, int* status, void* stream) {
  wait_kernel<<<1, 32, 0, ST(stream)>>>(flags, world, value, status, PEER_WAIT_NS);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_signal_ctr(const long long* flag_arrays, int world, int my_rank, int* ctr, void* stream) {
  signal_ctr_kernel<<<1, 32, 0, ST(stream)>>>(make_ptrs(flag_arrays, world), world, my_rank, ctr);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_wait_ctr(const int* flags, int world, const int* ctr, int* status, void* stream) {
  wait_ctr_kernel<<<1, 32, 0, ST(stream)>>>(flags, world, ctr, status, PEER_WAIT_NS);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_counts_push_ctr(const int* my_counts, const long long* counts_mats, const long long* flag_arrays, int world, int my_rank,
                                       int n_experts, int* ctr, void* stream) {
  ep_counts_push_ctr_kernel<<<1, 128, 0, ST(stream)>>>(my_counts, make_ptrs(counts_mats, world), make_ptrs(flag_arrays, world), world, my_rank,
                                                       n_experts, ctr);
  LYRA_CHECK_LAUNCH();
  return 0;
}

// The same wait with a caller-chosen limit (clamped to the 2 s default): a peer that never raises its flag makes the kernel
// give up after `limit_ms`, record the peer-timeout code in `status` and return, so the host can tell a dead peer from a
// slow one and the CUDA context stays usable.
extern "C" int lyra_wait_limit(const int* flags, int world, int value, int* status, int limit_ms, void* stream) {
  long long ns = (long long)limit_ms * 1000000LL;
  if (ns <= 0 || ns > PEER_WAIT_NS) ns = PEER_WAIT_NS;
  wait_kernel<<<1, 32, 0, ST(stream)>>>(flags, world, value, status, ns);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_counts_push(const int* my_counts, const long long* counts_mats, const long long* flag_arrays, int world, int my_rank,
                                   int n_experts, int epoch, void* stream) {
  ep_counts_push_kernel<<<world, 128, 0, ST(stream)>>>(my_counts, make_ptrs(counts_mats, world), make_ptrs(flag_arrays, world), world, my_rank,
                                                       n_experts, epoch);
  LYRA_CHECK_LAUNCH();
  return 0;
}

// valid (optional): [e_local] real row counts of this rank's experts
extern "C" int lyra_ep_layout(const int* counts, int world, int my_rank, int n_experts, int e_local, int cap_rows, int* send_base,
                              int* recv_offsets, int* tile_group, int* recv_total, int* valid, int* status, void* stream) {
  ep_layout_kernel<<<1, 256, 2 * n_experts * sizeof(int), ST(stream)>>>(counts, world, my_rank, n_experts, e_local, cap_rows, send_base, recv_offsets,
                                                                         tile_group, recv_total, valid, status);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_dispatch(const void* src, const int* expert_of, const int* rank_in_expert, const int* send_base, const long long* recv_bufs,
                                const long long* recv_meta, int world, int my_rank, int e_local, int cap_rows, int n_assign, int src_div, int C,
                                void* stream) {
  if (n_assign <= 0) return 0;
  if (C % 8) return -52;
  PeerPtrs meta = recv_meta ? make_ptrs(recv_meta, world) : make_ptrs(recv_bufs, 0);
  ep_dispatch_kernel<<<n_assign, 128, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(src), expert_of, rank_in_expert, send_base,
                                                       make_ptrs(recv_bufs, world), meta, my_rank, e_local, cap_rows, n_assign, src_div, C);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_return(const void* rows, const int* meta, const int* recv_offsets, const int* counts, int world, int my_rank, int n_experts,
                              int e_local, const long long* ret_bufs, int cap_rows, int C, void* stream) {
  ep_return_kernel<<<cap_rows, 128, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(rows), meta, recv_offsets, counts, world, my_rank,
                                                     n_experts, e_local, make_ptrs(ret_bufs, world), C);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_row_dest(const int* meta, const int* recv_offsets, const int* counts, int world, int my_rank, int n_experts, int e_local,
                                int cap_rows, int* dest, void* stream) {
  ep_row_dest_kernel<<<(cap_rows + 255) / 256, 256, 0, ST(stream)>>>(meta, recv_offsets, counts, world, my_rank, n_experts, e_local, cap_rows, dest);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_zero_pad(void* rows, const int* recv_offsets, const int* counts, int world, int my_rank, int n_experts, int e_local,
                                int cap_rows, int C, void* stream) {
  ep_zero_pad_kernel<<<cap_rows, 128, 0, ST(stream)>>>(reinterpret_cast<__nv_bfloat16*>(rows), recv_offsets, counts, world, my_rank, n_experts,
                                                       e_local, C);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_layout_tiles(const int* counts, int world, int my_rank, int n_experts, int e_local, int cap_rows, int* send_base,
                                    int* recv_offsets, int* tile_group, int* recv_total, int* starts, int* send_starts, int* tile_valid,
                                    int* tile_perm, int* status, void* stream) {
  if (world > MAX_RANKS || cap_rows % 128) return -53;
  const size_t smem = (2 * (size_t)n_experts + 32 + cap_rows / 128) * sizeof(int);
  if (smem > 200 * 1024) return -54;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(ep_layout_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return -4;
    configured = true;
  }
  ep_layout_tiles_kernel<<<1, 1024, smem, ST(stream)>>>(counts, world, my_rank, n_experts, e_local, cap_rows, send_base, recv_offsets, tile_group,
                                                          recv_total, starts, send_starts, tile_valid, tile_perm, status);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_expect_bump(int* expect, const int* tile_valid, int n_tiles, void* stream) {
  if (n_tiles <= 0) return 0;
  ep_expect_bump_kernel<<<(n_tiles + 255) / 256, 256, 0, ST(stream)>>>(expect, tile_valid, n_tiles);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_ep_dispatch_sorted(const void* src, const int* order, const int* starts, const int* send_base, const int* send_starts,
                                       const float* scores, const long long* recv_bufs, const long long* recv_meta, const long long* recv_score,
                                       const long long* arrive, int world, int my_rank, int n_experts, int e_local, int cap_rows, int n_assign,
                                       int src_div, int C, void* stream) {
  if (n_assign <= 0) return 0;
  if (C % 8 || world > MAX_RANKS || !arrive || n_experts != world * e_local) return -52;
  const PeerPtrs none = make_ptrs(recv_bufs, 0);
  ep_dispatch_sorted_kernel<<<n_assign, 128, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(src), order, starts, send_base, send_starts, scores,
                                                              make_ptrs(recv_bufs, world), recv_meta ? make_ptrs(recv_meta, world) : none,
                                                              recv_score ? make_ptrs(recv_score, world) : none, make_ptrs(arrive, world), world,
                                                              my_rank, n_experts, e_local, cap_rows, n_assign, src_div, C);
  LYRA_CHECK_LAUNCH();
  return 0;
}

extern "C" int lyra_wait_arrivals(const int* arrived, int* expect, int add, int* status, int limit_ms, void* stream) {
  long long ns = (long long)limit_ms * 1000000LL;
  if (ns <= 0 || ns > PEER_WAIT_NS) ns = PEER_WAIT_NS;
  wait_arrivals_kernel<<<1, 32, 0, ST(stream)>>>(arrived, expect, add, status, ns);
  LYRA_CHECK_LAUNCH();
  return 0;
}

// `lyra_reduce_pull` that also writes per-block sums of squares of the result: partial [grid, 2] fp32 where grid is the return
// value of `lyra_reduce_pull_norm_blocks(n)`; seg_len must be a multiple of 8 when n_seg == 2.
extern "C" int lyra_reduce_pull_norm_blocks(long long n) { return copy_grid(n / 8); }

extern "C" int lyra_reduce_pull_norm(void* out, const long long* peer_ptrs, int world, long long n, int in_bf16, int out_bf16, long long seg_len, int n_seg,
                                     float* partial, void* stream) {
  if (n <= 0) return 0;
  if (n % 8 || world > MAX_RANKS || n_seg < 1 || n_seg > 2 || (n_seg == 2 && (seg_len <= 0 || seg_len % 8))) return -51;
  const PeerPtrs p = make_ptrs(peer_ptrs, world);
  const int grid = copy_grid(n / 8);
  if (in_bf16 && out_bf16) reduce_pull_norm_kernel<true, true><<<grid, 256, 0, ST(stream)>>>(out, p, world, n, seg_len, n_seg, partial);
  else if (in_bf16) reduce_pull_norm_kernel<true, false><<<grid, 256, 0, ST(stream)>>>(out, p, world, n, seg_len, n_seg, partial);
  else if (out_bf16) reduce_pull_norm_kernel<false, true><<<grid, 256, 0, ST(stream)>>>(out, p, world, n, seg_len, n_seg, partial);
  else reduce_pull_norm_kernel<false, false><<<grid, 256, 0, ST(stream)>>>(out, p, world, n, seg_len, n_seg, partial);
  LYRA_CHECK_LAUNCH();
  return 0;
}

// `mc`: multicast address of an fp32 buffer of n elements (n a multiple of 4) present on every rank; see the kernel's comment for
// the barriers the caller owes.
extern "C" int lyra_multimem_all_reduce(void* mc, long long n, int world, int my_rank, void* stream) {
  if (n <= 0) return 0;
  if (!mc || n % 4 || world < 1 || world > MAX_RANKS || my_rank < 0 || my_rank >= world) return -55;
  const long long n4 = n / 4, per = (n4 + world - 1) / world;
  multimem_all_reduce_kernel<<<copy_grid(per), 256, 0, ST(stream)>>>(static_cast<float*>(mc), n4, world, my_rank);
  LYRA_CHECK_LAUNCH();
  return 0;
}
