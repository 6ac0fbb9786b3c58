// RMSNorm backward without any allocation.
//
// This entry point has no counterpart in the reference project; it exists for callers of this library that are not
// able to obtain device memory at call time:
//   * a host program that hands all device memory to its own pool at start-up, so cudaMalloc (and torch's caching
//     allocator) would fail or fight that pool;
//   * a latency-sensitive loop that must not pay the device-wide synchronisation cudaMalloc / cudaFree can imply;
//   * plain C / C++ callers that load the shared library without PyTorch and therefore have no allocator to give the
//     regular entry point (`lyra_rmsnorm_bwd`) its per-block scratch rows.
//
// The regular entry point needs a caller-allocated fp32 scratch of [blocks, C] for the per-block partial sums of the
// scale gradient. Here that scratch is a fixed array inside the library (device memory reserved by every GPU that
// loads the library, for the life of the process): LYRA_RMSNORM_NOALLOC_BLOCKS x LYRA_RMSNORM_NOALLOC_MAX_C floats
// = 4 MiB. The caller passes inputs and outputs only.
//
// Limits and rules:
//   * C must be a multiple of 8 and at most LYRA_RMSNORM_NOALLOC_MAX_C; larger C is rejected with
//     LYRA_NOALLOC_ERR_TOO_LARGE and a message on stderr - nothing is launched.
//   * The first call on each device looks up the device address of the scratch array (one cudaGetSymbolAddress with
//     that device current). Make that first call during set-up, before starting any stream capture on the device.
//   * Every call on a device shares the one scratch array. Two calls whose kernels overlap in time on the same device
//     (different streams, or different host threads) race on it; order them on one stream or with events.
//   * Nothing needs zeroing between calls: each call overwrites every scratch row it later reads. The array keeps the
//     last call's partial sums afterwards.
//   * The call performs no cudaMalloc / cudaFree and calls no allocating library routine.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define LYRA_RMSNORM_NOALLOC_MAX_C 8192
#define LYRA_RMSNORM_NOALLOC_BLOCKS 128
#define LYRA_NOALLOC_ERR_TOO_LARGE (-70)
#define LYRA_NOALLOC_ERR_BAD_SHAPE (-71)
#define LYRA_NOALLOC_ERR_SYMBOL (-72)

// x, dy, dx: [rows, C] bf16 (device). scale: [C] fp32. rstd: [rows] fp32 from the forward pass.
// dscale: [C] fp32 output = sum over rows of dy * x * rstd. Returns 0 on success, a negative code otherwise.
int lyra_rmsnorm_bwd_noalloc(const void* x, const float* scale, const float* rstd, const void* dy, void* dx, float* dscale, int rows, int C,
                             void* stream);

#ifdef __cplusplus
}
#endif
