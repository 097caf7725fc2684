// Allocation-free entry point. This function has no counterpart in the reference library.
//
// Who needs it: code that may not allocate device memory at the point where it wants the RMSNorm
// backward -- a plugin running inside another runtime's memory plan, a host callback, a serving
// loop whose allocator is frozen after start-up. The regular entry point fmb_rmsnorm_bwd() expects
// the caller to hand in a scratch buffer for the per-block weight-gradient partial sums; here that
// scratch is a fixed array that lives in the library's device image instead, so the call performs
// no cudaMalloc / cudaFree and uses no allocating library routine. The caller still owns every
// input and output.
//
// Limits and rules
//   * d (row width) times the number of thread blocks used must fit the built-in scratch:
//     d <= FMB_NOALLOC_MAX_D. Wider rows are refused with FMB_NOALLOC_TOO_LARGE and a message on stderr.
//   * d must be a positive multiple of 8 (the kernels move 16-byte vectors): FMB_NOALLOC_BAD_WIDTH otherwise.
//   * The array costs FMB_NOALLOC_SCRATCH_BYTES of device memory on every GPU that loads the library,
//     until the process exits.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress with that
//     device current) and remembers it. Make that first call before any stream capture begins.
//   * All calls on a device share the one array. Every call overwrites the part it uses before reading
//     it, so nothing has to be cleared between calls; but two calls that run at the same time on the
//     GPU (different streams) would race on it. Keep calls on a device ordered.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FMB_NOALLOC_MAX_D 4096
#define FMB_NOALLOC_MAX_BLOCKS 320
#define FMB_NOALLOC_SCRATCH_BYTES (FMB_NOALLOC_MAX_D * FMB_NOALLOC_MAX_BLOCKS * 4)
#define FMB_NOALLOC_TOO_LARGE (-20)
#define FMB_NOALLOC_SETUP_FAILED (-21)
#define FMB_NOALLOC_BAD_WIDTH (-22)

// dx[rows, d] = RMSNorm backward of dy through y = x * rstd * w;  dw[d] (fp32) = sum over rows.
// dtype / w_dtype: 0 = bf16, 1 = fp32 (as in fmb_api.h). Returns 0, one of the FMB_NOALLOC_* codes above, or the
// regular entry point's codes (-2: an argument it refuses, e.g. a misaligned pointer; -3: the launch failed).
// Safe to call from several host threads; see the ordering rule above for what runs on the GPU.
int fmb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                            long long rows, int d, int dtype, int w_dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
