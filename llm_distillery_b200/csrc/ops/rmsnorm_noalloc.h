// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference implementation; it exists for hosts of this library that
// cannot hand the kernel a scratch buffer of their own: processes whose device memory is owned entirely by another
// runtime's arena (so a cudaMalloc made here would fail or fragment it), latency-critical loops where cudaMalloc /
// cudaFree are banned because they synchronise the whole device, and plain C callers that load the shared object
// without any tensor library to allocate through.
//
// The regular entry point (b200_rmsnorm_bwd) takes the fp32 partial-sum workspace for the weight gradient from its
// caller. This variant keeps that workspace in a file-scope __device__ array instead:
//   * size: B200_RMSNORM_NOALLOC_MAX_BLOCKS x B200_RMSNORM_NOALLOC_MAX_H floats = 4 MiB, resident on every GPU that
//     loads the library until the process exits;
//   * limit: h <= B200_RMSNORM_NOALLOC_MAX_H (and h % 8 == 0). Larger rows are refused with B200_ERR_TOO_BIG (-4) and
//     a message readable through b200_last_cuda_error(); nothing is launched;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress) with that device
//     current. Make that first call outside any stream capture. The address is remembered per device for the life
//     of the process and is not valid across cudaDeviceReset: a process that resets a device must not call this
//     entry point on it afterwards;
//   * every call on a device shares the one array. A call overwrites the rows it uses before reading them, so
//     nothing has to be cleared between calls, but two calls that overlap in time on one GPU (different streams)
//     would corrupt each other's partial sums: serialise them;
//   * no cudaMalloc, cudaFree or allocating library routine is called. Inputs and outputs are the caller's.
#pragma once
#include <cuda_runtime.h>

#define B200_RMSNORM_NOALLOC_MAX_H 4096
#define B200_RMSNORM_NOALLOC_MAX_BLOCKS 256

#ifdef __cplusplus
extern "C" {
#endif

// dx[rows,h] = rmsnorm backward of dy through (x, w, rstd), plus dres when given; dw_out[h] (fp32) receives
// sum_rows dy * xhat, added to its previous content when dw_accumulate != 0. All pointers are device pointers;
// dy / x / w / dres / dx are bf16, rstd / dw_out fp32. Returns 0, or a negative B200_ERR_* code.
int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                             void* dx, float* dw_out, int dw_accumulate, int rows, int h, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
