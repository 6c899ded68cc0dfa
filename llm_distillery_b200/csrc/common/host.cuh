// Host-side helpers shared by every launcher: TMA tensor-map encoding (driver entry point
// fetched through the runtime, so nothing links against libcuda), the per-device error word
// that bounded in-kernel waits report into, and small launch utilities.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdint.h>
#include <stdio.h>

namespace b200 {

// Return codes of the extern "C" launchers.
enum : int {
  B200_OK = 0,
  B200_ERR_ARG = -1,      // bad shape / alignment / null pointer
  B200_ERR_CUDA = -2,     // a CUDA runtime call failed (see b200_last_cuda_error)
  B200_ERR_TMAP = -3,     // cuTensorMapEncodeTiled refused the descriptor
  B200_ERR_TOO_BIG = -4,  // size exceeds a compiled-in maximum
};

int set_last_cuda_error(cudaError_t e, const char* where);

#define B200_CUDA_CHECK(expr)                                        \
  do {                                                               \
    cudaError_t _e = (expr);                                         \
    if (_e != cudaSuccess) return b200::set_last_cuda_error(_e, #expr); \
  } while (0)

// Device-visible error word for the current device (pinned, mapped host memory: the host can
// read it without touching the stream). Allocated on first use per device.
unsigned int* device_err_word();

int sm_count();

// 2D bf16/fp16/fp32 tensor map. `inner` is the contiguous dimension. Returns B200_OK or B200_ERR_TMAP.
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                 CUtensorMapSwizzle swizzle);
// 3D variant (dims innermost first).
int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t d0,
                 uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                 uint32_t b2, CUtensorMapSwizzle swizzle);

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

}  // namespace b200
