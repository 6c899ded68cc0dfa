#include "host.cuh"

#include <mutex>
#include <string.h>

namespace b200 {

static char g_last_err[512] = {0};
static std::mutex g_mu;

int set_last_cuda_error(cudaError_t e, const char* where) {
  std::lock_guard<std::mutex> lk(g_mu);
  snprintf(g_last_err, sizeof(g_last_err), "%s: %s (%d)", where, cudaGetErrorString(e), (int)e);
  return B200_ERR_CUDA;
}

static unsigned int* g_err_words[64] = {nullptr};
static unsigned int* g_err_words_host[64] = {nullptr};

unsigned int* device_err_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_err_words[dev]) {
    unsigned int* h = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped) != cudaSuccess) return nullptr;
    memset(h, 0, 64);
    unsigned int* d = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0) != cudaSuccess) return nullptr;
    g_err_words_host[dev] = h;
    g_err_words[dev] = d;
  }
  return g_err_words[dev];
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t inner,
                 uint64_t outer, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                 CUtensorMapSwizzle swizzle) {
  auto enc = get_encode();
  if (!enc) return B200_ERR_TMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (outer_stride_bytes & 15)) return B200_ERR_ARG;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {outer_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  (void)elem_bytes;
  CUresult r = enc(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::lock_guard<std::mutex> lk(g_mu);
    snprintf(g_last_err, sizeof(g_last_err), "cuTensorMapEncodeTiled(2d) failed: CUresult %d", (int)r);
    return B200_ERR_TMAP;
  }
  return B200_OK;
}

int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t d0,
                 uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                 uint32_t b2, CUtensorMapSwizzle swizzle) {
  auto enc = get_encode();
  if (!enc) return B200_ERR_TMAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (stride1_bytes & 15) || (stride2_bytes & 15)) return B200_ERR_ARG;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  (void)elem_bytes;
  CUresult r = enc(out, dtype, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::lock_guard<std::mutex> lk(g_mu);
    snprintf(g_last_err, sizeof(g_last_err), "cuTensorMapEncodeTiled(3d) failed: CUresult %d", (int)r);
    return B200_ERR_TMAP;
  }
  return B200_OK;
}

}  // namespace b200

extern "C" {

// Last CUDA / driver error string recorded by a launcher of this library (empty if none).
const char* b200_last_cuda_error() { return b200::g_last_err; }

// Reads and clears the device error word of the current device. Non-zero means an in-kernel
// bounded wait gave up (codes in common/ptx.cuh). The caller should synchronize the stream first.
unsigned int b200_take_device_error() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!b200::g_err_words_host[dev]) return 0;
  unsigned int v = *reinterpret_cast<volatile unsigned int*>(b200::g_err_words_host[dev]);
  *reinterpret_cast<volatile unsigned int*>(b200::g_err_words_host[dev]) = 0;
  return v;
}

int b200_sm_count() { return b200::sm_count(); }
}
