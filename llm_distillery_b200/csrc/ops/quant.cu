// Dequantisation of frozen low-bit weights into bf16, layer by layer, just before the layer's GEMMs read them.
//
// The reference's `training_precision` "4bit" and "8bit" load the student's linear layers through bitsandbytes as
// NF4 (block-wise absmax over 64 values, the absmax values themselves quantised a second time) or row-wise int8
// weights, which are then FROZEN: only embeddings, norms and the LM head keep training (classes/student/model.py:
// 138-148, 194-201). Here the packed weights stay resident and a layer's matrices are expanded into a rotating bf16
// buffer by these kernels before its forward and again before its backward; the tensor-core GEMMs then run on bf16
// as everywhere else.
//
//   NF4   byte = (code of element 2i) << 4 | code of element 2i+1; value = nf4[code] * absmax(block of 64)
//         absmax(block) = int8 code * scale(group of 256 blocks) + offset      (second-level quantisation)
//   int8  value = code * scale(row)
#include "../common/ptx.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace quant {

__constant__ float kNF4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                               -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                               0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                               0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

// 16 values (8 packed bytes) per thread; n is a multiple of 64, so a thread never straddles a block.
__global__ void __launch_bounds__(256) dequant_nf4_kernel(const uint8_t* __restrict__ packed,
                                                          const int8_t* __restrict__ absmax_code,
                                                          const float* __restrict__ absmax_scale, float offset,
                                                          __nv_bfloat16* __restrict__ out, long long n) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = kNF4[threadIdx.x];
  __syncthreads();
  const long long groups = n >> 4;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    const long long blk = g >> 2;  // 64-value block
    const float am = (float)absmax_code[blk] * absmax_scale[blk >> 8] + offset;
    const uint2 q = reinterpret_cast<const uint2*>(packed)[g];
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = ((i < 4 ? q.x : q.y) >> (8 * (i & 3))) & 0xffu;
      w[i] = pack_bf16x2(lut[byte >> 4] * am, lut[byte & 15u] * am);
    }
    uint4* o = reinterpret_cast<uint4*>(out + (g << 4));
    o[0] = make_uint4(w[0], w[1], w[2], w[3]);
    o[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// 16 values per thread; cols is a multiple of 16.
__global__ void __launch_bounds__(256) dequant_int8_kernel(const int8_t* __restrict__ code,
                                                           const float* __restrict__ row_scale,
                                                           __nv_bfloat16* __restrict__ out, long long rows, int cols) {
  const int gpr = cols >> 4;
  const long long groups = rows * gpr;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    const float sc = row_scale[g / gpr];
    const uint4 q = reinterpret_cast<const uint4*>(code)[g];
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t two = words[i >> 1] >> (16 * (i & 1));
      w[i] = pack_bf16x2((float)(int8_t)(two & 0xffu) * sc, (float)(int8_t)((two >> 8) & 0xffu) * sc);
    }
    uint4* o = reinterpret_cast<uint4*>(out + (g << 4));
    o[0] = make_uint4(w[0], w[1], w[2], w[3]);
    o[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

static int grid_for(long long items) {
  long long b = (items + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

}  // namespace quant
}  // namespace b200

extern "C" {
using namespace b200;

int b200_dequant_nf4(const void* packed, const void* absmax_code, const float* absmax_scale, float offset, void* out,
                     long long n, cudaStream_t st) {
  if (!packed || !absmax_code || !absmax_scale || !out || n <= 0 || (n & 63)) return B200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) return B200_ERR_ARG;
  quant::dequant_nf4_kernel<<<quant::grid_for(n >> 4), 256, 0, st>>>((const uint8_t*)packed, (const int8_t*)absmax_code,
                                                                    absmax_scale, offset, (__nv_bfloat16*)out, n);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_dequant_int8(const void* code, const float* row_scale, void* out, long long rows, int cols, cudaStream_t st) {
  if (!code || !row_scale || !out || rows <= 0 || cols <= 0 || (cols & 15)) return B200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(code) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return B200_ERR_ARG;
  quant::dequant_int8_kernel<<<quant::grid_for(rows * (cols >> 4)), 256, 0, st>>>((const int8_t*)code, row_scale,
                                                                                 (__nv_bfloat16*)out, rows, cols);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
}
