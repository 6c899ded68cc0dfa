// Per-conversation reductions over the rows of a micro-batch, in a fixed order.
//
// A micro-batch lists the content rows of its conversations one conversation after the other, so the conversation
// index `seg[r]` is non-decreasing in r. One warp owns one conversation: it finds the conversation's row range by
// binary search, the lanes walk it with stride 32 and the lane partials meet in a butterfly. The order of the
// additions depends on the row range only, never on scheduling, so the result is bit-identical from run to run
// (an atomic scatter-add is not). The reference adds its per-conversation losses in a Python loop
// (classes/student/model.py:415-436, classes/losses.py:43-47), which is a fixed order too.
#include "../common/ptx.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace seg {

__device__ __forceinline__ long long lower_bound(const long long* __restrict__ seg, long long M, long long key) {
  long long lo = 0, hi = M;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if (seg[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// op 0: sum, op 1: max (-inf for an empty conversation), op 2: number of rows
__global__ void __launch_bounds__(256) segment_reduce_kernel(const float* __restrict__ x,
                                                             const long long* __restrict__ seg,
                                                             float* __restrict__ out, long long M, int n_seg, int op) {
  const int warp = (int)((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (warp >= n_seg) return;
  const long long r0 = lower_bound(seg, M, warp), r1 = lower_bound(seg, M, (long long)warp + 1);
  if (op == 2) {
    if (lane == 0) out[warp] = (float)(r1 - r0);
    return;
  }
  float acc = op == 1 ? -INFINITY : 0.f;
  for (long long r = r0 + lane; r < r1; r += 32) {
    const float v = x[r];
    acc = op == 1 ? fmaxf(acc, v) : acc + v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, acc, o);
    acc = op == 1 ? fmaxf(acc, other) : acc + other;
  }
  if (lane == 0) out[warp] = acc;
}

}  // namespace seg
}  // namespace b200

extern "C" int b200_segment_reduce(const float* x, const long long* seg, float* out, long long M, int n_seg, int op,
                                   cudaStream_t st) {
  using namespace b200;
  if (!seg || !out || M < 0 || n_seg <= 0 || op < 0 || op > 2 || (op != 2 && !x)) return B200_ERR_ARG;
  const int blocks = ceil_div(n_seg * 32, 256);
  seg::segment_reduce_kernel<<<blocks, 256, 0, st>>>(x, seg, out, M, n_seg, op);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
