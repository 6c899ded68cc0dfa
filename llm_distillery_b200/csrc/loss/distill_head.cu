// Fused LM-head + distillation loss against sparse teacher top-K targets, without ever forming fp32 logits.
//
//   pass 1  lmhead_lse_gather : tcgen05 GEMM  z = Hc W^T ; the epilogue keeps, per row and column tile, the running
//           max and sum-exp of z/T over the (cropped) vocabulary and picks out z at the teacher's top-K ids
//           (ids sorted ascending per row: each row walks its list with a cursor, no search per column).
//   rows    distill_rows      : one warp per row combines the partials into lse, forms s_k = z_k/T - lse,
//           t_k = log_softmax(U_k/T) and evaluates forward KL / reverse KL / JSD, and the gradient
//           a_k = dL/ds_k with A = sum_k a_k (every top-K loss has dL/dz_j = (1/T)(a_j[j in top-K] - A softmax_j)).
//   pass 2  lmhead_dlogits    : the same GEMM again; the epilogue writes bf16 dz = (g/T)(-A exp(z/T - lse) + a_k at
//           the teacher ids). dH = dz W and dW += dz^T Hc then run as plain tcgen05 GEMMs (NN and TN layouts).
//
// The custom per-conversation loss of the reference implementation is a function of the same (lse, z_k, U_k):
// it is evaluated in PyTorch on the [rows, K] tensors and enters pass 2 through the same a_k / A interface.
#include "../gemm/gemm_pair.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace head {

using namespace b200::gemm;
constexpr int BN = 256;
constexpr int STAGES = 4;
constexpr float LOG2E = 1.4426950408889634f;

// ------------------------------------------------------------------------------------------- pass 1 epilogue
struct LseParams {
  const int* ids;   // [M, K] teacher ids, ascending per row
  float* zk;        // [M, K] out: z[row, ids[row,k]] / T
  float* pmax;      // [n_tiles, M] out: max_j z_j/T over the tile's columns (log2 domain NOT applied: natural units)
  float* psum;      // [n_tiles, M] out: sum_j exp(z_j/T - pmax)
  int K;
  float inv_T;
  int id_off;       // vocabulary-parallel shard: this GEMM's column j is token id j + id_off (0 when unsharded)
};

struct EpiLse {
  static constexpr bool SPLIT_K = false;
  using Params = LseParams;
  static constexpr int SMEM_BYTES = 0;
  static __device__ __forceinline__ void tile(const Params& p, uint32_t taddr, int m0, int n0, int M, int N, int quad,
                                              int lane, uint8_t*) {
    const int row = m0 + quad * 32 + lane;
    const bool row_ok = row < M;
    const int* ids = p.ids + (long long)row * p.K;
    // cursor: first teacher id >= n0 (binary search once per tile)
    int pos = 0;
    if (row_ok) {
      int lo = 0, hi = p.K;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(ids + mid) - p.id_off < n0) lo = mid + 1; else hi = mid;
      }
      pos = lo;
    }
    int next_id = (row_ok && pos < p.K) ? __ldg(ids + pos) - p.id_off : 0x7fffffff;
    float mx = -INFINITY, sm = 0.f;
    const float c2 = p.inv_T * LOG2E;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      __syncwarp();  // lanes may have diverged in the previous chunk; tcgen05.ld is warp-collective
      tmem_ld_32x32b_x32(taddr + c * 32, r);
      tmem_ld_wait();
      const int col0 = n0 + c * 32;
      if (!row_ok || col0 >= N) continue;
      // gather teacher-id logits that fall into this chunk
      while (next_id < col0 + 32) {
        const int sel = next_id - col0;
        float v = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) v = (sel == j) ? __uint_as_float(r[j]) : v;
        if (next_id < N) p.zk[(long long)row * p.K + pos] = v * p.inv_T;
        ++pos;
        next_id = pos < p.K ? __ldg(ids + pos) - p.id_off : 0x7fffffff;
      }
      // online max / sum-exp (log2 domain internally)
      float cm = -INFINITY;
      const int ncols = min(32, N - col0);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float x = (j < ncols) ? __uint_as_float(r[j]) : -INFINITY;
        cm = fmaxf(cm, x);
      }
      const float nm = fmaxf(mx, cm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float x = (j < ncols) ? __uint_as_float(r[j]) : -INFINITY;
        acc += fast_exp2((x - nm) * c2);
      }
      sm = sm * fast_exp2((mx - nm) * c2) + acc;
      mx = nm;
    }
    if (row_ok) {
      const int nt = n0 / BN;
      p.pmax[(long long)nt * M + row] = mx * p.inv_T;
      p.psum[(long long)nt * M + row] = sm;
    }
  }
};

// ------------------------------------------------------------------------------------------- pass 2 epilogue
struct DzParams {
  const int* ids;      // [M, K] ascending
  const float* a;      // [M, K] dL/ds_k
  const float* A;      // [M]    sum_k a_k
  const float* lse;    // [M]    natural-log lse of z/T
  const float* g;      // [M]    upstream gradient of each row's loss (already includes 1/rows, grad-accum, ...)
  __nv_bfloat16* dz;   // [M, ldz]
  long long ldz;
  int K;
  float inv_T;
  int id_off;          // see LseParams
};

struct EpiDz {
  static constexpr bool SPLIT_K = false;
  using Params = DzParams;
  static constexpr int STAGE_BYTES = 32 * 256;   // per epilogue warp: 32 rows x 128 bf16 columns, chunks XOR-swizzled
  static constexpr int SMEM_BYTES = NUM_EPI_WARPS * STAGE_BYTES;
  static __device__ __forceinline__ void tile(const Params& p, uint32_t taddr, int m0, int n0, int M, int N, int quad,
                                              int lane, uint8_t* epi_smem) {
    // bf16 dlogits leave through a shared-memory stage as whole 256-byte row segments when the layout allows it
    const bool staged = !(N & 7) && !(p.ldz & 7) && !(reinterpret_cast<uintptr_t>(p.dz) & 15);
    uint8_t* stage = epi_smem + quad * STAGE_BYTES;
    const int row0 = m0 + quad * 32;
    const int rows_valid = min(32, M - row0);
    const int row = row0 + lane;
    const bool row_ok = row < M;
    const int* ids = p.ids + (long long)row * p.K;
    int pos = 0;
    float gs = 0.f, coef = 0.f, lse2 = 0.f;
    if (row_ok) {
      int lo = 0, hi = p.K;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(ids + mid) - p.id_off < n0) lo = mid + 1; else hi = mid;
      }
      pos = lo;
      gs = p.g[row] * p.inv_T;
      coef = -gs * p.A[row];
      lse2 = p.lse[row] * LOG2E;
    }
    int next_id = (row_ok && pos < p.K) ? __ldg(ids + pos) - p.id_off : 0x7fffffff;
    const float c2 = p.inv_T * LOG2E;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      __syncwarp();  // lanes may have diverged in the previous chunk; tcgen05.ld is warp-collective
      tmem_ld_32x32b_x32(taddr + c * 32, r);
      tmem_ld_wait();
      const int col0 = n0 + c * 32;
      const bool active = row_ok && col0 < N;
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = coef * fast_exp2(__uint_as_float(r[j]) * c2 - lse2);
      if (active) {
        while (next_id < col0 + 32) {
          const int sel = next_id - col0;
          const float add = gs * __ldg(p.a + (long long)row * p.K + pos);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += (sel == j) ? add : 0.f;
          ++pos;
          next_id = pos < p.K ? __ldg(ids + pos) - p.id_off : 0x7fffffff;
        }
      }
      if (staged) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 o;
          o.x = pack_bf16x2(v[q4 * 8 + 0], v[q4 * 8 + 1]);
          o.y = pack_bf16x2(v[q4 * 8 + 2], v[q4 * 8 + 3]);
          o.z = pack_bf16x2(v[q4 * 8 + 4], v[q4 * 8 + 5]);
          o.w = pack_bf16x2(v[q4 * 8 + 6], v[q4 * 8 + 7]);
          const int chunk = (c & 3) * 4 + q4;
          *reinterpret_cast<uint4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
        }
        if ((c & 3) == 3) {  // 128 columns staged: write them out, two 256-byte row segments per instruction
          __syncwarp();
          const int chunk = lane & 15;
          const int col = n0 + (c >> 2) * 128 + chunk * 8;
#pragma unroll 4
          for (int j = 0; j < 16; ++j) {
            const int rr = 2 * j + (lane >> 4);
            const uint4 o = *reinterpret_cast<const uint4*>(stage + rr * 256 + ((chunk ^ (rr & 15)) << 4));
            if (rr < rows_valid && col < N)
              *reinterpret_cast<uint4*>(p.dz + (long long)(row0 + rr) * p.ldz + col) = o;
          }
          __syncwarp();
        }
        continue;
      }
      if (!active) continue;
      __nv_bfloat16* dst = p.dz + (long long)row * p.ldz + col0;
      const int ncols = min(32, N - col0);
      if (ncols == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 o;
          o.x = pack_bf16x2(v[q4 * 8 + 0], v[q4 * 8 + 1]);
          o.y = pack_bf16x2(v[q4 * 8 + 2], v[q4 * 8 + 3]);
          o.z = pack_bf16x2(v[q4 * 8 + 4], v[q4 * 8 + 5]);
          o.w = pack_bf16x2(v[q4 * 8 + 6], v[q4 * 8 + 7]);
          *reinterpret_cast<uint4*>(dst + q4 * 8) = o;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) dst[j] = __float2bfloat16(v[j]);
      }
    }
  }
};

template <class Epi>
static int launch_head(const void* Hc, const void* W, int M, int N, int Kdim, long long ldh, long long ldw,
                       const typename Epi::Params& ep, cudaStream_t stream) {
  // enough 256 x 256 tiles: run on SM pairs (cta_group::2), else one CTA per 128 x 256 tile
  const bool pair = (long long)ceil_div(M, PAIR_BM) * ceil_div(N, PAIR_BN) >= sm_count() / 2 && Kdim >= 256;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, Hc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)Kdim, (uint64_t)M, (uint64_t)ldh * 2,
                        BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  rc = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)Kdim, (uint64_t)N, (uint64_t)ldw * 2, BK,
                    pair ? PAIR_HALF_N : BN, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  if (pair) {
    constexpr int PSTAGES = 6;
    auto kern = gemm_pair_kernel<PSTAGES, false, false, Epi>;
    const int smem_bytes = SmemPair<PSTAGES>::bytes(Epi::SMEM_BYTES);
    static bool attr = false;
    if (!attr) {
      B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
      attr = true;
    }
    const int tiles = ceil_div(M, PAIR_BM) * ceil_div(N, PAIR_BN);
    const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
    kern<<<2 * pairs, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, M, N, Kdim, 1, ep, device_err_word(), 1, nullptr, 0);
    B200_CUDA_CHECK(cudaGetLastError());
    return B200_OK;
  }
  using S = Smem<BN, STAGES>;
  auto kern = gemm_kernel<BN, STAGES, false, false, Epi>;
  const int smem_bytes = S::bytes(Epi::SMEM_BYTES);
  static bool attr = false;
  if (!attr) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    attr = true;
  }
  const int tiles = ceil_div(M, BM) * ceil_div(N, BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, M, N, Kdim, 1, default_desc_cfg<BN, false, false>(), ep,
                                                  device_err_word());
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// ------------------------------------------------------------------------------------------- row kernel
// kind: 0 forward KL, 1 reverse KL (student renormalised over the support), 2 JSD (student not renormalised),
//       3 JSD with the student renormalised over the support, 4 none (only lse / s_k are produced).
struct RowParams {
  const float* pmax; const float* psum;  // [n_tiles, M]
  const float* zk;                       // [M, K]
  const float* u;                        // [M, K] stored teacher log-probs (T = 1)
  const int* ids;                        // [M, K] (entries >= vocab are treated as absent)
  float* lse;                            // [M] out
  float* loss;                           // [M] out
  float* a;                              // [M, K] out
  float* A;                              // [M] out
  int M, K, n_tiles, vocab, kind;
  float inv_T;
};

__global__ void __launch_bounds__(128) distill_rows_kernel(RowParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= p.M) return;
  const int row = warp;
  // combine column-tile partials into the full-vocabulary lse
  float mx = -INFINITY;
  for (int t = lane; t < p.n_tiles; t += 32) mx = fmaxf(mx, p.pmax[(long long)t * p.M + row]);
  mx = warp_max(mx);
  float sm = 0.f;
  for (int t = lane; t < p.n_tiles; t += 32)
    sm += p.psum[(long long)t * p.M + row] * __expf(p.pmax[(long long)t * p.M + row] - mx);
  sm = warp_sum(sm);
  const float lse = mx + __logf(sm);
  if (lane == 0) p.lse[row] = lse;
  if (p.kind == 4) return;
  const float* zk = p.zk + (long long)row * p.K;
  const float* u = p.u + (long long)row * p.K;
  const int* ids = p.ids + (long long)row * p.K;
  // teacher log-softmax over the support at temperature T
  // an entry takes part when its id is inside the cropped vocabulary and the teacher gave it a finite log-prob
#define B200_ENTRY_OK(k) (ids[k] < p.vocab && u[k] > -1e30f)
  float umax = -INFINITY, zmax = -INFINITY;
  for (int k = lane; k < p.K; k += 32) {
    const bool ok = B200_ENTRY_OK(k);
    if (ok) {
      umax = fmaxf(umax, u[k] * p.inv_T);
      zmax = fmaxf(zmax, zk[k]);
    }
  }
  umax = warp_max(umax);
  zmax = warp_max(zmax);
  float us = 0.f, zs = 0.f;
  for (int k = lane; k < p.K; k += 32) {
    if (B200_ENTRY_OK(k)) {
      us += __expf(u[k] * p.inv_T - umax);
      zs += __expf(zk[k] - zmax);
    }
  }
  us = warp_sum(us);
  zs = warp_sum(zs);
  if (!(us > 0.f)) {  // no teacher target on this row (e.g. no shared token boundary): zero loss, zero gradient
    for (int k = lane; k < p.K; k += 32) p.a[(long long)row * p.K + k] = 0.f;
    if (lane == 0) { p.loss[row] = 0.f; p.A[row] = 0.f; }
    return;
  }
  const float ulse = umax + __logf(us);  // teacher normaliser over the support
  const float zlse = zmax + __logf(zs);  // student normaliser over the support
  float loss = 0.f;
  // first sweep: the loss itself (reverse KL and renormalised JSD need it before the gradient)
  for (int k = lane; k < p.K; k += 32) {
    if (!B200_ENTRY_OK(k)) continue;
    const float t = u[k] * p.inv_T - ulse;
    const float pt = __expf(t);
    if (p.kind == 0) {
      loss += pt * (t - (zk[k] - lse));
    } else if (p.kind == 1) {
      const float s1 = zk[k] - zlse;
      loss += __expf(s1) * (s1 - t);
    } else {
      const float s = (p.kind == 2) ? zk[k] - lse : zk[k] - zlse;
      const float q = __expf(s);
      const float lm = __logf(0.5f * (pt + q));
      loss += 0.5f * (pt * (t - lm) + q * (s - lm));
    }
  }
  loss = warp_sum(loss);
  // second sweep: a_k = dL/ds_k (for the renormalised variants chained through the support log-softmax)
  float asum = 0.f, inner = 0.f;
  if (p.kind == 3) {
    for (int k = lane; k < p.K; k += 32) {
      if (!B200_ENTRY_OK(k)) continue;
      const float t = u[k] * p.inv_T - ulse;
      const float s1 = zk[k] - zlse;
      const float q = __expf(s1);
      inner += 0.5f * q * (s1 - __logf(0.5f * (__expf(t) + q)));
    }
    inner = warp_sum(inner);
  }
  for (int k = lane; k < p.K; k += 32) {
    float ak = 0.f;
    if (B200_ENTRY_OK(k)) {
      const float t = u[k] * p.inv_T - ulse;
      const float pt = __expf(t);
      if (p.kind == 0) {
        ak = -pt;
      } else if (p.kind == 1) {
        const float s1 = zk[k] - zlse;
        ak = __expf(s1) * ((s1 - t) - loss);
      } else if (p.kind == 2) {
        const float s = zk[k] - lse;
        const float q = __expf(s);
        ak = 0.5f * q * (s - __logf(0.5f * (pt + q)));
      } else {
        const float s1 = zk[k] - zlse;
        const float q = __expf(s1);
        ak = 0.5f * q * (s1 - __logf(0.5f * (pt + q))) - q * inner;
      }
    }
    p.a[(long long)row * p.K + k] = ak;
    asum += ak;
  }
  asum = warp_sum(asum);
  if (lane == 0) {
    p.loss[row] = loss;
    p.A[row] = asum;
  }
}


// Vocabulary-parallel head: every rank ran pass 1 on its slice of the vocabulary. One warp per row reads ALL ranks'
// partial statistics straight out of their memory (peer loads over NVLink) and leaves, locally, one combined
// (max, sum-exp) pair per row and the summed z_k (an id lives in exactly one slice; the other ranks hold zeros),
// which distill_rows_kernel then consumes as a single column tile.
struct VpPeers { const void* p[16]; };
__global__ void __launch_bounds__(128) vp_combine_kernel(VpPeers pmax, VpPeers psum, VpPeers zk, int world,
                                                        int n_tiles, int M, int K, float* __restrict__ out_pmax,
                                                        float* __restrict__ out_psum, float* __restrict__ out_zk) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const int n = world * n_tiles;
  float mx = -INFINITY;
  for (int i = lane; i < n; i += 32) {
    const int q = i / n_tiles, t = i - q * n_tiles;
    mx = fmaxf(mx, reinterpret_cast<const float*>(pmax.p[q])[(long long)t * M + row]);
  }
  mx = warp_max(mx);
  float sm = 0.f;
  for (int i = lane; i < n; i += 32) {
    const int q = i / n_tiles, t = i - q * n_tiles;
    const long long o = (long long)t * M + row;
    sm += reinterpret_cast<const float*>(psum.p[q])[o] * __expf(reinterpret_cast<const float*>(pmax.p[q])[o] - mx);
  }
  sm = warp_sum(sm);
  if (lane == 0) {
    out_pmax[row] = mx;
    out_psum[row] = sm;
  }
  for (int k = lane; k < K; k += 32) {
    float z = 0.f;
    for (int q = 0; q < world; ++q) z += reinterpret_cast<const float*>(zk.p[q])[(long long)row * K + k];
    out_zk[(long long)row * K + k] = z;
  }
}

}  // namespace head
}  // namespace b200

extern "C" {
using namespace b200;
using namespace b200::head;

// Column tiles the partial buffers need: pmax/psum are [b200_head_num_tiles(N), M] floats.
int b200_head_num_tiles(int N) { return ceil_div(N, BN); }

// Pass 1. Hc [M, h] bf16 (row stride ldh), W [N, h] bf16 (row stride ldw; pass the cropped vocabulary size as N).
// ids must be ascending per row; entries >= N are ignored (their zk is left untouched).
int b200_lmhead_lse_gather(const void* Hc, const void* W, int M, int N, int h, long long ldh, long long ldw,
                           const int* ids, int K, float inv_T, float* zk, float* pmax, float* psum,
                           cudaStream_t st) {
  if (!Hc || !W || !ids || !zk || !pmax || !psum || M <= 0 || N <= 0 || h <= 0 || K <= 0 || (ldh & 7) || (ldw & 7))
    return B200_ERR_ARG;
  LseParams ep{ids, zk, pmax, psum, K, inv_T, 0};
  return launch_head<EpiLse>(Hc, W, M, N, h, ldh, ldw, ep, st);
}

// Pass 1 on one vocabulary slice: W holds the rows [id_off, id_off + N) of the LM head; ids stay global.
int b200_lmhead_lse_gather_shard(const void* Hc, const void* W, int M, int N, int h, long long ldh, long long ldw,
                                 const int* ids, int K, float inv_T, int id_off, float* zk, float* pmax, float* psum,
                                 cudaStream_t st) {
  if (!Hc || !W || !ids || !zk || !pmax || !psum || M <= 0 || N <= 0 || h <= 0 || K <= 0 || (ldh & 7) || (ldw & 7))
    return B200_ERR_ARG;
  LseParams ep{ids, zk, pmax, psum, K, inv_T, id_off};
  return launch_head<EpiLse>(Hc, W, M, N, h, ldh, ldw, ep, st);
}

// Combine the slices' statistics (arrays of `world` device pointers, peers' memory included) into one local tile.
int b200_vp_combine(const void* const* pmax_ptrs, const void* const* psum_ptrs, const void* const* zk_ptrs, int world,
                    int n_tiles, int M, int K, float* out_pmax, float* out_psum, float* out_zk, cudaStream_t st) {
  if (!pmax_ptrs || !psum_ptrs || !zk_ptrs || world < 1 || world > 16 || n_tiles <= 0 || M <= 0 || K <= 0 ||
      !out_pmax || !out_psum || !out_zk)
    return B200_ERR_ARG;
  VpPeers a{}, b{}, c{};
  for (int i = 0; i < world; ++i) {
    a.p[i] = pmax_ptrs[i];
    b.p[i] = psum_ptrs[i];
    c.p[i] = zk_ptrs[i];
  }
  vp_combine_kernel<<<ceil_div(M, 4), 128, 0, st>>>(a, b, c, world, n_tiles, M, K, out_pmax, out_psum, out_zk);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_distill_rows(const float* pmax, const float* psum, const float* zk, const float* u, const int* ids,
                      float* lse, float* loss, float* a, float* A, int M, int K, int n_tiles, int vocab, int kind,
                      float inv_T, cudaStream_t st) {
  if (!pmax || !psum || !lse || M <= 0 || n_tiles <= 0 || kind < 0 || kind > 4) return B200_ERR_ARG;
  if (kind != 4 && (!zk || !u || !ids || !loss || !a || !A || K <= 0)) return B200_ERR_ARG;
  RowParams p{pmax, psum, zk, u, ids, lse, loss, a, A, M, K, n_tiles, vocab, kind, inv_T};
  const int warps_per_block = 4;
  distill_rows_kernel<<<ceil_div(M, warps_per_block), warps_per_block * 32, 0, st>>>(p);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// Pass 2: dz[M, N] (bf16, row stride ldz) = (g/T) * (-A * exp(z/T - lse) + a_k at ids).
int b200_lmhead_dlogits(const void* Hc, const void* W, int M, int N, int h, long long ldh, long long ldw,
                        const int* ids, const float* a, const float* A, const float* lse, const float* g, int K,
                        float inv_T, void* dz, long long ldz, cudaStream_t st) {
  if (!Hc || !W || !ids || !a || !A || !lse || !g || !dz || M <= 0 || N <= 0 || h <= 0 || K <= 0 || (ldh & 7) ||
      (ldw & 7))
    return B200_ERR_ARG;
  DzParams ep{ids, a, A, lse, g, (__nv_bfloat16*)dz, ldz, K, inv_T, 0};
  return launch_head<EpiDz>(Hc, W, M, N, h, ldh, ldw, ep, st);
}

// Pass 2 on one vocabulary slice (see b200_lmhead_lse_gather_shard).
int b200_lmhead_dlogits_shard(const void* Hc, const void* W, int M, int N, int h, long long ldh, long long ldw,
                              const int* ids, const float* a, const float* A, const float* lse, const float* g, int K,
                              float inv_T, int id_off, void* dz, long long ldz, cudaStream_t st) {
  if (!Hc || !W || !ids || !a || !A || !lse || !g || !dz || M <= 0 || N <= 0 || h <= 0 || K <= 0 || (ldh & 7) ||
      (ldw & 7))
    return B200_ERR_ARG;
  DzParams ep{ids, a, A, lse, g, (__nv_bfloat16*)dz, ldz, K, inv_T, id_off};
  return launch_head<EpiDz>(Hc, W, M, N, h, ldh, ldw, ep, st);
}
}
