// Plain GEMM entry points on the tcgen05 mainloop (gemm_core.cuh):
//   C[M,N] = alpha * A * B^T (+ C) (+ residual)     bf16/fp16 operands, fp32 accumulate,
// with A and B each either K-major or MN-major, so forward (NT), dgrad (NN) and wgrad (TN)
// GEMMs of a linear layer all run without a transpose pass.
#include "gemm_pair.cuh"
#include <stdlib.h>
#include <atomic>
#include "../common/host.cuh"

namespace b200 {
namespace gemm {

struct StoreParams {
  void* C;
  long long ldc;               // elements
  const __nv_bfloat16* resid;  // optional residual added to the result (bf16, same shape as C), may be null
  long long ldr;
  float alpha;
  int out_f32;     // 1: C is fp32, 0: C is 16-bit (bf16 or fp16 according to fmt)
  int accumulate;  // 1: C += result
  int fmt;         // 0 fp16, 1 bf16 (16-bit output type)
};

template <int BN>
struct EpiStore {
  using Params = StoreParams;
  static constexpr bool SPLIT_K = true;   // the pair kernel may cut the K loop into slices that are added in order
  // slice 0 of a tile stores (or adds to what C held, if the caller accumulates); every later slice adds
  static __device__ __forceinline__ Params slice_params(const Params& p, int slice) {
    Params q = p;
    if (slice > 0) q.accumulate = 1;
    return q;
  }
  static constexpr int STAGE_BYTES = 32 * 256;              // per epilogue warp: 32 rows x 128 bf16 columns
  static constexpr int SMEM_BYTES = NUM_EPI_WARPS * STAGE_BYTES;

  // bf16 output without accumulation (forward and dgrad GEMMs): the warp's 32 x 128 slice goes through a swizzled
  // shared-memory stage so that each store instruction writes two whole 256-byte row segments instead of 32
  // scattered 16-byte pieces. alpha and the residual are applied in fp32 before the rounding to bf16.
  static __device__ __forceinline__ void tile_staged(const Params& p, uint32_t taddr, int m0, int n0, int M, int N,
                                                     int quad, int lane, uint8_t* epi_smem) {
    uint8_t* stage = epi_smem + quad * STAGE_BYTES;
    const int row0 = m0 + quad * 32;
    const int rows_valid = min(32, M - row0);
    const bool my_row_ok = lane < rows_valid;
    __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C);
#pragma unroll 1
    for (int half = 0; half < BN / 128; ++half) {
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + half * 128 + c4 * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + half * 128 + c4 * 32;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        if (p.resid && my_row_ok && col0 < N) {
          const __nv_bfloat16* rp = p.resid + (long long)(row0 + lane) * p.ldr + col0;
          if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 q = *reinterpret_cast<const uint4*>(rp + j * 8);
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                const float2 f = __bfloat1622float2(h[t]);
                v[j * 8 + t * 2] += f.x;
                v[j * 8 + t * 2 + 1] += f.y;
              }
            }
          } else {
            const int ncols = min(32, N - col0);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ncols) v[j] += __bfloat162float(rp[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 o;
          o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
          o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
          o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
          o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
          const int chunk = c4 * 4 + j;
          *reinterpret_cast<uint4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
        }
      }
      __syncwarp();
      const int chunk = lane & 15;
      const int col = n0 + half * 128 + chunk * 8;
#pragma unroll 4
      for (int j = 0; j < 16; ++j) {
        const int row = 2 * j + (lane >> 4);
        const uint4 o = *reinterpret_cast<const uint4*>(stage + row * 256 + ((chunk ^ (row & 15)) << 4));
        if (row < rows_valid && col < N) *reinterpret_cast<uint4*>(C + (long long)(row0 + row) * p.ldc + col) = o;
      }
      __syncwarp();
    }
  }

  // fp32 output (weight gradients, with or without accumulation): 64 columns of the warp's 32 rows at a time go
  // through the same swizzled stage, so that one instruction reads-modifies-writes 256 contiguous bytes of two rows
  // (whole sectors) instead of 16 bytes of 32 different rows.
  static __device__ __forceinline__ void tile_staged_f32(const Params& p, uint32_t taddr, int m0, int n0, int M, int N,
                                                         int quad, int lane, uint8_t* epi_smem) {
    uint8_t* stage = epi_smem + quad * STAGE_BYTES;
    const int row0 = m0 + quad * 32;
    const int rows_valid = min(32, M - row0);
    float* C = reinterpret_cast<float*>(p.C);
#pragma unroll 1
    for (int g = 0; g < BN / 64; ++g) {
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + g * 64 + c2 * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 o = make_float4(__uint_as_float(r[4 * j]) * p.alpha, __uint_as_float(r[4 * j + 1]) * p.alpha,
                                       __uint_as_float(r[4 * j + 2]) * p.alpha, __uint_as_float(r[4 * j + 3]) * p.alpha);
          const int chunk = c2 * 8 + j;
          *reinterpret_cast<float4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
        }
      }
      __syncwarp();
      const int chunk = lane & 15;
      const int col = n0 + g * 64 + chunk * 4;
#pragma unroll 4
      for (int j = 0; j < 16; ++j) {
        const int row = 2 * j + (lane >> 4);
        float4 o = *reinterpret_cast<const float4*>(stage + row * 256 + ((chunk ^ (row & 15)) << 4));
        if (row < rows_valid && col < N) {
          float* cp = C + (long long)(row0 + row) * p.ldc + col;
          if (p.accumulate) {
            // a reduction, not a load + add + store: the L2 round trip of the load made short K slices epilogue-bound.
            // The order of the additions into one element is still fixed: the slices of a tile take turns (the
            // counter protocol of the pair kernel, with a fence before each hand-over) and nothing else adds to C.
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(cp), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w)
                         : "memory");
          } else {
            *reinterpret_cast<float4*>(cp) = o;
          }
        }
      }
      __syncwarp();
    }
  }

  static __device__ __forceinline__ void tile(const Params& p, uint32_t taddr, int m0, int n0, int M, int N, int quad,
                                              int lane, uint8_t* epi_smem) {
    if (!p.out_f32 && p.fmt == 1 && !p.accumulate && !(N & 7) && !(p.ldc & 7) &&
        !(reinterpret_cast<uintptr_t>(p.C) & 15)) {
      tile_staged(p, taddr, m0, n0, M, N, quad, lane, epi_smem);
      return;
    }
    if (p.out_f32 && !p.resid && !(N & 3) && !(p.ldc & 3) && !(reinterpret_cast<uintptr_t>(p.C) & 15)) {
      tile_staged_f32(p, taddr, m0, n0, M, N, quad, lane, epi_smem);
      return;
    }
    const int row = m0 + quad * 32 + lane;
    const bool row_ok = row < M;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      __syncwarp();  // lanes may have diverged in the previous chunk; tcgen05.ld is warp-collective
      tmem_ld_32x32b_x32(taddr + c * 32, r);
      tmem_ld_wait();
      const int col0 = n0 + c * 32;
      if (!row_ok || col0 >= N) continue;
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
      const int ncols = min(32, N - col0);
      if (p.resid) {
        const __nv_bfloat16* rp = p.resid + (long long)row * p.ldr + col0;
        if (ncols == 32 && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 q = *reinterpret_cast<const uint4*>(rp + j * 8);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              float2 f = __bfloat1622float2(h[t]);
              v[j * 8 + t * 2] += f.x;
              v[j * 8 + t * 2 + 1] += f.y;
            }
          }
        } else {
          for (int j = 0; j < ncols; ++j) v[j] += __bfloat162float(rp[j]);
        }
      }
      if (p.out_f32) {
        float* cp = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
        if (ncols == 32 && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0)) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
            if (p.accumulate) {
              float4 old = *reinterpret_cast<float4*>(cp + j * 4);
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            *reinterpret_cast<float4*>(cp + j * 4) = o;
          }
        } else {
          for (int j = 0; j < ncols; ++j) cp[j] = p.accumulate ? cp[j] + v[j] : v[j];
        }
      } else if (p.fmt == 1) {
        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
        if (ncols == 32 && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0)) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (p.accumulate) {
              uint4 q = *reinterpret_cast<const uint4*>(cp + j * 8);
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                float2 f = __bfloat1622float2(h[t]);
                v[j * 8 + t * 2] += f.x;
                v[j * 8 + t * 2 + 1] += f.y;
              }
            }
            uint4 o;
            o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
            o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
            o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
            o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
            *reinterpret_cast<uint4*>(cp + j * 8) = o;
          }
        } else {
          for (int j = 0; j < ncols; ++j) {
            float x = v[j] + (p.accumulate ? __bfloat162float(cp[j]) : 0.f);
            cp[j] = __float2bfloat16(x);
          }
        }
      } else {
        __half* cp = reinterpret_cast<__half*>(p.C) + (long long)row * p.ldc + col0;
        for (int j = 0; j < ncols; ++j) {
          float x = v[j] + (p.accumulate ? __half2float(cp[j]) : 0.f);
          cp[j] = __float2half(x);
        }
      }
    }
  }
};

// Fused gate / up projection + SwiGLU on the CTA-pair kernel. The accumulator of a tile holds, for 256 rows, the gate
// (columns 0-127) and the up projection (columns 128-255) of the same 128 features (the B halves come from rows
// j*128 and f + j*128 of the fused weight, gemm_pair.cuh). The epilogue writes three things per row: gate and up,
// rounded to bf16, into gu [M, 2f] (the backward pass reads them), and act = silu(gate) * up computed from the ROUNDED
// values, so that it equals what the stand-alone SwiGLU kernel makes of gu bit for bit. Each leaves through the
// swizzled stage as 256-byte row segments.
struct SwigluParams {
  __nv_bfloat16* gu;    // [M, 2f]
  long long ld_gu;
  __nv_bfloat16* act;   // [M, f]
  long long ld_act;
  int f;
};

struct EpiSwiglu {
  using Params = SwigluParams;
  static constexpr bool SPLIT_K = false;
  static constexpr int STAGE_BYTES = 32 * 256;
  static constexpr int SMEM_BYTES = NUM_EPI_WARPS * STAGE_BYTES;

  static __device__ __forceinline__ void flush(uint8_t* stage, __nv_bfloat16* dst, long long ld, int row0, int rows_valid,
                                               int col0, int f, int lane) {
    __syncwarp();
    const int chunk = lane & 15;
    const int col = col0 + chunk * 8;
#pragma unroll 4
    for (int j = 0; j < 16; ++j) {
      const int row = 2 * j + (lane >> 4);
      const uint4 o = *reinterpret_cast<const uint4*>(stage + row * 256 + ((chunk ^ (row & 15)) << 4));
      if (row < rows_valid && col < f) *reinterpret_cast<uint4*>(dst + (long long)(row0 + row) * ld + col) = o;
    }
    __syncwarp();
  }

  static __device__ __forceinline__ void tile(const Params& p, uint32_t taddr, int m0, int n0, int M, int N, int quad,
                                              int lane, uint8_t* epi_smem) {
    uint8_t* stage = epi_smem + quad * STAGE_BYTES;
    const int row0 = m0 + quad * 32;
    const int rows_valid = min(32, M - row0);
    const int col0 = (n0 / PAIR_BN) * PAIR_HALF_N;       // first of the tile's 128 features
    // gate, then up: rounded copies into gu
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + half * 128 + c4 * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[j * 8 + 0]), __uint_as_float(r[j * 8 + 1]));
          o.y = pack_bf16x2(__uint_as_float(r[j * 8 + 2]), __uint_as_float(r[j * 8 + 3]));
          o.z = pack_bf16x2(__uint_as_float(r[j * 8 + 4]), __uint_as_float(r[j * 8 + 5]));
          o.w = pack_bf16x2(__uint_as_float(r[j * 8 + 6]), __uint_as_float(r[j * 8 + 7]));
          const int chunk = c4 * 4 + j;
          *reinterpret_cast<uint4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
        }
      }
      flush(stage, p.gu + (half ? p.f : 0), p.ld_gu, row0, rows_valid, col0, p.f, lane);
    }
    // act = silu(gate) * up from the rounded values
#pragma unroll 1
    for (int c4 = 0; c4 < 4; ++c4) {
      uint32_t g[32], u[32];
      tmem_ld_32x32b_x32(taddr + c4 * 32, g);
      tmem_ld_32x32b_x32(taddr + 128 + c4 * 32, u);
      tmem_ld_wait();
      float a[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float gj = __bfloat162float(__float2bfloat16(__uint_as_float(g[j])));
        const float uj = __bfloat162float(__float2bfloat16(__uint_as_float(u[j])));
        a[j] = __fdividef(gj, 1.f + __expf(-gj)) * uj;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 o;
        o.x = pack_bf16x2(a[j * 8 + 0], a[j * 8 + 1]);
        o.y = pack_bf16x2(a[j * 8 + 2], a[j * 8 + 3]);
        o.z = pack_bf16x2(a[j * 8 + 4], a[j * 8 + 5]);
        o.w = pack_bf16x2(a[j * 8 + 6], a[j * 8 + 7]);
        const int chunk = c4 * 4 + j;
        *reinterpret_cast<uint4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
      }
    }
    flush(stage, p.act, p.ld_act, row0, rows_valid, col0, p.f, lane);
  }
};

// Rotary embedding in the epilogue of the fused q/k/v projection. A head of d = 64 is two 32-column chunks of the
// accumulator, a head of d = 128 four; the rotation pairs column i with i + d/2, i.e. chunk c with chunk c + 1 (d = 64)
// or c + 2 (d = 128) of the same 128-column half. Each lane owns one row, fetches the cos / sin entries of that row's
// position, rounds the two chunks to bf16 first (what the stand-alone kernel reads back from memory) and rotates with
// the same expressions, so the result is bit-identical to GEMM + rope kernel. Columns from n_rot on (the value heads)
// are stored unrotated.
struct RopeParams {
  __nv_bfloat16* C;     // [M, N]
  long long ldc;
  const int* pos;       // [M]
  const float* cs;      // [max_pos, d/2]
  const float* sn;
  int d;                // 64 or 128
  int n_rot;            // first n_rot columns are rotated ((H + Hkv) * d)
};

struct EpiRope {
  using Params = RopeParams;
  static constexpr bool SPLIT_K = false;
  static constexpr int STAGE_BYTES = 32 * 256;
  static constexpr int SMEM_BYTES = NUM_EPI_WARPS * STAGE_BYTES;

  static __device__ __forceinline__ void put(uint8_t* stage, int lane, int c4, const float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 o;
      o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
      o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
      o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
      o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
      const int chunk = c4 * 4 + j;
      *reinterpret_cast<uint4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
    }
  }

  static __device__ __forceinline__ void tile(const Params& p, uint32_t taddr, int m0, int n0, int M, int N, int quad,
                                              int lane, uint8_t* epi_smem) {
    uint8_t* stage = epi_smem + quad * STAGE_BYTES;
    const int row0 = m0 + quad * 32;
    const int rows_valid = min(32, M - row0);
    const int half_d = p.d >> 1;
    const long long tpos = lane < rows_valid ? (long long)p.pos[row0 + lane] : 0;
    const int step = p.d == 64 ? 1 : 2;                   // distance, in chunks, between the two halves of a pair
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      const int colh = n0 + half * 128;
      if (colh >= N) break;                               // N is a multiple of 128
#pragma unroll 1
      for (int k = 0; k < 2; ++k) {
        // d = 64: pair (0,1) then (2,3); d = 128: pair (0,2) then (1,3)
        const int ca = p.d == 64 ? 2 * k : k;
        const int cb = ca + step;
        uint32_t ra[32], rb[32];
        tmem_ld_32x32b_x32(taddr + half * 128 + ca * 32, ra);
        tmem_ld_32x32b_x32(taddr + half * 128 + cb * 32, rb);
        tmem_ld_wait();
        float a[32], b[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          a[j] = __bfloat162float(__float2bfloat16(__uint_as_float(ra[j])));
          b[j] = __bfloat162float(__float2bfloat16(__uint_as_float(rb[j])));
        }
        if (colh + ca * 32 < p.n_rot) {
          const int j0 = p.d == 64 ? 0 : k * 32;          // first cos / sin entry of chunk ca
          const float* cp = p.cs + tpos * half_d + j0;
          const float* sp = p.sn + tpos * half_d + j0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 c4v = *reinterpret_cast<const float4*>(cp + j);
            const float4 s4v = *reinterpret_cast<const float4*>(sp + j);
            const float cc[4] = {c4v.x, c4v.y, c4v.z, c4v.w}, ss[4] = {s4v.x, s4v.y, s4v.z, s4v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float fa = a[j + e], fb = b[j + e];
              a[j + e] = __fmaf_rn(fa, cc[e], -__fmul_rn(fb, ss[e]));
              b[j + e] = __fmaf_rn(fb, cc[e], __fmul_rn(fa, ss[e]));
            }
          }
        }
        put(stage, lane, ca, a);
        put(stage, lane, cb, b);
      }
      EpiSwiglu::flush(stage, p.C, p.ldc, row0, rows_valid, colh, N, lane);
    }
  }
};

static int launch_rope_pair(const void* A, const void* W, int M, int N, int K, long long lda, long long ldb,
                            const RopeParams& rp, cudaStream_t stream) {
  using Epi = EpiRope;
  constexpr int STAGES = 6;
  using S = SmemPair<STAGES>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  rc = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK,
                    PAIR_HALF_N, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  auto kern = gemm_pair_kernel<STAGES, false, false, Epi>;
  const int smem_bytes = S::bytes(Epi::SMEM_BYTES);
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    attr_set = true;
  }
  const int tiles = ceil_div(M, PAIR_BM) * ceil_div(N, PAIR_BN);
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, M, N, K, 1, rp, device_err_word(), 1, nullptr, 0);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// Backward of SwiGLU in the epilogue of the down projection's dgrad GEMM: the accumulator tile is d(act) for 256 tokens
// x 256 features; the warp pulls the matching gate and up values (32 rows x 128 columns each, coalesced 256-byte row
// segments) into two swizzled stages, every lane then works on its own row - d(act) rounded to bf16 first, so that the
// result equals GEMM + stand-alone kernel bit for bit - and overwrites the stages with d(gate) and d(up), which leave
// as whole row segments. d(act) itself is never written.
struct SwigluBwdParams {
  const __nv_bfloat16* gu;   // [M, 2f] saved by the forward pass
  long long ld_gu;
  __nv_bfloat16* dgu;        // [M, 2f]
  long long ld_dgu;
  int f;
};

struct EpiSwigluBwd {
  using Params = SwigluBwdParams;
  static constexpr bool SPLIT_K = false;
  static constexpr int STAGE_BYTES = 2 * 32 * 256;     // gate and up stage per epilogue warp
  static constexpr int SMEM_BYTES = NUM_EPI_WARPS * STAGE_BYTES;

  static __device__ __forceinline__ void tile(const Params& p, uint32_t taddr, int m0, int n0, int M, int N, int quad,
                                              int lane, uint8_t* epi_smem) {
    uint8_t* sg = epi_smem + quad * STAGE_BYTES;
    uint8_t* su = sg + 32 * 256;
    const int row0 = m0 + quad * 32;
    const int rows_valid = min(32, M - row0);
    const int chunk = lane & 15;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      const int col0 = n0 + half * 128;
      if (col0 >= N) break;                              // N is a multiple of 128: a half is whole or absent
      const int col = col0 + chunk * 8;
      {
        uint4 t[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int row = 2 * j + (lane >> 4);
          t[j] = row < rows_valid ? __ldg(reinterpret_cast<const uint4*>(p.gu + (long long)(row0 + row) * p.ld_gu + col))
                                  : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int row = 2 * j + (lane >> 4);
          *reinterpret_cast<uint4*>(sg + row * 256 + ((chunk ^ (row & 15)) << 4)) = t[j];
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int row = 2 * j + (lane >> 4);
          t[j] = row < rows_valid
                     ? __ldg(reinterpret_cast<const uint4*>(p.gu + (long long)(row0 + row) * p.ld_gu + p.f + col))
                     : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int row = 2 * j + (lane >> 4);
          *reinterpret_cast<uint4*>(su + row * 256 + ((chunk ^ (row & 15)) << 4)) = t[j];
        }
      }
      __syncwarp();
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + half * 128 + c4 * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int off = lane * 256 + (((c4 * 4 + j) ^ (lane & 15)) << 4);
          const uint4 qg = *reinterpret_cast<const uint4*>(sg + off);
          const uint4 qu = *reinterpret_cast<const uint4*>(su + off);
          const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&qg);
          const __nv_bfloat162* hu = reinterpret_cast<const __nv_bfloat162*>(&qu);
          float dg[8], du[8];
#pragma unroll
          for (int t2 = 0; t2 < 4; ++t2) {
            const float2 g2 = __bfloat1622float2(hg[t2]);
            const float2 u2 = __bfloat1622float2(hu[t2]);
            const float gg[2] = {g2.x, g2.y}, uu[2] = {u2.x, u2.y};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float d = __bfloat162float(__float2bfloat16(__uint_as_float(r[j * 8 + t2 * 2 + e])));
              const float sgm = __fdividef(1.f, 1.f + __expf(-gg[e]));
              const float silu = gg[e] * sgm;
              dg[t2 * 2 + e] = d * uu[e] * (sgm + silu * (1.f - sgm));
              du[t2 * 2 + e] = d * silu;
            }
          }
          uint4 og, ou;
          og.x = pack_bf16x2(dg[0], dg[1]); og.y = pack_bf16x2(dg[2], dg[3]);
          og.z = pack_bf16x2(dg[4], dg[5]); og.w = pack_bf16x2(dg[6], dg[7]);
          ou.x = pack_bf16x2(du[0], du[1]); ou.y = pack_bf16x2(du[2], du[3]);
          ou.z = pack_bf16x2(du[4], du[5]); ou.w = pack_bf16x2(du[6], du[7]);
          *reinterpret_cast<uint4*>(sg + off) = og;
          *reinterpret_cast<uint4*>(su + off) = ou;
        }
      }
      EpiSwiglu::flush(sg, p.dgu, p.ld_dgu, row0, rows_valid, col0, p.f, lane);
      EpiSwiglu::flush(su, p.dgu + p.f, p.ld_dgu, row0, rows_valid, col0, p.f, lane);
    }
  }
};

static int launch_swiglu_bwd_pair(const void* dY, const void* Wd, int M, int f, int K, long long lda, long long ldb,
                                  const SwigluBwdParams& sp, cudaStream_t stream) {
  using Epi = EpiSwigluBwd;
  constexpr int STAGES = 5;                    // one ring stage less than the store kernel: the epilogue needs 64 KB
  using S = SmemPair<STAGES>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, dY, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  // W_d is [K = h, N = f] in memory: an MN-major B operand
  rc = make_tmap_2d(&tmB, Wd, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)f, (uint64_t)K, (uint64_t)ldb * 2, 64, BK,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  auto kern = gemm_pair_kernel<STAGES, false, true, Epi>;
  const int smem_bytes = S::bytes(Epi::SMEM_BYTES);
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    attr_set = true;
  }
  const int tiles = ceil_div(M, PAIR_BM) * ceil_div(f, PAIR_BN);
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, M, f, K, 1, sp, device_err_word(), 1, nullptr, 0);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

static int launch_swiglu_pair(const void* A, const void* Wgu, int M, int f, int K, long long lda, long long ldb,
                              const SwigluParams& sp, cudaStream_t stream) {
  using Epi = EpiSwiglu;
  constexpr int STAGES = 6;
  using S = SmemPair<STAGES>;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM,
                        CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  rc = make_tmap_2d(&tmB, Wgu, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)(2 * f), (uint64_t)ldb * 2, BK,
                    PAIR_HALF_N, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  auto kern = gemm_pair_kernel<STAGES, false, false, Epi>;
  const int smem_bytes = S::bytes(Epi::SMEM_BYTES);
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    attr_set = true;
  }
  const int N = 2 * f;
  const int tiles = ceil_div(M, PAIR_BM) * ceil_div(N, PAIR_BN);
  const int max_pairs = sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kern<<<2 * pairs, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, M, N, K, 1, sp, device_err_word(), 1, nullptr, f);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_store(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int fmt,
                        const StoreParams& sp, const DescCfg* dc_override, cudaStream_t stream) {
  using Epi = EpiStore<BN>;
  using S = Smem<BN, STAGES>;
  CUtensorMap tmA, tmB;
  const CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  int rc;
  if (!A_MN)
    rc = make_tmap_2d(&tmA, A, dt, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = make_tmap_2d(&tmA, A, dt, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  if (!B_MN)
    rc = make_tmap_2d(&tmB, B, dt, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = make_tmap_2d(&tmB, B, dt, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;

  auto kern = gemm_kernel<BN, STAGES, A_MN, B_MN, Epi>;
  const int smem_bytes = S::bytes(Epi::SMEM_BYTES);
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    attr_set = true;
  }
  const int tiles = ceil_div(M, BM) * ceil_div(N, BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  DescCfg dc = dc_override ? *dc_override : default_desc_cfg<BN, A_MN, B_MN>();
  kern<<<grid, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, M, N, K, fmt, dc, sp, device_err_word());
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// Counters of the ordered split-K epilogue: 8 per tile (one per epilogue warp of a CTA pair), zero between launches.
constexpr int SPLIT_MAX_TILES = 1024;
constexpr int SPLIT_MAX_SLICES = 15;
constexpr int SPLIT_REGIONS = 8;
__device__ unsigned int g_split_sync[SPLIT_REGIONS * SPLIT_MAX_TILES * 8];

// B200_GEMM_KSPLITS=n forces n slices wherever split-K is possible (experiments); unset: the launcher's estimate
static int split_k_forced() {
  static int n = -1;
  if (n < 0) {
    const char* e = getenv("B200_GEMM_KSPLITS");
    n = e ? atoi(e) : 0;
  }
  return n;
}

static bool split_k_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("B200_GEMM_SPLITK");
    on = e ? (atoi(e) != 0) : 1;
  }
  return on != 0;
}

// Two-SM (cta_group::2) launch: 256 x 256 tiles, one CTA pair per tile.
template <bool A_MN, bool B_MN>
static int launch_store_pair(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int fmt,
                             const StoreParams& sp, cudaStream_t stream) {
  using Epi = EpiStore<PAIR_BN>;
  constexpr int STAGES = 6;
  using S = SmemPair<STAGES>;
  CUtensorMap tmA, tmB;
  const CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  int rc;
  if (!A_MN)
    rc = make_tmap_2d(&tmA, A, dt, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = make_tmap_2d(&tmA, A, dt, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  if (!B_MN)
    rc = make_tmap_2d(&tmB, B, dt, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, PAIR_HALF_N,
                      CU_TENSOR_MAP_SWIZZLE_128B);
  else
    rc = make_tmap_2d(&tmB, B, dt, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  auto kern = gemm_pair_kernel<STAGES, A_MN, B_MN, Epi>;
  const int smem_bytes = S::bytes(Epi::SMEM_BYTES);
  static bool attr_set = false;
  if (!attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    attr_set = true;
  }
  const int tiles = ceil_div(M, PAIR_BM) * ceil_div(N, PAIR_BN);
  const int max_pairs = sm_count() / 2;
  // split-K for fp32 outputs with a long reduction and too few tiles for even waves (weight-gradient GEMMs); the
  // slices of a tile are added in a fixed order (gemm_pair.cuh)
  int k_splits = 1;
  const int num_kb = ceil_div(K, BK);
  if (sp.out_f32 && !sp.resid && !(N & 3) && !(sp.ldc & 3) && tiles <= SPLIT_MAX_TILES && split_k_enabled()) {
    const int forced = split_k_forced();
    if (forced > 0) {
      k_splits = forced;
    } else {
      // rounds of the pair grid in units of one whole tile: ceil(tiles * s / pairs) / s, plus 1.5 % per extra slice for
      // its read-modify-write epilogue; split only when that buys at least 7 %
      const double unsplit = (double)((tiles + max_pairs - 1) / max_pairs);
      double best = unsplit;
      for (int s2 = 2; s2 <= SPLIT_MAX_SLICES && num_kb / s2 >= 16; ++s2) {
        const double c = (double)((tiles * s2 + max_pairs - 1) / max_pairs) / s2 * (1.0 + 0.015 * (s2 - 1));
        if (c < best - 1e-9) { best = c; k_splits = s2; }
      }
      if (best > 0.93 * unsplit) k_splits = 1;
    }
    if (k_splits > num_kb) k_splits = num_kb;
    if (k_splits > SPLIT_MAX_SLICES) k_splits = SPLIT_MAX_SLICES;
  }
  unsigned int* sync = nullptr;
  if (k_splits > 1) {
    // one of 8 counter regions in turn, so that split launches on different streams do not share counters
    static unsigned int* base[64] = {};        // the array's address on each device of this process
    static std::atomic<unsigned int> turn{0};
    int dev = 0;
    B200_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B200_ERR_ARG;
    if (!base[dev]) B200_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&base[dev]), g_split_sync));
    sync = base[dev] + (size_t)(turn.fetch_add(1) % SPLIT_REGIONS) * (SPLIT_MAX_TILES * 8);
  }
  const long long units = (long long)tiles * k_splits;
  const int pairs = units < max_pairs ? (int)units : max_pairs;
  kern<<<2 * pairs, NUM_THREADS, smem_bytes, stream>>>(tmA, tmB, M, N, K, fmt, sp, device_err_word(), k_splits, sync, 0);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// 0 = never, 1 = whenever the shape allows, unset = heuristic (enough 256 x 256 tiles to fill the SM pairs)
static int pair_mode() {
  static int mode = -2;
  if (mode == -2) {
    const char* e = getenv("B200_GEMM_PAIR");
    mode = e ? atoi(e) : -1;
  }
  return mode;
}

static bool use_pair(int M, int N, int K) {
  const int mode = pair_mode();
  if (mode == 0 || N <= 128) return false;
  if (mode == 1) return true;
  const long long tiles = (long long)ceil_div(M, PAIR_BM) * ceil_div(N, PAIR_BN);
  return (tiles >= sm_count() / 2 && K >= 256) || (tiles >= sm_count() / 8 && K >= 4096);
}

}  // namespace gemm
}  // namespace b200

extern "C" {

// Zeroes the counters of the ordered split-K epilogue on the current device. A launch leaves them at zero by itself;
// a kernel that gave up on a bounded wait may not have, so the host calls this when it has taken note of such an error.
int b200_gemm_reset_split_sync(cudaStream_t stream) {
  using namespace b200;
  using namespace b200::gemm;
  unsigned int* base = nullptr;
  B200_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_split_sync));
  B200_CUDA_CHECK(cudaMemsetAsync(base, 0, sizeof(unsigned int) * SPLIT_REGIONS * SPLIT_MAX_TILES * 8, stream));
  return B200_OK;
}

// gu[M, 2f] = x[M, K] Wgu[2f, K]^T (rows 0..f-1 of Wgu: gate, f..2f-1: up) and act[M, f] = silu(gate) * up, bf16, in one
// launch. f must be a multiple of 128; row strides (elements) multiples of 8. Returns B200_ERR_ARG for shapes the fused
// kernel does not take (the caller then runs the GEMM and the SwiGLU kernel).
int b200_gemm_swiglu(const void* x, const void* Wgu, void* gu, void* act, int M, int f, int K, long long ldx,
                     long long ldw, long long ld_gu, long long ld_act, cudaStream_t stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (!x || !Wgu || !gu || !act || M <= 0 || f <= 0 || K <= 0 || (f % PAIR_HALF_N) || (ldx & 7) || (ldw & 7) ||
      (ld_gu & 7) || (ld_act & 7) || (reinterpret_cast<uintptr_t>(gu) & 15) || (reinterpret_cast<uintptr_t>(act) & 15))
    return B200_ERR_ARG;
  SwigluParams sp{reinterpret_cast<__nv_bfloat16*>(gu), ld_gu, reinterpret_cast<__nv_bfloat16*>(act), ld_act, f};
  return launch_swiglu_pair(x, Wgu, M, f, K, ldx, ldw, sp, stream);
}

// qkv[M, N] = x[M, K] W[N, K]^T with the rotary embedding applied to the first n_rot_heads heads of every row in the
// epilogue (pos int32 [M]; cos / sin fp32 [max_pos, d/2]). d = 64 or 128, N a multiple of 128.
int b200_gemm_rope(const void* x, const void* W, void* out, const int* pos, const float* cos_tab, const float* sin_tab,
                   int M, int N, int K, int n_rot_heads, int d, long long ldx, long long ldw, long long ldo,
                   cudaStream_t stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (!x || !W || !out || !pos || !cos_tab || !sin_tab || M <= 0 || N <= 0 || K <= 0 || (d != 64 && d != 128) ||
      (N % PAIR_HALF_N) || n_rot_heads < 0 || n_rot_heads * d > N || (ldx & 7) || (ldw & 7) || (ldo & 7) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return B200_ERR_ARG;
  RopeParams rp{reinterpret_cast<__nv_bfloat16*>(out), ldo, pos, cos_tab, sin_tab, d, n_rot_heads * d};
  return launch_rope_pair(x, W, M, N, K, ldx, ldw, rp, stream);
}

// dgu[M, 2f] = SwiGLU backward of (gu, d(act)) with d(act) = dy[M, K] Wd[K, f] taken straight from the accumulator
// (never written). f a multiple of 128; strides multiples of 8. B200_ERR_ARG for shapes the fused kernel does not take.
int b200_gemm_swiglu_bwd(const void* dy, const void* Wd, const void* gu, void* dgu, int M, int f, int K, long long ld_dy,
                         long long ldw, long long ld_gu, long long ld_dgu, cudaStream_t stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (!dy || !Wd || !gu || !dgu || M <= 0 || f <= 0 || K <= 0 || (f % PAIR_HALF_N) || (ld_dy & 7) || (ldw & 7) ||
      (ld_gu & 7) || (ld_dgu & 7) || (reinterpret_cast<uintptr_t>(gu) & 15) || (reinterpret_cast<uintptr_t>(dgu) & 15))
    return B200_ERR_ARG;
  SwigluBwdParams sp{reinterpret_cast<const __nv_bfloat16*>(gu), ld_gu, reinterpret_cast<__nv_bfloat16*>(dgu), ld_dgu, f};
  return launch_swiglu_bwd_pair(dy, Wd, M, f, K, ld_dy, ldw, sp, stream);
}

// C[M,N] = alpha * op(A) * op(B)^T (+ C if accumulate) (+ residual)
//   a_mn = 0: A is [M,K] with row stride lda;   a_mn = 1: A is stored [K,M] with row stride lda
//   b_mn = 0: B is [N,K] with row stride ldb;   b_mn = 1: B is stored [K,N] with row stride ldb
//   fmt: 1 = bf16 operands, 0 = fp16.  out_f32: C is fp32, else the operand type.
// Strides are in elements and must be multiples of 8 (16 bytes); base pointers 16-byte aligned.
// desc_cfg: optional 6 x uint32 override of the matrix-descriptor byte offsets (testing hook), else null.
int b200_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
              long long ldc, int a_mn, int b_mn, int fmt, int out_f32, int accumulate, float alpha,
              const void* residual, long long ldr, const unsigned int* desc_cfg, cudaStream_t stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return B200_ERR_ARG;
  if ((lda & 7) || (ldb & 7)) return B200_ERR_ARG;
  StoreParams sp;
  sp.C = C;
  sp.ldc = ldc;
  sp.resid = reinterpret_cast<const __nv_bfloat16*>(residual);
  sp.ldr = ldr;
  sp.alpha = alpha;
  sp.out_f32 = out_f32;
  sp.accumulate = accumulate;
  sp.fmt = fmt;
  DescCfg dco;
  const DescCfg* dcp = nullptr;
  if (desc_cfg) {
    dco.a_lbo = desc_cfg[0]; dco.a_sbo = desc_cfg[1]; dco.a_kadv = desc_cfg[2];
    dco.b_lbo = desc_cfg[3]; dco.b_sbo = desc_cfg[4]; dco.b_kadv = desc_cfg[5];
    dcp = &dco;
  }
  if (!dcp && use_pair(M, N, K)) {
    if (!a_mn && !b_mn) return launch_store_pair<false, false>(A, B, M, N, K, lda, ldb, fmt, sp, stream);
    if (!a_mn && b_mn) return launch_store_pair<false, true>(A, B, M, N, K, lda, ldb, fmt, sp, stream);
    if (a_mn && b_mn) return launch_store_pair<true, true>(A, B, M, N, K, lda, ldb, fmt, sp, stream);
    return launch_store_pair<true, false>(A, B, M, N, K, lda, ldb, fmt, sp, stream);
  }
  const bool small_n = N <= 128;
  if (!a_mn && !b_mn) {
    return small_n ? launch_store<128, 6, false, false>(A, B, M, N, K, lda, ldb, fmt, sp, dcp, stream)
                   : launch_store<256, 4, false, false>(A, B, M, N, K, lda, ldb, fmt, sp, dcp, stream);
  } else if (!a_mn && b_mn) {
    return small_n ? launch_store<128, 6, false, true>(A, B, M, N, K, lda, ldb, fmt, sp, dcp, stream)
                   : launch_store<256, 4, false, true>(A, B, M, N, K, lda, ldb, fmt, sp, dcp, stream);
  } else if (a_mn && b_mn) {
    return small_n ? launch_store<128, 6, true, true>(A, B, M, N, K, lda, ldb, fmt, sp, dcp, stream)
                   : launch_store<256, 4, true, true>(A, B, M, N, K, lda, ldb, fmt, sp, dcp, stream);
  } else {
    return small_n ? launch_store<128, 6, true, false>(A, B, M, N, K, lda, ldb, fmt, sp, dcp, stream)
                   : launch_store<256, 4, true, false>(A, B, M, N, K, lda, ldb, fmt, sp, dcp, stream);
  }
}
}
