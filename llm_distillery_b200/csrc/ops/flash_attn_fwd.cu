// Causal GQA flash-attention forward for sm_100a on tcgen05 tensor cores.
//
// One CTA = one (batch, q-head, 128-query block). Roles (192 threads):
//   warp 0    TMA producer : Q once, then K/V tiles of BN keys through a 2-stage smem ring (3D tensor map
//                            [B][L][width], so rows past the sequence end read zeros; no multicast)
//   warp 1    MMA issuer   : S = Q K^T   (tcgen05.mma, both operands K-major, accumulator S in TMEM)
//                            O += P V    (P from smem as K-major A, V as MN-major B, accumulator O in TMEM)
//   warps 2-5 softmax      : thread = query row. Reads S from TMEM, causal mask, online softmax in the exp2
//                            domain, writes P (bf16) into 128B-swizzled smem, rescales O in TMEM only when
//                            the running max grew by more than 2^8 (lazy rescale), final O / l and lse.
// S and O live in TMEM (BN + D <= 192 columns, 256 allocated) and smem is ~112 KB, so two CTAs share an SM
// and overlap each other's MMA and softmax phases.
//
// Layout: qkv [T, (H + 2*Hkv) * D] bf16 with T = B*L; out [T, H*D] bf16; lse [H, T] fp32 (natural log).
#include "../common/ptx.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace fa {

constexpr int BM = 128;
constexpr int NTHREADS = 192;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units

template <int D>
struct Cfg {
  static constexpr int BN = (D == 64) ? 128 : 64;
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int K_BYTES = BN * D * 2;
  static constexpr int V_BYTES = BN * D * 2;
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
  static constexpr int P_BYTES = BM * BN * 2;
  static constexpr int STAGES = 2;
  static constexpr int OFF_KV = Q_BYTES;
  static constexpr int OFF_P = OFF_KV + STAGES * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr uint32_t TMEM_COLS = 256;
  static constexpr uint32_t S_COL = 0;
  static constexpr uint32_t O_COL = BN;
};

struct FwdParams {
  __nv_bfloat16* out;
  float* lse;
  int B, L, H, Hkv;
  float scale;  // 1/sqrt(D)
};

template <int D>
__global__ void __launch_bounds__(NTHREADS, 2)
    flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, FwdParams p,
                     unsigned int* err_word) {
  using C = Cfg<D>;
  constexpr int BN = C::BN;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_ready = bars + 6;
  uint64_t* o_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.L + BM - 1) / BM;
  const int qb = nqb - 1 - blockIdx.x;  // heaviest (longest causal span) blocks first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hkv = hq / (p.H / p.Hkv);
  const int q0 = qb * BM;
  const int kv_end = min(p.L, q0 + BM);  // causal: keys < kv_end
  const int n_kv = (kv_end + BN - 1) / BN;

  if ((smem_u32(smem) & 1023u) != 0u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && err_word) atomicCAS(err_word, 0u, (unsigned)ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int colQ = hq * D;
  const int colK = p.H * D + hkv * D;
  const int colV = (p.H + p.Hkv) * D + hkv * D;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_3d(smem + c * (BM * 128), &tmQ, q_full, colQ + c * 64, q0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1u;
        if (!mbar_wait_bounded(&kv_empty[s], ph ^ 1u, abort_flag, err_word, ERR_WAIT_EMPTY)) break;
        uint8_t* sK = smem + C::OFF_KV + s * C::STAGE_BYTES;
        uint8_t* sV = sK + C::K_BYTES;
        mbar_arrive_expect_tx(&kv_full[s], C::STAGE_BYTES);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_3d(sK + c * (BN * 128), &tmKV, &kv_full[s], colK + c * 64, j * BN, b);
          tma_load_3d(sV + c * (BN * 128), &tmKV, &kv_full[s], colV + c * 64, j * BN, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(1, BM, BN, 0, 0);
      const uint32_t idesc_o = make_idesc_f16(1, BM, D, 0, 1);
      const uint32_t sQ = smem_u32(smem);
      const uint32_t sP = smem_u32(smem + C::OFF_P);
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, err_word, ERR_WAIT_FULL);
      // S = Q K^T for the K tile in stage s: D/16 k-steps; 64-column sub-tiles are BM*128 (Q) / BN*128 (K) bytes apart
      auto issue_s = [&](int s) {
        const uint32_t sK = smem_u32(smem + C::OFF_KV + s * C::STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t sub = k >> 2, kk = k & 3;
          const uint64_t da = make_smem_desc_sw128(sQ + sub * (BM * 128) + kk * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sK + sub * (BN * 128) + kk * 32, 16, 1024);
          umma_f16_ss(tmem_base + C::S_COL, da, db, idesc_s, k != 0 ? 1u : 0u);
        }
      };
      if (ok && n_kv > 0) {
        ok = mbar_wait_bounded(&kv_full[0], 0, abort_flag, err_word, ERR_WAIT_FULL);
        if (ok) {
          tc_fence_after_sync();
          issue_s(0);
          umma_commit(s_full);
        }
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int s = j & 1;
        // wait for P_j (and the O rescale) from the softmax warps: S is free again from here on
        if (!mbar_wait_bounded(p_ready, j & 1u, abort_flag, err_word, ERR_WAIT_AUX)) break;
        tc_fence_after_sync();
        if (j + 1 < n_kv) {
          // the next tile's scores go to the tensor core AHEAD of this tile's P V, so that the softmax warps find
          // S_{j+1} ready as soon as they are done with tile j
          const int s1 = (j + 1) & 1;
          if (!mbar_wait_bounded(&kv_full[s1], ((j + 1) >> 1) & 1u, abort_flag, err_word, ERR_WAIT_FULL)) break;
          tc_fence_after_sync();
          issue_s(s1);
          umma_commit(s_full);
        }
        const uint32_t sV = smem_u32(smem + C::OFF_KV + s * C::STAGE_BYTES) + C::K_BYTES;
        // O += P V : BN/16 k-steps over keys; V is MN-major (D contiguous), 64-wide D chunks BN*128 bytes apart
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint32_t sub = k >> 2, kk = k & 3;
          const uint64_t da = make_smem_desc_sw128(sP + sub * (BM * 128) + kk * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sV + k * (16 * 128), BN * 128, 1024);
          umma_f16_ss(tmem_base + C::O_COL, da, db, idesc_o, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&kv_empty[s]);
        umma_commit(o_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // row inside the q block
    const int qi = q0 + r;           // position in the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;  // scores -> log2 domain
    float m_used = -INFINITY, l = 0.f;
    uint8_t* sP = smem + C::OFF_P;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      int w = mbar_wait_bounded(s_full, j & 1u, abort_flag, err_word, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
      tc_fence_after_sync();
      const int kv0 = j * BN;
      const bool diag = (kv0 + BN - 1) > q0;  // some keys of this tile may be masked for some rows
      // pass 1: row max (the masked variant only runs on tiles that cross the diagonal)
      float mx = -INFINITY;
      if (!diag) {
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + C::S_COL + c * 32, v);
          tmem_ld_wait();
          float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
          for (int t = 0; t < 32; t += 2) {
            m0 = fmaxf(m0, __uint_as_float(v[t]));
            m1 = fmaxf(m1, __uint_as_float(v[t + 1]));
          }
          mx = fmaxf(mx, fmaxf(m0, m1));
        }
      } else {
        const int lim = qi - kv0;  // columns <= lim are visible
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + C::S_COL + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t)
            mx = fmaxf(mx, (c * 32 + t) <= lim ? __uint_as_float(v[t]) : -INFINITY);
        }
      }
      float alpha = 1.f;
      bool need = false;
      if (mx > m_used) {
        if (m_used == -INFINITY) {
          m_used = mx;  // first tile with a visible key: nothing accumulated yet for this row
          need = (j > 0);
          alpha = 0.f;  // anything accumulated so far came from fully masked tiles (all-zero P)
        } else if ((mx - m_used) * c2 > kRescaleThreshold) {
          alpha = exp2f((m_used - mx) * c2);
          m_used = mx;
          need = true;
        }
      }
      l *= alpha;
      // P smem is single-buffered and O is about to be touched: the previous P*V must be complete
      if (j > 0) {
        int w2 = mbar_wait_bounded(o_done, (j - 1) & 1u, abort_flag, err_word, ERR_WAIT_AUX) ? 1 : 0;
        if (!__all_sync(0xffffffffu, w2)) { ok = false; break; }
        tc_fence_after_sync();
      }
      // pass 2: p = exp2((s - m) * c2) -> bf16 -> swizzled smem ; l += sum(p)
      const float mb = (m_used == -INFINITY) ? 0.f : m_used * c2;
      float lsum = 0.f, lsum1 = 0.f;
      const int lim2 = diag ? (qi - kv0) : 0x7fffffff;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + C::S_COL + c * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
        if (!diag) {
#pragma unroll
          for (int t = 0; t < 32; t += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(v[t]), c2, -mb));
            const float p1 = fast_exp2(fmaf(__uint_as_float(v[t + 1]), c2, -mb));
            lsum += p0;
            lsum1 += p1;
            pk[t >> 1] = pack_bf16x2(p0, p1);
          }
        } else {
#pragma unroll
          for (int t = 0; t < 32; t += 2) {
            float p0 = fast_exp2(fmaf(__uint_as_float(v[t]), c2, -mb));
            float p1 = fast_exp2(fmaf(__uint_as_float(v[t + 1]), c2, -mb));
            if ((c * 32 + t) > lim2) p0 = 0.f;
            if ((c * 32 + t + 1) > lim2) p1 = 0.f;
            lsum += p0;
            lsum1 += p1;
            pk[t >> 1] = pack_bf16x2(p0, p1);
          }
        }
        // columns c*32 .. c*32+31 of row r: sub-tile (c*32)/64, 16-byte chunks ((c*32)%64)/8 + {0..3}
        const int sub = (c * 32) >> 6;
        const int chunk0 = ((c * 32) & 63) >> 3;
        uint8_t* rowp = sP + sub * (BM * 128) + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int ch = (chunk0 + q4) ^ (r & 7);
          *reinterpret_cast<uint4*>(rowp + ch * 16) =
              make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
        }
      }
      lsum += lsum1;
      l += lsum;
      // lazy rescale of the O accumulator (warp-uniform decision: tcgen05.ld/st are warp-collective)
      if (__any_sync(0xffffffffu, need)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + C::O_COL + c * 32, v);
          tmem_ld_wait();
          uint32_t lo[16], hi[16];
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            lo[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
            hi[t] = __float_as_uint(__uint_as_float(v[16 + t]) * alpha);
          }
          tmem_st_32x32b_x16(tmem_base + lane_addr + C::O_COL + c * 32, lo);
          tmem_st_32x32b_x16(tmem_base + lane_addr + C::O_COL + c * 32 + 16, hi);
        }
        tmem_st_wait();
      }
      fence_proxy_async_smem();  // generic-proxy smem writes -> visible to the tensor core (async proxy)
      tc_fence_before_sync();
      mbar_arrive(p_ready);
    }
    // epilogue: O / l -> bf16, lse
    if (ok) {
      int w3 = mbar_wait_bounded(o_done, (n_kv - 1) & 1u, abort_flag, err_word, ERR_WAIT_AUX) ? 1 : 0;
      if (__all_sync(0xffffffffu, w3)) {
        tc_fence_after_sync();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const bool row_ok = qi < p.L;
        const long long t = (long long)b * p.L + qi;
        __nv_bfloat16* orow = p.out + t * (long long)(p.H * D) + hq * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + C::O_COL + c * 32, v);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]) * inv, __uint_as_float(v[q4 * 8 + 1]) * inv);
              o.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]) * inv, __uint_as_float(v[q4 * 8 + 3]) * inv);
              o.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]) * inv, __uint_as_float(v[q4 * 8 + 5]) * inv);
              o.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]) * inv, __uint_as_float(v[q4 * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = o;
            }
          }
        }
        if (row_ok && p.lse)
          p.lse[(long long)hq * ((long long)p.B * p.L) + t] = m_used * p.scale + logf(l);
      }
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int D>
static int launch_fwd(const void* qkv, void* out, float* lse, int B, int L, int H, int Hkv, cudaStream_t st) {
  using C = Cfg<D>;
  const long long width = (long long)(H + 2 * Hkv) * D;
  CUtensorMap tmQ, tmKV;
  int rc = make_tmap_3d(&tmQ, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)width, (uint64_t)L, (uint64_t)B,
                        (uint64_t)width * 2, (uint64_t)L * width * 2, 64, BM, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  rc = make_tmap_3d(&tmKV, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)width, (uint64_t)L, (uint64_t)B,
                    (uint64_t)width * 2, (uint64_t)L * width * 2, 64, C::BN, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  auto kern = flash_fwd_kernel<D>;
  static bool attr = false;
  if (!attr) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    attr = true;
  }
  FwdParams p{(__nv_bfloat16*)out, lse, B, L, H, Hkv, 1.0f / sqrtf((float)D)};
  dim3 grid((L + BM - 1) / BM, H, B);
  kern<<<grid, NTHREADS, C::SMEM_BYTES, st>>>(tmQ, tmKV, p, device_err_word());
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace fa
}  // namespace b200

extern "C" int b200_flash_attn_fwd(const void* qkv, void* out, float* lse, int B, int L, int H, int Hkv, int D,
                                   cudaStream_t st) {
  using namespace b200;
  if (!qkv || !out || B <= 0 || L <= 0 || H <= 0 || Hkv <= 0 || (H % Hkv) != 0) return B200_ERR_ARG;
  if (D == 64) return fa::launch_fwd<64>(qkv, out, lse, B, L, H, Hkv, st);
  if (D == 128) return fa::launch_fwd<128>(qkv, out, lse, B, L, H, Hkv, st);
  return B200_ERR_ARG;
}
