// Causal GQA flash-attention forward for sm_100a on tcgen05 tensor cores.
//
// One CTA = one (batch, q-head, 128-query block); keys are walked in tiles of BN = 64. Roles (224 threads):
//   warp 0    TMA producer : Q once, then K tiles through a 3-stage ring and V tiles through a 2-stage ring (3D tensor
//                            map [B][L][width], so rows past the sequence end read zeros; no multicast)
//   warp 1    P V issuer   : O += P_j V_j with A = P_j read from TMEM and V_j as MN-major B from shared memory
//   warp 2    S issuer     : S_j = Q K_j^T (tcgen05.mma, both operands K-major) into one of TWO score buffers in TMEM
//                            (two issuing threads because every tcgen05 instruction - MMA, commit, a completed
//                            mbarrier wait - costs its issuer on the order of a hundred cycles here: one thread
//                            issuing both groups of a 64-key tile took longer than the softmax of that tile)
//   warps 3-6 softmax      : thread = query row. Reads S_j from TMEM once (both 32-column loads in flight),
//                            exponentiates against the maximum known so far (exp2 domain, packed f32x2 arithmetic,
//                            optionally part of the exponentials on the FMA pipe), writes P_j as bf16 pairs over the first half
//                            of the same score buffer, and only when a score outgrew the maximum by more than 2^8
//                            moves the maximum, rescales O in TMEM and redoes the tile; final O / l and lse.
// The score buffers alternate: S_{j+1} is computed while the softmax warps work on S_j, and S_{j+2} goes into S_j's
// buffer as soon as P_j V_j has completed, so in the steady state the softmax warps never wait for the tensor core.
// P never touches shared memory: an N = D MMA fed from shared memory on both sides is bound by shared-memory
// bandwidth, and the softmax warps issue no st.shared and no proxy fence.
// TMEM: 2 x 64 score columns + D output columns (<= 256); shared memory 56 KB (D = 64) / 112 KB (D = 128): two CTAs
// share an SM.
//
// Layout: qkv [T, (H + 2*Hkv) * D] bf16 with T = B*L; out [T, H*D] bf16; lse [H, T] fp32 (natural log).
#include "../common/ptx.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace fa {

constexpr int BM = 128;
constexpr int BN = 64;
constexpr int NTHREADS = 224;
constexpr int VS = 2;  // V ring
constexpr float kRescaleThreshold = 8.0f;  // in log2 units
// Measured (B200, 1965 MHz): 0.254 ms / 0.264 ms (head dim 64, batch 8 x 2048 / head dim 128, batch 2 x 4096) with every
// exponential on the MUFU unit, 0.268 / 0.283 with a quarter of them as polynomials, 0.297 / 0.311 with half: with
// one query row per thread the softmax warps are bound by instruction latency, not by the 16 exponentials per clock
// of the MUFU unit, so the extra FMA-pipe instructions cost more than they free. The polynomial path stays in the
// kernel (B200_FA_POLY = 2, 3 or 4 eighths) for shapes where that changes.
constexpr int kDefaultPoly8 = 0;

template <int D>
struct Cfg {
  // Score buffers in TMEM: S_{t} may be issued as soon as P_{t-NBUF} V_{t-NBUF} has completed. With two buffers that
  // dependency (softmax_j -> P_j V_j -> S_{j+2}) is longer than one softmax and the softmax warps idle a third of
  // the time; a third buffer (head dim 64: 3 x 64 + 64 columns = 256) takes it off the critical path.
  static constexpr int NBUF = (3 * BN + D <= 256) ? 3 : 2;
  static constexpr int KS = NBUF + 1;  // K ring: K runs NBUF tiles ahead of the softmax
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int T_BYTES = BN * D * 2;  // one K or V tile
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + KS * T_BYTES;   // KS declared above
  static constexpr int OFF_BAR = OFF_V + VS * T_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr uint32_t TMEM_COLS = 256;
  static constexpr uint32_t S_COL = 0;        // NBUF buffers of BN columns; P_j overwrites columns [0, BN/2) of S_j
  static constexpr uint32_t O_COL = NBUF * BN;
  static_assert(NBUF * BN + D <= 256, "TMEM budget");
};

struct FwdParams {
  __nv_bfloat16* out;
  float* lse;
  int B, L, H, Hkv;
  float scale;  // 1/sqrt(D)
  // Chunked prefill: the L queries are positions q_off .. q_off + L - 1 of a sequence whose earlier keys / values
  // sit in a cache (row p of the K / V tensors = position p). q_off = 0 and K / V inside the same packed tensor as Q
  // is the ordinary whole-sequence call.
  int q_off;
  int colQ0, colK0, colV0;  // first column of head 0 of Q / K / V in their tensors
};

// 2^x for x <= 0 (and a little above) on the FMA pipe: round-to-nearest split x = n + f, f in [-0.5, 0.5], a quartic
// for 2^f (relative error 4e-5, far below bf16 resolution), n added into the exponent field. The MUFU unit does 16
// exponentials per clock and SM, which is what bounds this kernel; taking a share of them off it is worth the
// extra FMA-pipe instructions.
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -126.f);
  const float magic = 12582912.f;  // 1.5 * 2^23: adding it rounds to an integer in the low mantissa bits
  const float xr = x + magic;
  const float f = x - (xr - magic);
  float pl = fmaf(f, 0.0096181291f, 0.0555041087f);
  pl = fmaf(pl, f, 0.2402265070f);
  pl = fmaf(pl, f, 0.6931471806f);
  pl = fmaf(pl, f, 1.0f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(xr) << 23));
}

// POLY8: of every 8 pairs of exponentials, this many are evaluated on the FMA pipe instead of the MUFU unit.
template <int D, int POLY8>
__global__ void __launch_bounds__(NTHREADS, 2)
    flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, FwdParams p, unsigned int* err_word) {
  using C = Cfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  constexpr int KS = C::KS, NBUF = C::NBUF;
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [KS]   (KS <= 4)
  uint64_t* k_empty = bars + 5;   // [KS]
  uint64_t* v_full = bars + 9;    // [VS]
  uint64_t* s_full = bars + 11;   // [NBUF] S_t complete (buffer t % NBUF)
  uint64_t* p_ready = bars + 14;  // [NBUF] P_j written by the 128 softmax threads
  uint64_t* pv_done = bars + 17;  // [NBUF] P_j V_j complete: its score buffer and V stage are free, O holds tile j
  uint64_t* o_final = bars + 20;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.L + BM - 1) / BM;
  // blockIdx.x runs over (head, batch) and blockIdx.y over the query blocks, longest causal span first: the hardware
  // hands out blocks x-fastest, so EVERY head's heaviest block starts before any light one and the light blocks fill
  // the tail (with the query block fastest, the last head's heaviest block started when the grid was almost through)
  const int qb = nqb - 1 - blockIdx.y;
  const int hq = blockIdx.x % p.H, b = blockIdx.x / p.H;
  const int hkv = hq / (p.H / p.Hkv);
  const int q0 = qb * BM;
  const int qpos0 = p.q_off + q0;                       // sequence position of the block's first query
  const int kv_end = p.q_off + min(p.L, q0 + BM);       // causal: keys < kv_end
  const int n_kv = (kv_end + BN - 1) / BN;

  if ((smem_u32(smem) & 1023u) != 0u) {  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && err_word) atomicCAS(err_word, 0u, (unsigned)ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    for (int s = 0; s < KS; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < VS; ++s) mbar_init(&v_full[s], 1);
    for (int s = 0; s < NBUF; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_ready[s], 128);
      mbar_init(&pv_done[s], 1);
    }
    mbar_init(o_final, 1);
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

  const int colQ = p.colQ0 + hq * D;
  const int colK = p.colK0 + hkv * D;
  const int colV = p.colV0 + hkv * D;

  if (warp == 0) {
    // two producer threads: K runs NBUF tiles ahead of the softmax and must not queue behind the V loads, which are
    // gated by the P V MMAs two tiles back
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_3d(smem + c * (BM * 128), &tmQ, q_full, colQ + c * 64, q0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int ks = j % KS;
        if (!mbar_spin_bounded(&k_empty[ks], ((j / KS) & 1u) ^ 1u, abort_flag, err_word, ERR_WAIT_EMPTY)) break;
        uint8_t* sK = smem + C::OFF_K + ks * C::T_BYTES;
        mbar_arrive_expect_tx(&k_full[ks], C::T_BYTES);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_3d(sK + c * (BN * 128), &tmK, &k_full[ks], colK + c * 64, j * BN, b);
      }
    } else if (lane == 1) {
      for (int j = 0; j < n_kv; ++j) {
        const int vs = j % VS;
        // V stage j % VS was read by P_{j-VS} V_{j-VS}
        if (j >= VS && !mbar_spin_bounded(&pv_done[(j - VS) % NBUF], ((j - VS) / NBUF) & 1u, abort_flag, err_word,
                                          ERR_WAIT_EMPTY))
          break;
        uint8_t* sV = smem + C::OFF_V + vs * C::T_BYTES;
        mbar_arrive_expect_tx(&v_full[vs], C::T_BYTES);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) tma_load_3d(sV + c * (BN * 128), &tmV, &v_full[vs], colV + c * 64, j * BN, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ O += P_j V_j
    if (lane == 0) {
      const uint32_t idesc_o = make_idesc_f16(1, BM, D, 0, 1);
      // descriptors are constants plus a stage offset (the address field counts 16-byte units): built once
      uint64_t dV[BN / 16];
#pragma unroll
      for (int k = 0; k < BN / 16; ++k)   // V is MN-major (D contiguous), 64-wide D chunks BN*128 bytes apart
        dV[k] = make_smem_desc_sw128(smem_u32(smem + C::OFF_V) + k * (16 * 128), BN * 128, 1024);
      bool ok = true;
      for (int j = 0; j < n_kv; ++j) {
        const int bsel = j % NBUF, vs = j % VS;
        // P_j is in TMEM (over the first half of S_j) once the softmax warps have arrived
        if (!mbar_spin_bounded(&p_ready[bsel], (j / NBUF) & 1u, abort_flag, err_word, ERR_WAIT_AUX)) { ok = false; break; }
        if (!mbar_spin_bounded(&v_full[vs], (j / VS) & 1u, abort_flag, err_word, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after_sync();
        const uint64_t stage = static_cast<uint64_t>((vs * C::T_BYTES) >> 4);
        const uint32_t pcol = tmem_base + C::S_COL + bsel * BN;   // bsel = j % NBUF
        // BN/16 k-steps over keys. A = P from TMEM (16 bf16 of a row = 8 columns per step)
        if (j == 0) {
#pragma unroll
          for (int k = 0; k < BN / 16; ++k)
            umma_f16_ts(tmem_base + C::O_COL, pcol + k * 8, dV[k] + stage, idesc_o, k != 0 ? 1u : 0u);
        } else {
#pragma unroll
          for (int k = 0; k < BN / 16; ++k) umma_f16_ts(tmem_base + C::O_COL, pcol + k * 8, dV[k] + stage, idesc_o, 1u);
        }
        umma_commit(&pv_done[bsel]);
      }
      if (ok) umma_commit(o_final);   // a barrier of its own for the last tile: the epilogue waits on nothing else
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ S_t = Q K_t^T
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(1, BM, BN, 0, 0);
      uint64_t dQ[D / 16], dK[D / 16];
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        const uint32_t sub = k >> 2, kk = k & 3;   // 64-column sub-tiles are BM*128 (Q) / BN*128 (K) bytes apart
        dQ[k] = make_smem_desc_sw128(smem_u32(smem) + sub * (BM * 128) + kk * 32, 16, 1024);
        dK[k] = make_smem_desc_sw128(smem_u32(smem + C::OFF_K) + sub * (BN * 128) + kk * 32, 16, 1024);
      }
      bool ok = mbar_spin_bounded(q_full, 0, abort_flag, err_word, ERR_WAIT_FULL);
      for (int t = 0; ok && t < n_kv; ++t) {
        const int ks = t % KS;
        // buffer t % NBUF held S_{t-NBUF} and then P_{t-NBUF}: it is free when that tile's P V has completed
        if (t >= NBUF && !mbar_spin_bounded(&pv_done[t % NBUF], ((t - NBUF) / NBUF) & 1u, abort_flag, err_word, ERR_WAIT_AUX))
          break;
        if (!mbar_spin_bounded(&k_full[ks], (t / KS) & 1u, abort_flag, err_word, ERR_WAIT_FULL)) break;
        tc_fence_after_sync();
        const uint64_t stage = static_cast<uint64_t>((ks * C::T_BYTES) >> 4);
        const uint32_t dcol = tmem_base + C::S_COL + (t % NBUF) * BN;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16_ss(dcol, dQ[k], dK[k] + stage, idesc_s, k != 0 ? 1u : 0u);
        umma_commit(&s_full[t % NBUF]);
        umma_commit(&k_empty[ks]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // row inside the q block
    const int qi = q0 + r;           // row of the query inside this call
    const int qpos = qpos0 + r;      // its position in the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;  // scores -> log2 domain
    const uint64_t c2p = pack_f32x2(c2, c2);
    const uint32_t tO = tmem_base + lane_addr + C::O_COL;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;

    // One 32-column chunk of scores -> probabilities (bf16 pairs) with the running maximum and the row sum.
    // `lim`: columns of this chunk with index <= lim are visible (>= 31: all of them). POLY8 of every 8 pairs of
    // exponentials are evaluated on the FMA pipe.
    auto chunk = [&](const uint32_t (&v)[32], const uint64_t nmb, const int lim, float& mx, uint64_t& sum2,
                     uint32_t (&pk)[16]) {
      if (lim >= 31) {
#pragma unroll
        for (int t = 0; t < 32; t += 2) {
          const float s0 = __uint_as_float(v[t]), s1 = __uint_as_float(v[t + 1]);
          mx = fmax3(mx, s0, s1);
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(s0, s1), c2p, nmb), x0, x1);
          const bool poly = ((t >> 1) & 7) < POLY8;
          const float p0 = poly ? poly_exp2(x0) : fast_exp2(x0);
          const float p1 = poly ? poly_exp2(x1) : fast_exp2(x1);
          sum2 = add_f32x2(sum2, pack_f32x2(p0, p1));
          pk[t >> 1] = pack_bf16x2(p0, p1);
        }
      } else {
#pragma unroll
        for (int t = 0; t < 32; t += 2) {
          const float s0 = t <= lim ? __uint_as_float(v[t]) : -INFINITY;
          const float s1 = (t + 1) <= lim ? __uint_as_float(v[t + 1]) : -INFINITY;
          mx = fmax3(mx, s0, s1);
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(s0, s1), c2p, nmb), x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);   // exp2(-inf) = 0 for the masked columns
          sum2 = add_f32x2(sum2, pack_f32x2(p0, p1));
          pk[t >> 1] = pack_bf16x2(p0, p1);
        }
      }
    };

    for (int j = 0; j < n_kv; ++j) {
      const int bsel = j % NBUF;
      const uint32_t tS = tmem_base + lane_addr + C::S_COL + bsel * BN;
      int w = mbar_wait_bounded(&s_full[bsel], (j / NBUF) & 1u, abort_flag, err_word, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
      tc_fence_after_sync();
      const int kv0 = j * BN;
      const bool diag = (kv0 + BN - 1) > qpos0;              // some keys of this tile are masked for some rows
      const int lim = diag ? (qpos - kv0) : 0x3fffffff;      // tile columns <= lim are visible to this row
      uint32_t va[32], vb[32], pka[16], pkb[16];
      tmem_ld_32x32b_x32(tS, va);
      tmem_ld_32x32b_x32(tS + 32, vb);
      tmem_ld_wait();
      if (j == 0) {
        // The first tile fixes the reference maximum (every row sees key 0, so it is finite). Later tiles are
        // exponentiated against the maximum known so far and only redone when a score exceeds it by more than
        // 2^kRescaleThreshold, which is rare once a row has seen a few hundred keys.
        float mx0 = -INFINITY;
#pragma unroll
        for (int t = 0; t < 32; t += 2) {
          mx0 = fmax3(mx0, t <= lim ? __uint_as_float(va[t]) : -INFINITY,
                      (t + 1) <= lim ? __uint_as_float(va[t + 1]) : -INFINITY);
          mx0 = fmax3(mx0, (t + 32) <= lim ? __uint_as_float(vb[t]) : -INFINITY,
                      (t + 33) <= lim ? __uint_as_float(vb[t + 1]) : -INFINITY);
        }
        m_used = mx0;
      }
      float mx = m_used;
      uint64_t sum2 = 0ull;
      uint64_t nmb = pack_f32x2(-m_used * c2, -m_used * c2);
      chunk(va, nmb, lim, mx, sum2, pka);
      chunk(vb, nmb, lim - 32, mx, sum2, pkb);
      const bool need = (mx - m_used) * c2 > kRescaleThreshold;
      if (__any_sync(0xffffffffu, need)) {
        // a score outgrew the reference maximum: move the maximum, rescale what is accumulated, redo the tile
        // (warp-uniform: tcgen05.ld / st are warp-collective; rows that did not need it repeat their own values).
        // O belongs to the previous tile's P V until that MMA is done.
        const float alpha = need ? fast_exp2((m_used - mx) * c2) : 1.f;
        if (need) m_used = mx;
        l *= alpha;
        if (j > 0) {
          int w2 = mbar_wait_bounded(&pv_done[(j - 1) % NBUF], ((j - 1) / NBUF) & 1u, abort_flag, err_word, ERR_WAIT_AUX) ? 1 : 0;
          if (!__all_sync(0xffffffffu, w2)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(tO + c * 32, v);
            tmem_ld_wait();
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              lo[t] = __float_as_uint(__uint_as_float(v[t]) * alpha);
              hi[t] = __float_as_uint(__uint_as_float(v[16 + t]) * alpha);
            }
            tmem_st_32x32b_x16(tO + c * 32, lo);
            tmem_st_32x32b_x16(tO + c * 32 + 16, hi);
          }
        }
        nmb = pack_f32x2(-m_used * c2, -m_used * c2);
        sum2 = 0ull;
        float mx2 = m_used;
        // S_j is still intact in TMEM (P_j is stored below): read it again rather than keep it in registers
        tmem_ld_32x32b_x32(tS, va);
        tmem_ld_wait();
        chunk(va, nmb, lim, mx2, sum2, pka);
        tmem_ld_32x32b_x32(tS + 32, va);
        tmem_ld_wait();
        chunk(va, nmb, lim - 32, mx2, sum2, pkb);
      }
      // P_j over the first half of S_j (both halves of S_j are in registers by now)
      tmem_st_32x32b_x16(tS, pka);
      tmem_st_32x32b_x16(tS + 16, pkb);
      {
        float s0, s1;
        unpack_f32x2(sum2, s0, s1);
        l += s0 + s1;
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[bsel]);
    }
    // epilogue: O / l -> bf16, lse
    if (ok) {
      int w3 = mbar_wait_bounded(o_final, 0, abort_flag, err_word, ERR_WAIT_AUX) ? 1 : 0;
      if (__all_sync(0xffffffffu, w3)) {
        tc_fence_after_sync();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const bool row_ok = qi < p.L;
        const long long t = (long long)b * p.L + qi;
        __nv_bfloat16* orow = p.out + t * (long long)(p.H * D) + hq * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tO + c * 32, v);
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
static int launch_fwd(const void* q, long long q_width, int colQ0, const void* k, const void* v, long long kv_width,
                      int colK0, int colV0, long long kv_rows, void* out, float* lse, int B, int L, int q_off, int H,
                      int Hkv, cudaStream_t st) {
  using C = Cfg<D>;
  CUtensorMap tmQ, tmK, tmV;
  int rc = make_tmap_3d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)q_width, (uint64_t)L, (uint64_t)B,
                        (uint64_t)q_width * 2, (uint64_t)L * q_width * 2, 64, BM, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  rc = make_tmap_3d(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)kv_width, (uint64_t)kv_rows, (uint64_t)B,
                    (uint64_t)kv_width * 2, (uint64_t)kv_rows * kv_width * 2, 64, BN, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  rc = make_tmap_3d(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)kv_width, (uint64_t)kv_rows, (uint64_t)B,
                    (uint64_t)kv_width * 2, (uint64_t)kv_rows * kv_width * 2, 64, BN, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  // share of the exponentials on the FMA pipe (eighths): B200_FA_POLY overrides the default for experiments
  static int poly8 = -1;
  if (poly8 < 0) {
    const char* e = getenv("B200_FA_POLY");
    poly8 = e ? atoi(e) : kDefaultPoly8;
    if (poly8 != 0 && poly8 != 2 && poly8 != 3 && poly8 != 4) poly8 = kDefaultPoly8;
  }
  void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, FwdParams, unsigned int*) =
      poly8 == 0 ? flash_fwd_kernel<D, 0> : poly8 == 3 ? flash_fwd_kernel<D, 3> : poly8 == 4 ? flash_fwd_kernel<D, 4>
                                                                                              : flash_fwd_kernel<D, 2>;
  static bool attr = false;
  if (!attr) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    attr = true;
  }
  FwdParams p{(__nv_bfloat16*)out, lse, B, L, H, Hkv, 1.0f / sqrtf((float)D), q_off, colQ0, colK0, colV0};
  dim3 grid(H * B, (L + BM - 1) / BM);
  kern<<<grid, NTHREADS, C::SMEM_BYTES, st>>>(tmQ, tmK, tmV, p, device_err_word());
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace fa
}  // namespace b200

extern "C" int b200_flash_attn_fwd(const void* qkv, void* out, float* lse, int B, int L, int H, int Hkv, int D,
                                   cudaStream_t st) {
  using namespace b200;
  if (!qkv || !out || B <= 0 || L <= 0 || H <= 0 || Hkv <= 0 || (H % Hkv) != 0) return B200_ERR_ARG;
  const long long width = (long long)(H + 2 * Hkv) * D;
  if (D == 64)
    return fa::launch_fwd<64>(qkv, width, 0, qkv, qkv, width, H * D, (H + Hkv) * D, L, out, lse, B, L, 0, H, Hkv, st);
  if (D == 128)
    return fa::launch_fwd<128>(qkv, width, 0, qkv, qkv, width, H * D, (H + Hkv) * D, L, out, lse, B, L, 0, H, Hkv, st);
  return B200_ERR_ARG;
}

// Chunked prefill against a key / value cache. qkv [B*L, (H + 2*Hkv)*D]: this chunk's projections (its K / V columns
// are NOT read: the caller has copied them into the caches first). k_cache, v_cache [B, cache_rows, Hkv*D] bf16 with
// row p = sequence position p, valid (and finite: allocate the caches zeroed) for p < q_off + L. The chunk's queries
// are positions q_off .. q_off + L - 1 and see keys <= their own position. out [B*L, H*D], lse [H, B*L] (may be null).
extern "C" int b200_flash_attn_fwd_cached(const void* qkv, const void* k_cache, const void* v_cache, long long cache_rows,
                                          void* out, float* lse, int B, int L, int q_off, int H, int Hkv, int D,
                                          cudaStream_t st) {
  using namespace b200;
  if (!qkv || !k_cache || !v_cache || !out || B <= 0 || L <= 0 || q_off < 0 || H <= 0 || Hkv <= 0 || (H % Hkv) != 0 ||
      cache_rows < (long long)q_off + L)
    return B200_ERR_ARG;
  const long long width = (long long)(H + 2 * Hkv) * D, kvw = (long long)Hkv * D;
  if (D == 64)
    return fa::launch_fwd<64>(qkv, width, 0, k_cache, v_cache, kvw, 0, 0, cache_rows, out, lse, B, L, q_off, H, Hkv, st);
  if (D == 128)
    return fa::launch_fwd<128>(qkv, width, 0, k_cache, v_cache, kvw, 0, 0, cache_rows, out, lse, B, L, q_off, H, Hkv, st);
  return B200_ERR_ARG;
}
