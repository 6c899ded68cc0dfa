// Causal GQA flash-attention backward for sm_100a on tcgen05 tensor cores.
//
// One CTA owns one (batch, kv-head, 128-key block): K_j and V_j stay resident in shared memory, dK_j and dV_j
// accumulate in TMEM over every query head of the group and every query block at or after the diagonal, and
// are written once. dQ is produced per (query block, key block) pair, staged in shared memory and added into an fp32
// buffer by TMA reduce-add (whole 32-byte sectors per request instead of scattered per-thread atomics, which bound
// an earlier version of this kernel), then converted to bf16 by a small kernel.
//
// Per iteration (query head hq, query block i), five tcgen05.mma groups:
//   S  = Q_i K_j^T                 (A K-major, B K-major)        -> TMEM
//   dP = dO_i V_j^T                (A K-major, B K-major)        -> TMEM
//   softmax warps: P = exp2(S*c - lse), dS = P * (dP - delta) * scale, both written to smem in bf16
//   dV += P^T  dO_i                (A = P  read MN-major, B = dO MN-major)
//   dK += dS^T Q_i                 (A = dS read MN-major, B = Q  MN-major)
//   dQ  = dS   K_j                 (A = dS K-major,       B = K  MN-major)
// A [q x k] tile written row-per-thread in the 128B-swizzled K-major layout is, byte for byte, also the
// MN-major layout of its transpose, so P and dS are stored once and read both ways.
//
// Roles: warp 0 TMA producer (Q_i / dO_i ring); warps 1-4 issue the MMA groups, one group each (S and dP; dV; dK; dQ):
// every tcgen05 instruction - an MMA, a commit, a completed mbarrier wait - costs its issuing thread on the order of a
// hundred cycles here, so one thread issuing the 32 MMAs of a pair needed ~3.8 K cycles per pair and was what bound
// the kernel (the tensor core needs ~1.3 K); warps 5-20 softmax + dQ drain + epilogue: each TMEM lane quadrant is
// served by four warps that split the tile's columns.
// What bounds the kernel now is shared-memory bandwidth: a pair's MMAs read ~224 KB of operands from shared memory
// (every operand of the five groups lives there) next to ~100 KB of P / dS / dQ-staging traffic from the warps, at
// ~128 B per clock. Two variants measured no faster and were dropped: the next pair's S / dP MMAs issued ahead of
// this pair's dV / dK / dQ (0.654 against 0.648 ms at head dim 64), and dedicated dQ drain warps with packed f32x2
// softmax arithmetic (0.673 ms). Less operand traffic needs P^T / dS^T (and K, V) as TMEM operands, i.e. the
// transposed S^T = K Q^T formulation.
#include "../common/ptx.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace fab {

constexpr int BM = 128;  // queries per block
constexpr int BN = 128;  // keys per block
constexpr int NSPLIT = 4;        // softmax/drain warps per TMEM lane quadrant: each takes 1/4 of a tile's columns
constexpr int NISSUE = 4;                        // MMA-issuing warps: S/dP, dV, dK, dQ
constexpr int FIRST_WORK_WARP = 1 + NISSUE;      // warp 0 is the TMA producer
constexpr int NTHREADS = 32 * FIRST_WORK_WARP + 4 * NSPLIT * 32;  // + 16 softmax/drain warps
constexpr int NWORK = 4 * NSPLIT * 32;          // threads that arrive on the softmax/drain barriers

template <int D>
struct Cfg {
  static constexpr int STAGES = (D == 64) ? 2 : 1;
  static constexpr int KV_BYTES = BN * D * 2;   // one of K or V
  static constexpr int QDO_BYTES = BM * D * 2;  // one of Q or dO
  static constexpr int STAGE_BYTES = 2 * QDO_BYTES;
  static constexpr int P_BYTES = BM * BN * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = KV_BYTES;
  static constexpr int OFF_QDO = 2 * KV_BYTES;
  static constexpr int OFF_P = OFF_QDO + STAGES * STAGE_BYTES;
  static constexpr int OFF_DS = OFF_P + P_BYTES;
  static constexpr int OFF_DQS = OFF_DS + P_BYTES;  // dQ staging: two [128 x 32] fp32 sub-tiles, 128B-swizzled
  static constexpr int DQS_BYTES = 2 * BM * 128;
  static constexpr int OFF_BAR = OFF_DQS + DQS_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr bool ALIAS = (D == 128);  // dQ shares TMEM columns with S
  static constexpr uint32_t S_COL = 0;
  static constexpr uint32_t DP_COL = 128;
  static constexpr uint32_t DV_COL = 256;
  static constexpr uint32_t DK_COL = 256 + D;
  static constexpr uint32_t DQ_COL = ALIAS ? 0 : 256 + 2 * D;
  // head dim 64 leaves 64 TMEM columns free: a second dQ accumulator lets the pair loop run two pairs deep
  static constexpr bool PIPE = !ALIAS;
  static constexpr uint32_t DQ_COL1 = PIPE ? 256 + 3 * D : DQ_COL;
  static constexpr uint32_t TMEM_COLS = 512;
};

struct BwdParams {
  const float* lse;    // [H, T]
  const float* delta;  // [H, T]
  float* dq_acc;       // [T, H*D] fp32, zeroed by the launcher
  __nv_bfloat16* dqkv; // [T, (H+2Hkv)*D]
  int B, L, H, Hkv;
  float scale;
};

template <int D>
__global__ void __launch_bounds__(NTHREADS, 1)
    flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
                     const __grid_constant__ CUtensorMap tmDQ, BwdParams p, unsigned int* err_word) {
  using C = Cfg<D>;
  constexpr int ST = C::STAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* pds_ready = bars + 6;
  uint64_t* dq_full = bars + 7;
  uint64_t* dq_empty = bars + 8;
  uint64_t* stage_full = bars + 9;   // dQ staging tile written by the drain threads (all of them arrive)
  uint64_t* stage_free = bars + 10;  // ... and read out by the TMA reduce
  uint64_t* dq_full1 = bars + 11;    // second dQ accumulator (pipelined variant)
  uint64_t* dq_empty1 = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (p.L + BN - 1) / BN;
  // blockIdx.y = key block (block 0 has the most work), blockIdx.x = (kv head, batch): blocks are handed out x-fastest,
  // so all the heavy key blocks of every head start first and the light ones fill the tail
  const int jb = blockIdx.y;
  const int hkv = blockIdx.x % p.Hkv, b = blockIdx.x / p.Hkv;
  const int g = p.H / p.Hkv;
  const int kv0 = jb * BN;
  const int nqb = (p.L + BM - 1) / BM;
  const int i_start = kv0 / BM;
  const int nqi = nqb - i_start;
  const int n_it = g * nqi;
  const long long T = (long long)p.B * p.L;
  (void)nkb;

  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && err_word) atomicCAS(err_word, 0u, (unsigned)ERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQKV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmDQ);
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, NWORK);
    mbar_init(dq_full, 3);     // "pair done": the dV, dK and dQ issuers each commit to it
    mbar_init(dq_empty, NWORK);
    mbar_init(stage_full, NWORK);
    mbar_init(stage_free, 1);
    mbar_init(dq_full1, 3);
    mbar_init(dq_empty1, NWORK);
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

  const int colK = p.H * D + hkv * D;
  const int colV = (p.H + p.Hkv) * D + hkv * D;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * C::KV_BYTES);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_3d(smem + C::OFF_K + c * (BN * 128), &tmQKV, kv_full, colK + c * 64, kv0, b);
        tma_load_3d(smem + C::OFF_V + c * (BN * 128), &tmQKV, kv_full, colV + c * 64, kv0, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int s = it % ST;
        const uint32_t ph = (it / ST) & 1u;
        const int hq = hkv * g + it / nqi;
        const int q0 = (i_start + it % nqi) * BM;
        (void)ph;
        if (it >= ST) {
          // the stage was read by pair it - ST: free once that pair's dV, dK and dQ MMAs are done (the S / dP MMAs of a
          // pair complete before its softmax and so before these are even issued)
          const int pd = it - ST;
          uint64_t* done = (C::PIPE && (pd & 1)) ? dq_full1 : dq_full;
          const uint32_t par = C::PIPE ? ((pd >> 1) & 1u) : (pd & 1u);
          if (!mbar_spin_bounded(done, par, abort_flag, err_word, ERR_WAIT_EMPTY)) break;
        }
        uint8_t* sQ = smem + C::OFF_QDO + s * C::STAGE_BYTES;
        uint8_t* sDO = sQ + C::QDO_BYTES;
        mbar_arrive_expect_tx(&qdo_full[s], C::STAGE_BYTES);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_3d(sQ + c * (BM * 128), &tmQKV, &qdo_full[s], hq * D + c * 64, q0, b);
          tma_load_3d(sDO + c * (BM * 128), &tmDO, &qdo_full[s], hq * D + c * 64, q0, b);
        }
      }
    }
  } else if (warp < FIRST_WORK_WARP) {
    // ------------------------------------------------------------------ MMA issuers (one elected thread per warp)
    if (lane == 0) {
      const uint32_t sK = smem_u32(smem + C::OFF_K);
      const uint32_t sV = smem_u32(smem + C::OFF_V);
      const uint32_t sP = smem_u32(smem + C::OFF_P);
      const uint32_t sDS = smem_u32(smem + C::OFF_DS);
      // Base descriptors, built once: inside the loops an MMA's operands are a base plus a constant (k-step) and a
      // stage offset. The address field counts 16-byte units and never carries out of its 14 bits below 256 KB.
      const uint32_t sQ0 = smem_u32(smem + C::OFF_QDO), sDO0 = sQ0 + C::QDO_BYTES;
      auto koff = [](int k) -> uint64_t {   // k-step inside a K-major tile: 64-column sub-tiles 16 KB apart, 32 B per step
        return static_cast<uint64_t>(((k >> 2) * (128 * 128) + (k & 3) * 32) >> 4);
      };
      auto stage_off = [](int it) -> uint64_t { return static_cast<uint64_t>(((it % ST) * C::STAGE_BYTES) >> 4); };
      // "pair done" barrier of pair `it` (count 3) and the parity of its phase
      auto pair_bar = [&](int it) -> uint64_t* { return (C::PIPE && (it & 1)) ? dq_full1 : dq_full; };
      if (warp == 1) {
        // S = Q K^T and dP = dO V^T (both operands K-major) -> TMEM. Pair it + 1 is issued as soon as the softmax warps
        // have read S / dP of pair it, i.e. AHEAD of pair it's dV / dK / dQ, which the other issuers handle.
        const uint32_t idesc_kk = make_idesc_f16(1, BM, BN, 0, 0);
        const uint64_t kQ = make_smem_desc_sw128(sQ0, 16, 1024), kDO = make_smem_desc_sw128(sDO0, 16, 1024);
        const uint64_t kK = make_smem_desc_sw128(sK, 16, 1024), kV = make_smem_desc_sw128(sV, 16, 1024);
        bool ok = mbar_spin_bounded(kv_full, 0, abort_flag, err_word, ERR_WAIT_FULL);
        for (int it = 0; ok && it < n_it; ++it) {
          if (!mbar_spin_bounded(&qdo_full[it % ST], (it / ST) & 1u, abort_flag, err_word, ERR_WAIT_FULL)) break;
          if (it > 0) {
            if constexpr (C::PIPE) {
              if (!mbar_spin_bounded(pds_ready, (it - 1) & 1u, abort_flag, err_word, ERR_WAIT_AUX)) break;
            } else {  // dQ shares its TMEM columns with S: they are free when the drain of pair it - 1 is through
              if (!mbar_spin_bounded(dq_empty, (it - 1) & 1u, abort_flag, err_word, ERR_WAIT_AUX)) break;
            }
          }
          tc_fence_after_sync();
          const uint64_t stage = stage_off(it);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_f16_ss(tmem_base + C::S_COL, kQ + stage + koff(k), kK + koff(k), idesc_kk, k != 0 ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_f16_ss(tmem_base + C::DP_COL, kDO + stage + koff(k), kV + koff(k), idesc_kk, k != 0 ? 1u : 0u);
          umma_commit(sdp_full);
        }
      } else if (warp == 2 || warp == 3) {
        // dV += P^T dO (warp 2) ; dK += dS^T Q (warp 3): reduction over the 128 queries, 16 per step = 2048 B per step
        // in both tiles, both operands MN-major
        const uint32_t idesc_tt = make_idesc_f16(1, BN, D, 1, 1);
        const uint64_t tA = make_smem_desc_sw128(warp == 2 ? sP : sDS, BM * 128, 1024);
        const uint64_t tB = make_smem_desc_sw128(warp == 2 ? sDO0 : sQ0, BM * 128, 1024);
        const uint32_t dcol = tmem_base + (warp == 2 ? C::DV_COL : C::DK_COL);
        for (int it = 0; it < n_it; ++it) {
          if (!mbar_spin_bounded(pds_ready, it & 1u, abort_flag, err_word, ERR_WAIT_AUX)) break;
          tc_fence_after_sync();
          const uint64_t stage = stage_off(it);
          if (it == 0) {
#pragma unroll
            for (int k = 0; k < BM / 16; ++k)
              umma_f16_ss(dcol, tA + (uint64_t)(k * 128), tB + stage + (uint64_t)(k * 128), idesc_tt, k != 0 ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < BM / 16; ++k)
              umma_f16_ss(dcol, tA + (uint64_t)(k * 128), tB + stage + (uint64_t)(k * 128), idesc_tt, 1u);
          }
          umma_commit(pair_bar(it));
        }
      } else {
        // dQ = dS K (reduction over the 128 keys; dS K-major, K MN-major) into the pair's accumulator
        const uint32_t idesc_kt = make_idesc_f16(1, BM, D, 0, 1);
        const uint64_t kDS = make_smem_desc_sw128(sDS, 16, 1024);
        const uint64_t tK = make_smem_desc_sw128(sK, BN * 128, 1024);
        bool ok = mbar_spin_bounded(kv_full, 0, abort_flag, err_word, ERR_WAIT_FULL);
        for (int it = 0; ok && it < n_it; ++it) {
          if (!mbar_spin_bounded(pds_ready, it & 1u, abort_flag, err_word, ERR_WAIT_AUX)) break;
          uint32_t dq_col = C::DQ_COL;
          if constexpr (C::PIPE) {
            dq_col = (it & 1) ? C::DQ_COL1 : C::DQ_COL;
            if (it >= 2) {  // the drain of pair it-2 has emptied this accumulator
              if (!mbar_spin_bounded((it & 1) ? dq_empty1 : dq_empty, ((it >> 1) - 1) & 1u, abort_flag, err_word,
                                     ERR_WAIT_AUX))
                break;
            }
          }
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < BN / 16; ++k)
            umma_f16_ss(tmem_base + dq_col, kDS + koff(k), tK + (uint64_t)(k * 128), idesc_kt, k != 0 ? 1u : 0u);
          umma_commit(pair_bar(it));
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int part = (warp - FIRST_WORK_WARP) >> 2;  // which quarter of the columns this warp handles
    const int r = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const float c2 = p.scale * 1.4426950408889634f;
    uint8_t* sP = smem + C::OFF_P;
    uint8_t* sDS = smem + C::OFF_DS;
    constexpr int DW = D / NSPLIT;     // columns of dQ / dK / dV per warp: 16 (D = 64) or 32 (D = 128)
    constexpr int ROUNDS = D / 64;     // the dQ staging area holds two 32-column sub-tiles per round
    const int dc0 = part * DW;         // first dQ / dK / dV column of this warp
    bool ok = true;
    uint32_t rd = 0;  // staging rounds so far
    uint8_t* sDQ = smem + C::OFF_DQS;
    const int st = dc0 >> 5;               // 32-column sub-tile of dQ this warp contributes to
    const int chunkbase = (dc0 & 31) >> 2;  // first 16-byte chunk (4 floats) inside the 128-byte row
    // Drain the dQ accumulator of pair `itd` into the fp32 gradient: TMEM -> registers -> swizzled staging tile in
    // shared memory (row r, 128-byte rows of 32 floats) -> TMA reduce-add issued by one thread. The staging area holds
    // two 32-column sub-tiles: D = 128 takes two rounds, and in each round only the warps whose columns belong to
    // that round write (everybody arrives on the barriers). The caller has waited for the pair's dq_full barrier.
    auto drain = [&](int itd) {
      const int hq = hkv * g + itd / nqi;
      const int q0 = (i_start + itd % nqi) * BM;
      const uint32_t dq_col = (C::PIPE && (itd & 1)) ? C::DQ_COL1 : C::DQ_COL;
      uint32_t v[DW];
      if constexpr (DW == 32) tmem_ld_32x32b_x32(tmem_base + lane_addr + dq_col + dc0, v);
      else tmem_ld_32x32b_x16(tmem_base + lane_addr + dq_col + dc0, v);
      tmem_ld_wait();
#pragma unroll
      for (int rr = 0; rr < ROUNDS; ++rr) {
        // the previous round's reduce must have finished READING the staging tile. The thread that issued it checks
        // that only now, a whole softmax phase later, so that the TMA engine's latency is off the critical path.
        if (warp == FIRST_WORK_WARP && lane == 0 && rd > 0) {
          tma_store_wait_read0();
          mbar_arrive(stage_free);
        }
        __syncwarp();
        if (rd > 0) {
          int w3 = mbar_wait_bounded(stage_free, (rd - 1) & 1u, abort_flag, err_word, ERR_WAIT_AUX) ? 1 : 0;
          if (!__all_sync(0xffffffffu, w3)) { ok = false; break; }
        }
        if ((st >> 1) == rr) {
          uint8_t* rowp = sDQ + (st & 1) * (BM * 128) + r * 128;
#pragma unroll
          for (int q4 = 0; q4 < DW / 4; ++q4)
            *reinterpret_cast<uint4*>(rowp + (((chunkbase + q4) ^ (r & 7)) * 16)) =
                make_uint4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
        }
        fence_proxy_async_smem();
        mbar_arrive(stage_full);
        if (warp == FIRST_WORK_WARP && lane == 0) {
          if (mbar_wait_bounded(stage_full, rd & 1u, abort_flag, err_word, ERR_WAIT_AUX)) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
              tma_reduce_add_3d(&tmDQ, sDQ + hh * (BM * 128), hq * D + (rr * 2 + hh) * 32, q0, b);
            tma_store_commit();
          }
        }
        __syncwarp();
        ++rd;
      }
      if (ok) {
        tc_fence_before_sync();
        mbar_arrive((C::PIPE && (itd & 1)) ? dq_empty1 : dq_empty);
      }
    };
    // dq_full of pair itd: one barrier per accumulator, each used by every second pair in the pipelined variant
    auto wait_dq_full = [&](int itd) -> bool {
      uint64_t* bar = (C::PIPE && (itd & 1)) ? dq_full1 : dq_full;
      const uint32_t parity = C::PIPE ? ((itd >> 1) & 1u) : (itd & 1u);
      int w2 = mbar_wait_bounded(bar, parity, abort_flag, err_word, ERR_WAIT_AUX) ? 1 : 0;
      if (!__all_sync(0xffffffffu, w2)) return false;
      tc_fence_after_sync();
      return true;
    };
    for (int it = 0; ok && it < n_it; ++it) {
      const int hq = hkv * g + it / nqi;
      const int q0 = (i_start + it % nqi) * BM;
      const int qi = q0 + r;
      const bool row_ok = qi < p.L;
      const long long t = (long long)b * p.L + qi;
      // a row past the end of the sequence gets lse = +inf: exp2(s - inf) = 0, so P and dS vanish without a mask
      const float lse2 = row_ok ? p.lse[(long long)hq * T + t] * 1.4426950408889634f : INFINITY;
      const float dlts = row_ok ? p.delta[(long long)hq * T + t] * p.scale : 0.f;
      const bool diag = (kv0 + BN - 1) > q0;
      const int lim = diag ? (qi - kv0) : 0x7fffffff;  // tile columns <= lim are visible to this row
      int w = mbar_wait_bounded(sdp_full, it & 1u, abort_flag, err_word, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
      tc_fence_after_sync();
      // this warp's 32 columns of S and dP, 16 at a time (keeps the register count under the 18-warp budget)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int col0 = part * 32 + hf * 16;
        uint32_t sv[16], dv[16];
        tmem_ld_32x32b_x16(tmem_base + lane_addr + C::S_COL + col0, sv);
        tmem_ld_32x32b_x16(tmem_base + lane_addr + C::DP_COL + col0, dv);
        tmem_ld_wait();
        uint32_t pkP[8], pkS[8];
        if (!diag) {
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(sv[e]), c2, -lse2));
            const float p1 = fast_exp2(fmaf(__uint_as_float(sv[e + 1]), c2, -lse2));
            const float d0 = p0 * fmaf(__uint_as_float(dv[e]), p.scale, -dlts);
            const float d1 = p1 * fmaf(__uint_as_float(dv[e + 1]), p.scale, -dlts);
            pkP[e >> 1] = pack_bf16x2(p0, p1);
            pkS[e >> 1] = pack_bf16x2(d0, d1);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            float p0 = fast_exp2(fmaf(__uint_as_float(sv[e]), c2, -lse2));
            float p1 = fast_exp2(fmaf(__uint_as_float(sv[e + 1]), c2, -lse2));
            if ((col0 + e) > lim) p0 = 0.f;
            if ((col0 + e + 1) > lim) p1 = 0.f;
            const float d0 = p0 * fmaf(__uint_as_float(dv[e]), p.scale, -dlts);
            const float d1 = p1 * fmaf(__uint_as_float(dv[e + 1]), p.scale, -dlts);
            pkP[e >> 1] = pack_bf16x2(p0, p1);
            pkS[e >> 1] = pack_bf16x2(d0, d1);
          }
        }
        if (C::PIPE && hf == 0 && it > 0) {
          // P / dS in shared memory still belong to pair it-1 until its dV / dK / dQ MMAs are done (they were issued
          // behind this pair's S / dP MMAs); the first 16 columns above were computed while waiting for that
          if (!wait_dq_full(it - 1)) { ok = false; break; }
        }
        // columns col0 .. col0+15 of row r: 64-column sub-tile col0/64, 16-byte chunks (col0 % 64)/8 + {0, 1}
        const int sub = col0 >> 6;
        const int chunk0 = (col0 & 63) >> 3;
        const int off = sub * (BM * 128) + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 2; ++q4) {
          const int ch = (chunk0 + q4) ^ (r & 7);
          *reinterpret_cast<uint4*>(sP + off + ch * 16) =
              make_uint4(pkP[q4 * 4], pkP[q4 * 4 + 1], pkP[q4 * 4 + 2], pkP[q4 * 4 + 3]);
          *reinterpret_cast<uint4*>(sDS + off + ch * 16) =
              make_uint4(pkS[q4 * 4], pkS[q4 * 4 + 1], pkS[q4 * 4 + 2], pkS[q4 * 4 + 3]);
        }
      }
      if (!ok) break;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(pds_ready);
      if constexpr (C::PIPE) {
        if (it > 0) drain(it - 1);   // its dq_full was waited for above
      } else {
        if (!wait_dq_full(it)) { ok = false; break; }
        drain(it);
      }
    }
    if (C::PIPE && ok && n_it > 0) {   // the last pair's dQ; this wait also covers every MMA of the CTA
      if (wait_dq_full(n_it - 1)) drain(n_it - 1);
      else ok = false;
    }
    if (warp == FIRST_WORK_WARP && lane == 0) tma_store_wait_all0();
    // epilogue: dK_j, dV_j (thread = key row). The last dq_full wait covered every MMA of this CTA.
    if (ok && n_it > 0) {
      const int kvi = kv0 + r;
      const bool row_ok = kvi < p.L;
      const long long width = (long long)(p.H + 2 * p.Hkv) * D;
      __nv_bfloat16* krow = p.dqkv + ((long long)b * p.L + kvi) * width + colK;
      __nv_bfloat16* vrow = p.dqkv + ((long long)b * p.L + kvi) * width + colV;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t col = which == 0 ? C::DK_COL : C::DV_COL;
        __nv_bfloat16* dst = which == 0 ? krow : vrow;
        uint32_t v[DW];
        if constexpr (DW == 32) tmem_ld_32x32b_x32(tmem_base + lane_addr + col + dc0, v);
        else tmem_ld_32x32b_x16(tmem_base + lane_addr + col + dc0, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q4 = 0; q4 < DW / 8; ++q4) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[q4 * 8 + 0]), __uint_as_float(v[q4 * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2]), __uint_as_float(v[q4 * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(v[q4 * 8 + 4]), __uint_as_float(v[q4 * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(v[q4 * 8 + 6]), __uint_as_float(v[q4 * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + dc0 + q4 * 8) = o;
          }
        }
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

// delta[h, t] = sum_d dout[t, h*D + d] * out[t, h*D + d]; one group of D/8 lanes per (t, h).
template <int D>
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                             float* __restrict__ delta, long long T, int H) {
  constexpr int LPG = D / 8;  // lanes per (t,h)
  const long long gid = (blockIdx.x * (long long)blockDim.x + threadIdx.x);
  const long long grp = gid / LPG;
  const int sub = (int)(gid % LPG);
  float s = 0.f;
  const bool ok = grp < T * H;
  long long t = 0;
  int h = 0;
  if (ok) {
    t = grp / H;
    h = (int)(grp - t * H);
    const size_t off = (size_t)t * H * D + (size_t)h * D + sub * 8;
    uint4 a = *reinterpret_cast<const uint4*>(dout + off);
    uint4 b = *reinterpret_cast<const uint4*>(out + off);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
      s += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int o = LPG / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (ok && sub == 0) delta[(size_t)h * T + t] = s;
}

// dqkv[t, 0:H*D] = bf16(dq_acc[t, :])
__global__ void dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv, long long T, int HD,
                                  long long width) {
  const int hv = HD >> 3;
  const long long total = T * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / hv;
    const int v = (int)(i - t * hv);
    const float4 a = reinterpret_cast<const float4*>(acc + t * HD)[2 * v];
    const float4 b = reinterpret_cast<const float4*>(acc + t * HD)[2 * v + 1];
    uint4 o;
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(a.z, a.w);
    o.z = pack_bf16x2(b.x, b.y);
    o.w = pack_bf16x2(b.z, b.w);
    reinterpret_cast<uint4*>(dqkv + t * width)[v] = o;
  }
}

// The same with the inverse rotary embedding of the query heads applied on the way: one thread takes the two 8-element
// vectors that the rotation pairs (i and i + D/2 of a head), rounds them to bf16 first - what the stand-alone rope
// kernel would read back - and rotates with that kernel's expressions, so the result is bit-identical to convert + rope.
__global__ void dq_convert_rope_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv,
                                       const int* __restrict__ pos, const float* __restrict__ cs,
                                       const float* __restrict__ sn, long long T, int H, int D, long long width) {
  const int half = D >> 1;
  const int vph = half >> 3;                 // vector pairs per head
  const int vpt = H * vph;
  const long long total = T * vpt;
  const int HD = H * D;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vpt;
    const int r = (int)(i - t * vpt);
    const int hd = r / vph;
    const int j = (r - hd * vph) * 8;
    const float* a = acc + t * HD + (long long)hd * D + j;
    const float4 a0 = reinterpret_cast<const float4*>(a)[0], a1 = reinterpret_cast<const float4*>(a)[1];
    const float4 b0 = reinterpret_cast<const float4*>(a + half)[0], b1 = reinterpret_cast<const float4*>(a + half)[1];
    const float fa_in[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float fb_in[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    const int p = pos[t];
    const float4 c0 = *reinterpret_cast<const float4*>(cs + (size_t)p * half + j);
    const float4 c1 = *reinterpret_cast<const float4*>(cs + (size_t)p * half + j + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sn + (size_t)p * half + j);
    const float4 s1 = *reinterpret_cast<const float4*>(sn + (size_t)p * half + j + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sg[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float oa[8], ob[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float fa = __bfloat162float(__float2bfloat16(fa_in[k]));
      const float fb = __bfloat162float(__float2bfloat16(fb_in[k]));
      const float sk = sg[k] * -1.f;                       // the transposed rotation
      oa[k] = __fmaf_rn(fa, c[k], -__fmul_rn(fb, sk));
      ob[k] = __fmaf_rn(fb, c[k], __fmul_rn(fa, sk));
    }
    uint4 o1, o2;
    o1.x = pack_bf16x2(oa[0], oa[1]); o1.y = pack_bf16x2(oa[2], oa[3]);
    o1.z = pack_bf16x2(oa[4], oa[5]); o1.w = pack_bf16x2(oa[6], oa[7]);
    o2.x = pack_bf16x2(ob[0], ob[1]); o2.y = pack_bf16x2(ob[2], ob[3]);
    o2.z = pack_bf16x2(ob[4], ob[5]); o2.w = pack_bf16x2(ob[6], ob[7]);
    __nv_bfloat16* dst = dqkv + t * width + (long long)hd * D + j;
    *reinterpret_cast<uint4*>(dst) = o1;
    *reinterpret_cast<uint4*>(dst + half) = o2;
  }
}

template <int D>
static int launch_bwd(const void* dout, const void* qkv, const void* out, const float* lse, float* delta, void* dqkv,
                      float* dq_acc, int B, int L, int H, int Hkv, const int* pos, const float* cos_tab,
                      const float* sin_tab, cudaStream_t st) {
  using C = Cfg<D>;
  const long long width = (long long)(H + 2 * Hkv) * D;
  const long long T = (long long)B * L;
  const long long HD = (long long)H * D;
  CUtensorMap tmQKV, tmDO;
  int rc = make_tmap_3d(&tmQKV, qkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)width, (uint64_t)L, (uint64_t)B,
                        (uint64_t)width * 2, (uint64_t)L * width * 2, 64, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  rc = make_tmap_3d(&tmDO, dout, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)HD, (uint64_t)L, (uint64_t)B,
                    (uint64_t)HD * 2, (uint64_t)L * HD * 2, 64, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  CUtensorMap tmDQ;
  rc = make_tmap_3d(&tmDQ, dq_acc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)HD, (uint64_t)L, (uint64_t)B,
                    (uint64_t)HD * 4, (uint64_t)L * HD * 4, 32, 128, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  {
    const long long threads = T * H * (D / 8);
    delta_kernel<D><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)dout,
                                                                      (const __nv_bfloat16*)out, delta, T, H);
    B200_CUDA_CHECK(cudaGetLastError());
  }
  B200_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, (size_t)T * HD * sizeof(float), st));
  auto kern = flash_bwd_kernel<D>;
  static bool attr = false;
  if (!attr) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    attr = true;
  }
  BwdParams p{lse, delta, dq_acc, (__nv_bfloat16*)dqkv, B, L, H, Hkv, 1.0f / sqrtf((float)D)};
  dim3 grid(Hkv * B, (L + BN - 1) / BN);
  kern<<<grid, NTHREADS, C::SMEM_BYTES, st>>>(tmQKV, tmDO, tmDQ, p, device_err_word());
  B200_CUDA_CHECK(cudaGetLastError());
  {
    const bool rot = pos != nullptr;
    long long work = rot ? T * (HD >> 4) : T * (HD >> 3);
    long long blocks = (work + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (rot)
      dq_convert_rope_kernel<<<(unsigned)blocks, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dqkv, pos, cos_tab, sin_tab, T, H,
                                                              D, width);
    else
      dq_convert_kernel<<<(unsigned)blocks, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dqkv, T, (int)HD, width);
    B200_CUDA_CHECK(cudaGetLastError());
  }
  return B200_OK;
}

}  // namespace fab
}  // namespace b200

// dq_acc: fp32 scratch [T, H*D] (zeroed here); delta: fp32 scratch [H, T]. dqkv receives dQ | dK | dV.
extern "C" int b200_flash_attn_bwd(const void* dout, const void* qkv, const void* out, const float* lse, float* delta,
                                   void* dqkv, float* dq_acc, int B, int L, int H, int Hkv, int D, cudaStream_t st) {
  using namespace b200;
  if (!dout || !qkv || !out || !lse || !delta || !dqkv || !dq_acc || B <= 0 || L <= 0 || H <= 0 || Hkv <= 0 ||
      (H % Hkv) != 0)
    return B200_ERR_ARG;
  if (D == 64) return fab::launch_bwd<64>(dout, qkv, out, lse, delta, dqkv, dq_acc, B, L, H, Hkv, nullptr, nullptr, nullptr, st);
  if (D == 128)
    return fab::launch_bwd<128>(dout, qkv, out, lse, delta, dqkv, dq_acc, B, L, H, Hkv, nullptr, nullptr, nullptr, st);
  return B200_ERR_ARG;
}

// The same, with the inverse rotary embedding of the QUERY heads applied where the fp32 dQ accumulator is converted to
// bf16 (pos int32 [B*L]; cos / sin fp32 [max_pos, D/2]). The key heads' gradient comes out of the main kernel's epilogue
// and is rotated by the caller.
extern "C" int b200_flash_attn_bwd_rope(const void* dout, const void* qkv, const void* out, const float* lse,
                                        float* delta, void* dqkv, float* dq_acc, const int* pos, const float* cos_tab,
                                        const float* sin_tab, int B, int L, int H, int Hkv, int D, cudaStream_t st) {
  using namespace b200;
  if (!dout || !qkv || !out || !lse || !delta || !dqkv || !dq_acc || !pos || !cos_tab || !sin_tab || B <= 0 || L <= 0 ||
      H <= 0 || Hkv <= 0 || (H % Hkv) != 0)
    return B200_ERR_ARG;
  if (D == 64) return fab::launch_bwd<64>(dout, qkv, out, lse, delta, dqkv, dq_acc, B, L, H, Hkv, pos, cos_tab, sin_tab, st);
  if (D == 128)
    return fab::launch_bwd<128>(dout, qkv, out, lse, delta, dqkv, dq_acc, B, L, H, Hkv, pos, cos_tab, sin_tab, st);
  return B200_ERR_ARG;
}

// The conversion pass alone (fp32 dQ accumulator -> bf16 query columns of dqkv with the inverse rotation): exported so
// that its bit-exactness against convert + rope kernel can be tested on a given accumulator.
extern "C" int b200_dq_convert_rope(const float* acc, void* dqkv, const int* pos, const float* cos_tab,
                                    const float* sin_tab, long long T, int H, int D, long long width, cudaStream_t st) {
  using namespace b200;
  if (!acc || !dqkv || !pos || !cos_tab || !sin_tab || T <= 0 || H <= 0 || (D != 64 && D != 128)) return B200_ERR_ARG;
  long long work = T * ((long long)H * D >> 4);
  long long blocks = (work + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  fab::dq_convert_rope_kernel<<<(unsigned)blocks, 256, 0, st>>>(acc, (__nv_bfloat16*)dqkv, pos, cos_tab, sin_tab, T, H, D,
                                                              width);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
