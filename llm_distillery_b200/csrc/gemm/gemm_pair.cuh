// Two-SM variant of the tcgen05 GEMM mainloop: a cluster of two CTAs works on one 256 x 256 output tile with
// tcgen05.mma.cta_group::2. Each CTA TMA-loads its own 128 rows of A and its own 128-row half of B (no multicast:
// the pair MMA reads both halves), so every SM fills and reads half the B bytes of the one-SM kernel - which is what
// the shared-memory pipe was saturated by - and the ring holds 6 stages instead of 4.
//
//   rank 0 (leader): TMA producer, MMA issuer (256 x 256 x 16 per instruction), 4 epilogue warps for rows 0-127
//   rank 1         : TMA producer,                                              4 epilogue warps for rows 128-255
// Barriers: "full" lives in the leader (both CTAs' TMA bytes are credited there); "empty" and "accumulator full" are
// per CTA and are released by tcgen05.commit multicast to both; "accumulator empty" lives in the leader and is
// arrived on by all 8 epilogue warps (the peer's through its cluster address). Epilogue functors are the same as for
// the one-SM kernel (gemm_core.cuh).
//
// Split-K (k_splits > 1, epilogues with SPLIT_K only): a work unit is (slice of the K loop, tile), slice-major, so
// the pairs that run side by side work on the same K window of neighbouring tiles. The slices of one tile are added
// into C in the order of their index: slice s of a tile waits until a counter in global memory says that slice s - 1
// has been added (8 counters per tile, one per epilogue warp of the pair, because each warp owns its own rows), adds,
// and releases the counter; the last slice sets it back to zero for the next launch. The order of the additions is
// therefore fixed and the result repeats bit for bit, which atomic adds did not give. Units are handed out in
// increasing order and all CTAs of the grid are resident, so the unit a slice waits for is always running or done.
#pragma once
#include "gemm_core.cuh"

namespace b200 {
namespace gemm {

constexpr int PAIR_BM = 256;  // rows per tile pair
constexpr int PAIR_BN = 256;
constexpr int PAIR_HALF_N = 128;

template <int STAGES>
struct SmemPair {
  static constexpr int A_BYTES = BM * BK * 2;           // 128 x 64
  static constexpr int B_BYTES = PAIR_HALF_N * BK * 2;  // 128 x 64
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int bytes(int epi_bytes) { return RING_BYTES + BAR_BYTES + epi_bytes + 1024; }
};

template <int STAGES, bool A_MN, bool B_MN, class Epi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                     int K, int fmt, typename Epi::Params ep, unsigned int* err_word, int k_splits,
                     unsigned int* split_sync, int b_half_stride) {
  using S = SmemPair<STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::RING_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_smem = smem + S::RING_BYTES + S::BAR_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  constexpr uint32_t TMEM_COLS = 2 * PAIR_BN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 2 * NUM_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before any remote arrive / pair TMA
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = (M + PAIR_BM - 1) / PAIR_BM;
  const int n_tiles = (N + PAIR_BN - 1) / PAIR_BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;
  // split-K: a work unit is (slice of the K loop, tile), slice-major. k_splits = 1: one unit per tile.
  const int num_units = num_tiles * k_splits;
  auto unit_range = [&](int unit, int& tile, int& kb0, int& kb1) {
    const int sp = unit / num_tiles;
    tile = unit - sp * num_tiles;
    kb0 = (int)((long long)num_kb * sp / k_splits);
    kb1 = (int)((long long)num_kb * (sp + 1) / k_splits);
  };
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  constexpr int GROUP_M = 8;
  auto tile_coords = [&](int tile, int& m_blk, int& n_blk) {
    const int per_group = GROUP_M * n_tiles;
    const int g = tile / per_group;
    const int first_m = g * GROUP_M;
    const int gsz = min(GROUP_M, m_tiles - first_m);
    const int r = tile - g * per_group;
    m_blk = first_m + (r % gsz);
    n_blk = r / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int unit = pair_id; ok && unit < num_units; unit += num_pairs) {
        int tile, kb0, kb1, m_blk, n_blk;
        unit_range(unit, tile, kb0, kb1);
        tile_coords(tile, m_blk, n_blk);
        const int m0 = m_blk * PAIR_BM + (int)cta * BM;
        // B rows of this CTA's half of the tile. b_half_stride > 0 (fused gate / up projection): the leader takes 128
        // rows of the first half of B and its peer the 128 rows that lie b_half_stride below them, so columns 0-127 of
        // the accumulator are the gate and columns 128-255 the up projection of the SAME 128 output features.
        const int n0 = b_half_stride > 0 ? n_blk * PAIR_HALF_N + (int)cta * b_half_stride
                                         : n_blk * PAIR_BN + (int)cta * PAIR_HALF_N;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, err_word, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          if (cta == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);  // both CTAs' bytes land here
          if constexpr (!A_MN) {
            tma_load_2d_pair(sA, &tmA, &full_bar[s], kb * BK, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d_pair(sA + i * (BK * 128), &tmA, &full_bar[s], m0 + i * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sB, &tmB, &full_bar[s], kb * BK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < PAIR_HALF_N / 64; ++i)
              tma_load_2d_pair(sB + i * (BK * 128), &tmB, &full_bar[s], n0 + i * 64, kb * BK);
          }
        }
      }
      // drain: the last commits must have released every stage before this CTA's shared memory goes away
      for (uint32_t d = 0; ok && d < (uint32_t)STAGES && d < it; ++d) {
        const uint32_t j = it - 1 - d;
        if (!mbar_wait_bounded(&empty_bar[j % STAGES], (j / STAGES) & 1u, abort_flag, err_word, ERR_WAIT_EMPTY)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && cta == 0) {
      const uint32_t idesc = make_idesc_f16(fmt, PAIR_BM, PAIR_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t a_lbo = A_MN ? BK * 128 : 16, a_kadv = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      constexpr uint32_t b_lbo = B_MN ? BK * 128 : 16, b_kadv = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      uint32_t it = 0, tl = 0;
      bool ok = true;
      for (int unit = pair_id; ok && unit < num_units; unit += num_pairs, ++tl) {
        int tile, kb0, kb1;
        unit_range(unit, tile, kb0, kb1);
        const uint32_t acc = tl & 1u;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait_bounded(&tempty_bar[acc], aph ^ 1u, abort_flag, err_word, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * PAIR_BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, err_word, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b_base = a_base + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(a_base + k * a_kadv, a_lbo, 1024);
            const uint64_t db = make_smem_desc_sw128(b_base + k * b_kadv, b_lbo, 1024);
            umma_f16_ss_pair(d_tmem, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s], 0x3);
        }
        if (ok) umma_commit_pair(&tfull_bar[acc], 0x3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (both CTAs)
    const int quad = warp & 3;
    const uint32_t leader_tempty0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    uint32_t tl = 0;
    for (int unit = pair_id; unit < num_units; unit += num_pairs, ++tl) {
      int tile, kb0, kb1, m_blk, n_blk;
      unit_range(unit, tile, kb0, kb1);
      tile_coords(tile, m_blk, n_blk);
      const uint32_t acc = tl & 1u;
      const uint32_t aph = (tl >> 1) & 1u;
      int ok = mbar_wait_bounded(&tfull_bar[acc], aph, abort_flag, err_word, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * PAIR_BN + (static_cast<uint32_t>(quad * 32) << 16);
      if constexpr (Epi::SPLIT_K) {
        if (k_splits > 1) {
          const int sp = unit / num_tiles;
          unsigned int* ctr = split_sync + (size_t)tile * 8 + cta * 4 + quad;
          if (sp > 0) {      // the slices before this one have been added
            int ok2 = 1;
            if (lane == 0) ok2 = wait_equal_bounded(ctr, (unsigned)sp, abort_flag, err_word, ERR_WAIT_AUX) ? 1 : 0;
            ok2 = __all_sync(0xffffffffu, ok2);
            if (!ok2) break;
          }
          Epi::tile(Epi::slice_params(ep, sp), taddr, m_blk * PAIR_BM + (int)cta * BM, n_blk * PAIR_BN, M, N, quad,
                    lane, epi_smem);
          __threadfence();
          __syncwarp();
          if (lane == 0) st_release_gpu_u32(ctr, sp + 1 == k_splits ? 0u : (unsigned)(sp + 1));
        } else {
          Epi::tile(ep, taddr, m_blk * PAIR_BM + (int)cta * BM, n_blk * PAIR_BN, M, N, quad, lane, epi_smem);
        }
      } else {
        Epi::tile(ep, taddr, m_blk * PAIR_BM + (int)cta * BM, n_blk * PAIR_BN, M, N, quad, lane, epi_smem);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty0 + acc * 8);
    }
  }

  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace b200
