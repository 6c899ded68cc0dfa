// Persistent, warp-specialised tcgen05 GEMM mainloop for sm_100a, shared by every GEMM-shaped
// kernel in this tree (plain GEMMs, the LM-head log-sum-exp/gather head, the distillation dlogits pass).
//
//   D[M,N] (fp32, TMEM) = A[M,K] * B[N,K]^T        bf16 or fp16 operands
//
// Roles inside one 192-thread CTA (one CTA per SM, static persistent tile loop):
//   warp 0    : TMA producer  - one lane issues cp.async.bulk.tensor loads into a STAGES-deep smem ring
//   warp 1    : MMA issuer    - one lane issues tcgen05.mma (128 x BN x 16) and tcgen05.commit
//   warps 2-5 : epilogue      - read the fp32 accumulator from TMEM (tcgen05.ld) and run Epi::tile()
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i overlaps
// the mainloop of tile i+1. No TMA load uses cluster multicast.
//
// Operand layouts. "K-major" means the reduction dimension is contiguous in global memory
// (A stored [M,K], B stored [N,K]); "MN-major" means the M (or N) dimension is contiguous
// (A stored [K,M], B stored [K,N]). Both are fed to the tensor core without a transpose pass:
// the smem tile is whatever a 128B-swizzled TMA box writes and the matrix descriptor names the layout.
#pragma once
#include "../common/ptx.cuh"

namespace b200 {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;      // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;  // K per tcgen05.mma for 16-bit operands
constexpr int NUM_THREADS = 192;
constexpr int NUM_EPI_WARPS = 4;

struct DescCfg {
  // Byte offsets used to build the shared-memory matrix descriptors (see make_smem_desc_sw128).
  uint32_t a_lbo, a_sbo, a_kadv;  // kadv: start-address advance per UMMA_K step
  uint32_t b_lbo, b_sbo, b_kadv;
};

template <int BN, bool A_MN, bool B_MN>
__host__ __device__ constexpr DescCfg default_desc_cfg() {
  DescCfg c{};
  // K-major, SW128: rows are 128 B, 8-row groups 1024 B apart; K advances inside the swizzle row.
  // MN-major, SW128: k-rows are 128 B (64 MN elements), 8-k groups 1024 B apart, 64-wide MN chunks
  // BK*128 B apart; K advances by UMMA_K rows.
  c.a_lbo = A_MN ? BK * 128 : 16;
  c.a_sbo = 1024;
  c.a_kadv = A_MN ? UMMA_K * 128 : UMMA_K * 2;
  c.b_lbo = B_MN ? BK * 128 : 16;
  c.b_sbo = 1024;
  c.b_kadv = B_MN ? UMMA_K * 128 : UMMA_K * 2;
  return c;
}

template <int BN, int STAGES>
struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = 256;
  // 1024 B of slack so the ring can be aligned to the swizzle period.
  static constexpr int bytes(int epi_bytes) { return RING_BYTES + BAR_BYTES + epi_bytes + 1024; }
};

// Tile order: groups of GROUP_M row-tiles sweep all column tiles, so concurrently running CTAs
// share A and B tiles through L2.
struct TileMap {
  int m_tiles, n_tiles, num_tiles, group_m;
  __device__ __forceinline__ void init(int M, int N, int BN, int group) {
    m_tiles = (M + BM - 1) / BM;
    n_tiles = (N + BN - 1) / BN;
    num_tiles = m_tiles * n_tiles;
    group_m = group;
  }
  __device__ __forceinline__ void get(int tile, int& m_blk, int& n_blk) const {
    const int per_group = group_m * n_tiles;
    const int g = tile / per_group;
    const int first_m = g * group_m;
    const int gsz = min(group_m, m_tiles - first_m);
    const int r = tile - g * per_group;
    m_blk = first_m + (r % gsz);
    n_blk = r / gsz;
  }
};

// Epi concept:
//   struct Params;                          trivially copyable, passed by value to the kernel
//   static constexpr int SMEM_BYTES;        extra dynamic smem the epilogue wants (per CTA)
//   static __device__ void tile(const Params&, uint32_t taddr, int m0, int n0, int M, int N,
//                               int quad, int lane, uint8_t* epi_smem);
//     taddr addresses TMEM lane quad*32, first accumulator column of this tile; thread `lane`
//     of epilogue warp `quad` owns accumulator row m0 + quad*32 + lane, columns n0 .. n0+BN-1.
//     All 32 lanes must execute the same tcgen05.ld sequence.

template <int BN, int STAGES, bool A_MN, bool B_MN, class Epi>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                int K, int fmt, DescCfg dc, typename Epi::Params ep, unsigned int* err_word) {
  using S = Smem<BN, STAGES>;
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
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 512 or 256: a power of two >= 32

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], NUM_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  TileMap tm;
  tm.init(M, N, BN, 16);
  const int num_kb = (K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tm.num_tiles; tile += gridDim.x) {
        int m_blk, n_blk;
        tm.get(tile, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, err_word, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
          if constexpr (!A_MN) {
            tma_load_2d(sA, &tmA, &full_bar[s], kb * BK, m_blk * BM);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d(sA + i * (BK * 128), &tmA, &full_bar[s], m_blk * BM + i * 64, kb * BK);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sB, &tmB, &full_bar[s], kb * BK, n_blk * BN);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sB + i * (BK * 128), &tmB, &full_bar[s], n_blk * BN + i * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(fmt, BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, tl = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tm.num_tiles; tile += gridDim.x, ++tl) {
        const uint32_t acc = tl & 1u;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait_bounded(&tempty_bar[acc], aph ^ 1u, abort_flag, err_word, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
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
            const uint64_t da = make_smem_desc_sw128(a_base + k * dc.a_kadv, dc.a_lbo, dc.a_sbo);
            const uint64_t db = make_smem_desc_sw128(b_base + k * dc.b_kadv, dc.b_lbo, dc.b_sbo);
            umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // frees the smem stage once these MMAs have read it
        }
        if (ok) umma_commit(&tfull_bar[acc]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    uint32_t tl = 0;
    for (int tile = blockIdx.x; tile < tm.num_tiles; tile += gridDim.x, ++tl) {
      int m_blk, n_blk;
      tm.get(tile, m_blk, n_blk);
      const uint32_t acc = tl & 1u;
      const uint32_t aph = (tl >> 1) & 1u;
      int ok = mbar_wait_bounded(&tfull_bar[acc], aph, abort_flag, err_word, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
      Epi::tile(ep, taddr, m_blk * BM, n_blk * BN, M, N, quad, lane, epi_smem);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  // Teardown. After an abort, give in-flight TMA / MMA work a bounded grace period before the
  // CTA's shared memory and TMEM go away.
  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace b200
