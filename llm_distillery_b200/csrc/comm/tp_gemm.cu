// Tensor-parallel linear layers with the collective inside the GEMM kernel (sm_100a, tcgen05 mainloop of
// gemm_core.cuh, peer loads/stores over NVLink on symmetric buffers; no NCCL, no multimem, no TMA multicast).
//
//   ag_gemm   Y[T, N_local] = gather_rows(X)[T, K] * W[N_local, K]^T          (column-parallel: QKV, gate/up, lm_head)
//     X lives token-sharded: rank q produced rows [q*Ts, (q+1)*Ts) of ITS copy of the gathered buffer XF. Four extra
//     "copy warps" per CTA pull the other ranks' slabs into the local XF, 128-row block by block, in the order
//     rank+1, rank+2, ...; the tile loop runs over the same order starting with the rank's own slab, and the TMA
//     producer starts a tile only when the block's arrival counter says that all copy warps have delivered it.
//     So the NVLink transfer of slab j+1 hides behind the MMAs on slab j, every byte crosses NVLink once, and the
//     tensor core only ever reads local memory.
//
//   gemm_rs   Y_shard[Ts, N] = reduce_scatter_rows( X[T, K_local] * W[N, K_local]^T ) (+ residual)   (row-parallel: O, down)
//     The epilogue stores each bf16 partial tile straight into the OWNER rank's staging buffer (slot = this rank);
//     tiles owned by other ranks come first, so their stores travel while the own tiles are computed. When the grid is
//     through with one destination's tiles, that destination is told "my partials for you have landed"; after their
//     last tile the epilogue warps of all CTAs wait for every rank's message and sum the `world` staged partials
//     (+ residual) of their shard in fp32.
//
// Cross-rank flags are epoch numbers that only grow; each wait is bounded (2 s) and reports ERR_WAIT_PEER /
// ERR_WAIT_AUX through the error word. A kernel here needs all its CTAs resident at once (they wait on one another
// through the block counters): the grid never exceeds the SM count and the kernel takes a whole SM per CTA.
#include "peer.cuh"
#include "../gemm/gemm_pair.cuh"
#include "../common/host.cuh"
#include <stdlib.h>

namespace b200 {
namespace tp {
using namespace gemm;
using comm::Peers;

constexpr int TBN = 256;
constexpr int TSTAGES = 4;
constexpr int AG_THREADS = 320;  // TMA warp, MMA warp, 4 epilogue warps, 4 copy warps
constexpr int RS_THREADS = 192;
constexpr int COPY_WARPS = 4;
constexpr int COPY_UNROLL = 8;  // 16-byte peer loads in flight per copy thread: NVLink latency needs MBs in flight

enum Mode { MODE_AG = 0, MODE_RS = 1 };

struct TpParams {
  // common
  int rank, world;
  int blocks_per_shard;  // 128-row blocks per rank slab (Ts / 128)
  int group_m;           // row tiles per L2 tile group: a divisor of the tiles per slab, so that no group spans two
                         // slabs and every CTA meets the slabs (= destinations, sources) in one monotonic order
  unsigned int epoch;    // this call's number on the flag words it uses
  Peers flags;           // every rank's flag array for this kind of call: flags.p[dst][src] = epoch
  // ag_gemm
  Peers xf;                 // every rank's gathered buffer [T, K] bf16
  unsigned int* blk_count;  // local [m_tiles] arrival counters, zeroed before the launch
  long long row_bytes;      // K * 2
  void* C;                  // [T, N] output, bf16 or fp32
  long long ldc;
  int out_f32;
  // gemm_rs
  Peers stg;                 // every rank's staging buffer [world][Ts][N] bf16
  unsigned int* done_count;  // local [world] counters of epilogue warps through with each destination, zeroed before the launch
  const __nv_bfloat16* resid;  // [Ts, N] or null
  __nv_bfloat16* out;          // [Ts, N]
};

__device__ __forceinline__ uint4 ld_peer_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void acc_bf16x8(float (&a)[8], const uint4& q) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 f = __bfloat1622float2(h[t]);
    a[2 * t] += f.x;
    a[2 * t + 1] += f.y;
  }
}

// Store this warp's 32 x 256 slice of the accumulator tile as bf16. The slice goes through a per-warp shared-memory
// stage (32 rows x 256 B, 16-byte chunks XOR-swizzled by row) so that every global store instruction writes two
// whole 256-byte row segments: stores that cross NVLink then travel as full sectors instead of 16-byte fragments.
// dst points at the slice's first row (row stride ld elements); rows_valid of its 32 rows exist; N % 8 == 0.
constexpr int EPI_STAGE_BYTES = 32 * 256;
__device__ __forceinline__ void store_tile_bf16(uint32_t taddr, uint8_t* stage, __nv_bfloat16* dst, long long ld,
                                                int rows_valid, int n0, int N, int lane) {
#pragma unroll 1
  for (int half = 0; half < TBN / 128; ++half) {
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
    __syncwarp();
    const int chunk = lane & 15;
    const int col = n0 + half * 128 + chunk * 8;
#pragma unroll 4
    for (int j = 0; j < 16; ++j) {
      const int row = 2 * j + (lane >> 4);
      const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 256 + ((chunk ^ (row & 15)) << 4));
      if (row < rows_valid && col < N) *reinterpret_cast<uint4*>(dst + (long long)row * ld + col) = v;
    }
    __syncwarp();
  }
}

__device__ __forceinline__ void store_tile_f32(uint32_t taddr, float* dst_row, bool row_ok, int n0, int N) {
#pragma unroll 1
  for (int c = 0; c < TBN / 32; ++c) {
    uint32_t r[32];
    __syncwarp();
    tmem_ld_32x32b_x32(taddr + c * 32, r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
    if (!row_ok || col0 >= N) continue;
    float* cp = dst_row + col0;
    if (col0 + 32 <= N && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0)) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(cp + j * 4) = make_uint4(r[j * 4], r[j * 4 + 1], r[j * 4 + 2], r[j * 4 + 3]);
    } else {
      for (int j = 0; j < min(32, N - col0); ++j) cp[j] = __uint_as_float(r[j]);
    }
  }
}

// gemm_rs signalling. The tile loop visits the destinations in phases: phase ph holds the tiles owned by rank
// (rank + 1 + ph) % world, the own tiles come last. When a warp has moved past its tiles of a phase (stores fenced at
// system scope) it counts itself on that destination's counter; the last of the grid's epilogue warps tells the
// destination "rank `rank`'s partials for you have landed". A destination therefore hears from a source as soon as
// that source is through with ITS rows, not when the source's whole GEMM is over.
__device__ __forceinline__ void rs_signal_phases(const TpParams& p, int from_phase, int to_phase, int lane) {
  if (to_phase <= from_phase) return;
  __threadfence_system();
  __syncwarp();
  if (lane == 0) {
    for (int ph = from_phase; ph < to_phase; ++ph) {
      const int dest = (p.rank + 1 + ph) % p.world;
      const unsigned int old = atomicAdd(p.done_count + dest, 1u);
      if (old + 1u == gridDim.x * NUM_EPI_WARPS) {
        __threadfence_system();
        comm::st_release_sys(reinterpret_cast<unsigned int*>(p.flags.p[dest]) + p.rank, p.epoch);
      }
    }
  }
  __syncwarp();
}
__device__ __forceinline__ int rs_phase_of(const TpParams& p, int owner) {
  return (owner - p.rank - 1 + 2 * p.world) % p.world;
}

// gemm_rs, after a warp's last tile: signal the phases not yet signalled, wait for every rank's message to this rank,
// then sum the staged partials (+ residual) of the own shard. ew = epilogue warp index 0..3.
__device__ __forceinline__ void rs_tail(const TpParams& p, int N, bool ok_all, int phases_signalled, int ew, int lane,
                                        volatile int* abort_flag, unsigned int* err_word) {
  const long long Ts = (long long)p.blocks_per_shard * BM;
  rs_signal_phases(p, phases_signalled, p.world, lane);
  int okw = 1;
  if (ok_all && lane < p.world)
    okw = comm::wait_reached_bounded<true>(reinterpret_cast<const unsigned int*>(p.flags.p[p.rank]) + lane, p.epoch,
                                           abort_flag, err_word, ERR_WAIT_PEER) ? 1 : 0;
  okw = __all_sync(0xffffffffu, okw);
  if (!(ok_all && okw)) return;
  const long long nvec = Ts * N / 8;
  const uint4* st = reinterpret_cast<const uint4*>(p.stg.p[p.rank]);
  const uint4* rs = reinterpret_cast<const uint4*>(p.resid);
  uint4* out = reinterpret_cast<uint4*>(p.out);
  const long long step = (long long)gridDim.x * (NUM_EPI_WARPS * 32);
  constexpr int U = 8;  // independent 16-byte streams per thread: ~64 KB in flight per SM is what HBM latency needs
  for (long long i0 = (long long)blockIdx.x * (NUM_EPI_WARPS * 32) + ew * 32 + lane; i0 < nvec; i0 += U * step) {
    float a[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int e = 0; e < 8; ++e) a[u][e] = 0.f;
      const long long i = i0 + u * step;
      if (rs && i < nvec) acc_bf16x8(a[u], ld_cg_v4(rs + i));
    }
    for (int q = 0; q < p.world; ++q) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * step;
        v[u] = i < nvec ? ld_cg_v4(st + q * nvec + i) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) acc_bf16x8(a[u], v[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * step;
      if (i < nvec) {
        uint4 o;
        o.x = pack_bf16x2(a[u][0], a[u][1]);
        o.y = pack_bf16x2(a[u][2], a[u][3]);
        o.z = pack_bf16x2(a[u][4], a[u][5]);
        o.w = pack_bf16x2(a[u][6], a[u][7]);
        out[i] = o;
      }
    }
  }
}

// ag_gemm copy warps (ct = 0..127 inside the CTA): announce the own slab, then pull the other ranks' slabs into the
// local gathered buffer, one 128-row block at a time, and count each finished block.
__device__ __forceinline__ void ag_copy_warps(const TpParams& p, int ct, int lane, volatile int* abort_flag,
                                              unsigned int* err_word) {
  const int bps = p.blocks_per_shard;
  if (blockIdx.x == 0 && ct == 0) {
    // the own slab was written by the kernel before this one on the stream: tell the peers it is ready
    __threadfence_system();
    for (int q = 0; q < p.world; ++q)
      if (q != p.rank) comm::st_release_sys(reinterpret_cast<unsigned int*>(p.flags.p[q]) + p.rank, p.epoch);
  }
  const long long blk_vecs = (long long)BM * p.row_bytes / 16;
  const long long step = (long long)gridDim.x * (COPY_WARPS * 32);
  uint4* dst_base = reinterpret_cast<uint4*>(p.xf.p[p.rank]);
  for (int j = 1; j < p.world; ++j) {
    const int src = (p.rank + j) % p.world;
    int w = comm::wait_reached_bounded<true>(reinterpret_cast<const unsigned int*>(p.flags.p[p.rank]) + src, p.epoch,
                                             abort_flag, err_word, ERR_WAIT_PEER) ? 1 : 0;
    if (!__all_sync(0xffffffffu, w)) break;
    const uint4* src_base = reinterpret_cast<const uint4*>(p.xf.p[src]);
    for (int b = 0; b < bps; ++b) {
      const int m_blk = src * bps + b;
      const long long off = (long long)m_blk * blk_vecs;
      // every thread keeps COPY_UNROLL peer loads in flight (predicated at the block's end), then stores them
      for (long long i0 = (long long)blockIdx.x * (COPY_WARPS * 32) + ct; i0 < blk_vecs; i0 += COPY_UNROLL * step) {
        uint4 v[COPY_UNROLL];
#pragma unroll
        for (int u = 0; u < COPY_UNROLL; ++u)
          if (i0 + u * step < blk_vecs) v[u] = ld_peer_v4(src_base + off + i0 + u * step);
#pragma unroll
        for (int u = 0; u < COPY_UNROLL; ++u)
          if (i0 + u * step < blk_vecs) dst_base[off + i0 + u * step] = v[u];
      }
      fence_proxy_async_all();
      __threadfence();
      __syncwarp();
      if (lane == 0) comm::red_release_gpu_add(p.blk_count + m_blk, 1u);
    }
  }
}

// One warp's share of a finished accumulator tile: rows row0 .. row0+31 of the GEMM, columns n0 .. n0+255.
template <int MODE>
__device__ __forceinline__ void epilogue_slice(const TpParams& p, uint32_t taddr, uint8_t* stage, int row0, int n0,
                                               int M, int N, int lane) {
  const int rows_valid = min(32, M - row0);
  if (MODE == MODE_AG) {
    if (p.out_f32)
      store_tile_f32(taddr, reinterpret_cast<float*>(p.C) + (long long)(row0 + lane) * p.ldc, lane < rows_valid, n0, N);
    else
      store_tile_bf16(taddr, stage, reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row0 * p.ldc, p.ldc, rows_valid,
                      n0, N, lane);
  } else {
    const long long Ts = (long long)p.blocks_per_shard * BM;
    const int owner = row0 / (int)Ts;
    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.stg.p[owner]);
    const long long lrow0 = (long long)p.rank * Ts + (row0 - (long long)owner * Ts);
    store_tile_bf16(taddr, stage, base + lrow0 * N, N, rows_valid, n0, N, lane);
  }
}

template <int MODE>
__global__ void __launch_bounds__(MODE == MODE_AG ? AG_THREADS : RS_THREADS, 1)
    tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                   int K, TpParams p, unsigned int* err_word) {
  using S = Smem<TBN, TSTAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::RING_BYTES);
  uint64_t* empty_bar = full_bar + TSTAGES;
  uint64_t* tfull_bar = empty_bar + TSTAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_smem = smem + S::RING_BYTES + S::BAR_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * TBN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < TSTAGES; ++s) {
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
  tm.init(M, N, TBN, p.group_m);
  const int num_kb = (K + BK - 1) / BK;
  const int bps = p.blocks_per_shard;
  // logical row-block order: ag_gemm starts with the own slab; gemm_rs ends with it
  const int rot = (MODE == MODE_AG ? p.rank : (p.rank + 1) % p.world) * bps;
  auto phys_block = [&](int lm) { return (lm + rot) % tm.m_tiles; };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const unsigned int arrivals = gridDim.x * COPY_WARPS;
      for (int tile = blockIdx.x; ok && tile < tm.num_tiles; tile += gridDim.x) {
        int lm, n_blk;
        tm.get(tile, lm, n_blk);
        const int m_blk = phys_block(lm);
        if (MODE == MODE_AG && m_blk / bps != p.rank) {
          // rows of another rank: wait until every CTA's copy warps have landed this block in local memory
          if (!comm::wait_reached_bounded<false>(p.blk_count + m_blk, arrivals, abort_flag, err_word, ERR_WAIT_AUX)) break;
          fence_proxy_async_all();  // generic-proxy stores (the copy) before async-proxy reads (TMA)
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % TSTAGES;
          const uint32_t ph = (it / TSTAGES) & 1u;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, err_word, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], S::STAGE_BYTES);
          tma_load_2d(sA, &tmA, &full_bar[s], kb * BK, m_blk * BM);
          tma_load_2d(sB, &tmB, &full_bar[s], kb * BK, n_blk * TBN);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(1, BM, TBN, 0, 0);
      uint32_t it = 0, tl = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tm.num_tiles; tile += gridDim.x, ++tl) {
        const uint32_t acc = tl & 1u;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait_bounded(&tempty_bar[acc], aph ^ 1u, abort_flag, err_word, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * TBN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % TSTAGES;
          const uint32_t ph = (it / TSTAGES) & 1u;
          if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, err_word, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b_base = a_base + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(a_base + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = make_smem_desc_sw128(b_base + k * (UMMA_K * 2), 16, 1024);
            umma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
        }
        if (ok) umma_commit(&tfull_bar[acc]);
      }
    }
  } else if (warp < 2 + NUM_EPI_WARPS) {
    // ------------------------------------------------------------ epilogue warps (2..5)
    const int quad = warp & 3;
    uint32_t tl = 0;
    bool ok_all = true;
    int phases_signalled = 0;
    for (int tile = blockIdx.x; tile < tm.num_tiles; tile += gridDim.x, ++tl) {
      int lm, n_blk;
      tm.get(tile, lm, n_blk);
      const int m_blk = phys_block(lm);
      const uint32_t acc = tl & 1u;
      const uint32_t aph = (tl >> 1) & 1u;
      int ok = mbar_wait_bounded(&tfull_bar[acc], aph, abort_flag, err_word, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        ok_all = false;
        break;
      }
      tc_fence_after_sync();
      if (MODE == MODE_RS) {
        const int ph = rs_phase_of(p, m_blk / bps);
        rs_signal_phases(p, phases_signalled, ph, lane);
        phases_signalled = max(phases_signalled, ph);
      }
      const uint32_t taddr = tmem_base + acc * TBN + (static_cast<uint32_t>(quad * 32) << 16);
      epilogue_slice<MODE>(p, taddr, epi_smem + (warp - 2) * EPI_STAGE_BYTES, m_blk * BM + quad * 32, n_blk * TBN, M, N,
                           lane);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
    if (MODE == MODE_RS) rs_tail(p, N, ok_all, phases_signalled, warp - 2, lane, abort_flag, err_word);
  } else {
    // ------------------------------------------------------------ copy warps (ag_gemm only)
    if (MODE == MODE_AG) ag_copy_warps(p, threadIdx.x - (2 + NUM_EPI_WARPS) * 32, lane, abort_flag, err_word);
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------------- CTA-pair variant
// Same two fused layers on the cta_group::2 mainloop (gemm_pair.cuh): a cluster of two CTAs per 256 x 256 tile, each
// CTA loading its own 128 rows of A and its own half of B (no multicast), 6 stages. Used when every rank's slab is a
// whole number of 256-row tiles. Block counters stay per 128 rows: each CTA's producer waits for its own rows.
constexpr int PSTAGES = 6;

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MODE == MODE_AG ? AG_THREADS : RS_THREADS, 1)
    tp_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                        int K, TpParams p, unsigned int* err_word) {
  using S = SmemPair<PSTAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::RING_BYTES);
  uint64_t* empty_bar = full_bar + PSTAGES;
  uint64_t* tfull_bar = empty_bar + PSTAGES;
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
    for (int s = 0; s < PSTAGES; ++s) {
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
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int m_tiles = (M + PAIR_BM - 1) / PAIR_BM;
  const int n_tiles = (N + PAIR_BN - 1) / PAIR_BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int bps2 = p.blocks_per_shard / 2;  // 256-row tiles per slab
  const int group_m = p.group_m;
  const int rot = (MODE == MODE_AG ? p.rank : (p.rank + 1) % p.world) * bps2;
  auto tile_coords = [&](int tile, int& m_blk, int& n_blk) {
    const int per_group = group_m * n_tiles;
    const int g = tile / per_group;
    const int first_m = g * group_m;
    const int gsz = min(group_m, m_tiles - first_m);
    const int r = tile - g * per_group;
    m_blk = (first_m + (r % gsz) + rot) % m_tiles;  // physical tile row: own slab first (ag) or last (rs)
    n_blk = r / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const unsigned int arrivals = gridDim.x * COPY_WARPS;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
        int m_blk, n_blk;
        tile_coords(tile, m_blk, n_blk);
        const int m0 = m_blk * PAIR_BM + (int)cta * BM;
        const int n0 = n_blk * PAIR_BN + (int)cta * PAIR_HALF_N;
        if (MODE == MODE_AG && m_blk / bps2 != p.rank) {
          if (!comm::wait_reached_bounded<false>(p.blk_count + m0 / BM, arrivals, abort_flag, err_word, ERR_WAIT_AUX)) break;
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1u;
          if (!mbar_wait_bounded(&empty_bar[s], ph ^ 1u, abort_flag, err_word, ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + s * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          if (cta == 0) mbar_arrive_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);
          tma_load_2d_pair(sA, &tmA, &full_bar[s], kb * BK, m0);
          tma_load_2d_pair(sB, &tmB, &full_bar[s], kb * BK, n0);
        }
      }
      for (uint32_t d = 0; ok && d < (uint32_t)PSTAGES && d < it; ++d) {
        const uint32_t j = it - 1 - d;
        if (!mbar_wait_bounded(&empty_bar[j % PSTAGES], (j / PSTAGES) & 1u, abort_flag, err_word, ERR_WAIT_EMPTY)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && cta == 0) {
      const uint32_t idesc = make_idesc_f16(1, PAIR_BM, PAIR_BN, 0, 0);
      uint32_t it = 0, tl = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs, ++tl) {
        const uint32_t acc = tl & 1u;
        const uint32_t aph = (tl >> 1) & 1u;
        if (!mbar_wait_bounded(&tempty_bar[acc], aph ^ 1u, abort_flag, err_word, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * PAIR_BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % PSTAGES;
          const uint32_t ph = (it / PSTAGES) & 1u;
          if (!mbar_wait_bounded(&full_bar[s], ph, abort_flag, err_word, ERR_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b_base = a_base + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = make_smem_desc_sw128(a_base + k * (UMMA_K * 2), 16, 1024);
            const uint64_t db = make_smem_desc_sw128(b_base + k * (UMMA_K * 2), 16, 1024);
            umma_f16_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s], 0x3);
        }
        if (ok) umma_commit_pair(&tfull_bar[acc], 0x3);
      }
    }
  } else if (warp < 2 + NUM_EPI_WARPS) {
    // ------------------------------------------------------------ epilogue warps (both CTAs)
    const int quad = warp & 3;
    const uint32_t leader_tempty0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    uint32_t tl = 0;
    bool ok_all = true;
    int phases_signalled = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++tl) {
      int m_blk, n_blk;
      tile_coords(tile, m_blk, n_blk);
      const uint32_t acc = tl & 1u;
      const uint32_t aph = (tl >> 1) & 1u;
      int ok = mbar_wait_bounded(&tfull_bar[acc], aph, abort_flag, err_word, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        ok_all = false;
        break;
      }
      tc_fence_after_sync();
      if (MODE == MODE_RS) {
        const int ph = rs_phase_of(p, m_blk / bps2);
        rs_signal_phases(p, phases_signalled, ph, lane);
        phases_signalled = max(phases_signalled, ph);
      }
      const uint32_t taddr = tmem_base + acc * PAIR_BN + (static_cast<uint32_t>(quad * 32) << 16);
      epilogue_slice<MODE>(p, taddr, epi_smem + (warp - 2) * EPI_STAGE_BYTES,
                           m_blk * PAIR_BM + (int)cta * BM + quad * 32, n_blk * PAIR_BN, M, N, lane);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty0 + acc * 8);
    }
    if (MODE == MODE_RS) rs_tail(p, N, ok_all, phases_signalled, warp - 2, lane, abort_flag, err_word);
  } else {
    // ------------------------------------------------------------ copy warps (ag_gemm only)
    if (MODE == MODE_AG) ag_copy_warps(p, threadIdx.x - (2 + NUM_EPI_WARPS) * 32, lane, abort_flag, err_word);
  }

  __syncwarp();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace tp
}  // namespace b200

namespace {

using namespace b200;
using namespace b200::tp;

int fill_peers(comm::Peers& dst, const void* const* src, int world) {
  if (!src) return B200_ERR_ARG;
  for (int i = 0; i < comm::MAX_RANKS; ++i) dst.p[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (!src[i]) return B200_ERR_ARG;
    dst.p[i] = const_cast<void*>(src[i]);
  }
  return B200_OK;
}

static int pair_mode() {
  static int mode = -2;
  if (mode == -2) {
    const char* e = getenv("B200_TP_PAIR");
    mode = e ? atoi(e) : -1;
  }
  return mode;
}

template <int MODE>
int launch(const void* A, long long lda, const void* W, long long ldw, int T, int N, int K, const TpParams& p_in,
           cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)T, (uint64_t)lda * 2,
                        gemm::BK, gemm::BM, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B200_OK) return rc;
  const int threads = MODE == MODE_AG ? AG_THREADS : RS_THREADS;
  const int epi_bytes = gemm::NUM_EPI_WARPS * EPI_STAGE_BYTES;
  // CTA pairs when every slab is whole 256-row tiles and there are enough tiles for all SM pairs
  const long long ptiles = (long long)(T / gemm::PAIR_BM) * ceil_div(N, gemm::PAIR_BN);
  const bool pair = pair_mode() != 0 && (p_in.blocks_per_shard % 2 == 0) && N > 128 &&
                    (pair_mode() == 1 || ptiles >= sm_count() / 2);
  TpParams p = p_in;
  {
    const int per_slab = pair ? p.blocks_per_shard / 2 : p.blocks_per_shard;
    const int cap = pair ? 8 : 16;
    int g = per_slab < cap ? per_slab : cap;
    while (per_slab % g) --g;
    p.group_m = g;
  }
  if (pair) {
    using S = gemm::SmemPair<PSTAGES>;
    rc = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldw * 2,
                      gemm::BK, gemm::PAIR_HALF_N, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != B200_OK) return rc;
    auto kern = tp_gemm_pair_kernel<MODE>;
    const int smem_bytes = S::bytes(epi_bytes);
    static bool attr_set = false;
    if (!attr_set) {
      B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
      attr_set = true;
    }
    const int max_pairs = sm_count() / 2;
    const int pairs = ptiles < max_pairs ? (int)ptiles : max_pairs;
    kern<<<2 * pairs, threads, smem_bytes, stream>>>(tmA, tmB, T, N, K, p, device_err_word());
  } else {
    using S = gemm::Smem<TBN, TSTAGES>;
    rc = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldw * 2,
                      gemm::BK, TBN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != B200_OK) return rc;
    auto kern = tp_gemm_kernel<MODE>;
    const int smem_bytes = S::bytes(epi_bytes);
    static bool attr_set = false;
    if (!attr_set) {
      B200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
      attr_set = true;
    }
    const int tiles = ceil_div(T, gemm::BM) * ceil_div(N, TBN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    kern<<<grid, threads, smem_bytes, stream>>>(tmA, tmB, T, N, K, p, device_err_word());
  }
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace

extern "C" {

// Column-parallel linear with the all-gather inside: C[T, N] = XF[T, K] * W[N, K]^T, where rank q has written rows
// [q*T/world, (q+1)*T/world) of ITS gathered buffer xf_ptrs[q] before this call (same stream) and the kernel pulls
// the other slabs into xf_ptrs[rank] while it computes. flag_ptrs[q] = rank q's flag array (16 words) reserved for
// ag_gemm calls; `epoch` must grow by one per call, identically on every rank. blk_count: T/128 words of scratch.
// C is bf16, or fp32 when out_f32 (the LM head's logits).
// The gathered buffer must not be reused for the next call's input (alternate between two).
int b200_tp_ag_gemm(const void* const* xf_ptrs, const void* const* flag_ptrs, const void* W, void* C,
                    unsigned int* blk_count, int T, int N, int K, long long ldc, int out_f32, int rank, int world,
                    unsigned int epoch, cudaStream_t stream) {
  if (!W || !C || !blk_count || T <= 0 || N <= 0 || K <= 0 || world < 1 || world > comm::MAX_RANKS || rank < 0 ||
      rank >= world)
    return B200_ERR_ARG;
  if (T % (world * gemm::BM) != 0 || (K & 7) || (!out_f32 && ((ldc & 7) || (N & 7)))) return B200_ERR_ARG;
  TpParams p{};
  p.rank = rank;
  p.world = world;
  p.blocks_per_shard = T / world / gemm::BM;
  p.epoch = epoch;
  p.out_f32 = out_f32;
  int rc = fill_peers(p.xf, xf_ptrs, world);
  if (rc != B200_OK) return rc;
  rc = fill_peers(p.flags, flag_ptrs, world);
  if (rc != B200_OK) return rc;
  p.blk_count = blk_count;
  p.row_bytes = (long long)K * 2;
  p.C = C;
  p.ldc = ldc;
  B200_CUDA_CHECK(cudaMemsetAsync(blk_count, 0, sizeof(unsigned int) * (T / gemm::BM), stream));
  return launch<MODE_AG>(xf_ptrs[rank], K, W, K, T, N, K, p, stream);
}

// Row-parallel linear with the reduce-scatter inside: out[T/world, N] = rows of this rank of
// sum over ranks ( X[T, K] * W[N, K]^T ) + residual. stg_ptrs[q] = rank q's staging buffer [world][T/world][N] bf16;
// flag_ptrs[q] = rank q's flag array reserved for gemm_rs calls; done_count: `world` words of scratch.
// Alternate between two staging buffers on consecutive calls.
int b200_tp_gemm_rs(const void* X, long long ldx, const void* W, const void* const* stg_ptrs,
                    const void* const* flag_ptrs, const void* residual, void* out, unsigned int* done_count, int T,
                    int N, int K, int rank, int world, unsigned int epoch, cudaStream_t stream) {
  if (!X || !W || !out || !done_count || T <= 0 || N <= 0 || K <= 0 || world < 1 || world > comm::MAX_RANKS ||
      rank < 0 || rank >= world)
    return B200_ERR_ARG;
  if (T % (world * gemm::BM) != 0 || (K & 7) || (N & 7) || (ldx & 7)) return B200_ERR_ARG;
  TpParams p{};
  p.rank = rank;
  p.world = world;
  p.blocks_per_shard = T / world / gemm::BM;
  p.epoch = epoch;
  int rc = fill_peers(p.stg, stg_ptrs, world);
  if (rc != B200_OK) return rc;
  rc = fill_peers(p.flags, flag_ptrs, world);
  if (rc != B200_OK) return rc;
  p.done_count = done_count;
  p.resid = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  B200_CUDA_CHECK(cudaMemsetAsync(done_count, 0, sizeof(unsigned int) * world, stream));
  return launch<MODE_RS>(X, ldx, W, K, T, N, K, p, stream);
}
}
