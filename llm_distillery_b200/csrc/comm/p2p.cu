// NVLink peer-to-peer collectives over symmetric memory (every rank's buffer mapped into every rank's address
// space). Kernels here use plain peer loads / stores and system-scope release/acquire flags; nothing uses TMA
// multicast or multimem. One process drives one GPU, so kernels that wait on a peer's flag always run on a
// different GPU than the kernel that sets it.
//
//   p2p_barrier        epoch-numbered flag exchange; every wait is bounded (2 s) and reports ERR_WAIT_PEER
//   rs_adamw_ag        THE data-parallel optimizer step: for this rank's shard of the flat parameter space, sum
//                      the fp32 gradients of all ranks straight out of their memory (reduce-scatter by peer loads),
//                      apply AdamW to the local fp32 master / moments, and store the new bf16 weights into every
//                      rank's weight buffer (all-gather by peer stores) - one pass, no staging buffers
//   reduce_scatter_f32 / allgather_16 / allreduce_f32   stand-alone pieces for the other optimizers and for tests
//   gather_pull / reduce_scatter_acc_f32   full parameter sharding: a unit's weights pulled from the ranks' shards
//                      just before it runs; its gradients summed onto this rank's slice right after its backward
//
// Wire format of the data-parallel gradient exchange: every rank casts its fp32 gradient to a bf16 copy in symmetric
// memory (cast_wire); the owner of a shard adds its OWN fp32 gradient and the peers' bf16 copies in fp32 registers.
// Half the bytes cross NVLink, and the sum is still fp32.
//
// A barrier whose wait runs out poisons this GPU's collectives: it sets a device word that every kernel of this
// file reads first, and a kernel that finds it set returns without touching anything. The reduction and optimizer
// kernels queued behind a failed barrier therefore leave master weights, moments and every rank's weights as the
// last good step wrote them. The host clears the word when it has taken note of the error (b200_p2p_clear_poison).
#include "peer.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace comm {

__device__ unsigned int g_poison = 0;
__device__ __forceinline__ bool poisoned() { return *reinterpret_cast<volatile unsigned int*>(&g_poison) != 0u; }

// sig[r] points at rank r's flag array (MAX_RANKS words). Thread t tells rank t "rank `rank` reached `epoch`" and
// waits until rank t has told us the same. Epochs only grow, so a late reader never sees a stale match.
__global__ void barrier_kernel(Peers sig, int rank, int world, unsigned int epoch, unsigned int* err_word) {
  const int t = threadIdx.x;
  if (t >= world) return;
  // an earlier barrier already gave up: post nothing (the peers' waits run out too, so every survivor skips the
  // step) and do not wait two more seconds
  if (poisoned()) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<unsigned int*>(sig.p[t]) + rank, epoch);
  const unsigned int* mine = reinterpret_cast<const unsigned int*>(sig.p[rank]) + t;
  const unsigned long long t0 = globaltimer_ns();
  unsigned int spins = 0;
  while (static_cast<int>(ld_acquire_sys(mine) - epoch) < 0) {
    if (((++spins) & 0xffu) == 0u && globaltimer_ns() - t0 > kWaitTimeoutNs) {
      atomicExch(&g_poison, 1u);
      if (err_word) atomicCAS(err_word, 0u, (unsigned)ERR_WAIT_PEER);
      return;
    }
    __nanosleep(64);
  }
}

__global__ void clear_poison_kernel() { g_poison = 0u; }

// Counts the optimizer steps whose reduction really ran: queued right behind the reduction kernels, it adds one
// unless the step's barrier gave up. The host compares the count with the steps it issued before it saves state.
__global__ void mark_step_kernel(unsigned int* counter) {
  if (!poisoned()) *counter += 1u;
}

// wire[lo + i] = bf16(grad[lo + i]), 8 elements per thread
__global__ void __launch_bounds__(256) cast_wire_kernel(const float* __restrict__ grad, __nv_bfloat16* __restrict__ wire,
                                                        long long lo, long long n) {
  if (poisoned()) return;
  const long long nv = n >> 3;
  const float4* src = reinterpret_cast<const float4*>(grad + lo);
  uint4* dst = reinterpret_cast<uint4*>(wire + lo);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 x = src[2 * i], y = src[2 * i + 1];
    uint4 o;
    o.x = pack_bf16x2(x.x, x.y);
    o.y = pack_bf16x2(x.z, x.w);
    o.z = pack_bf16x2(y.x, y.y);
    o.w = pack_bf16x2(y.z, y.w);
    dst[i] = o;
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale;
  int decoupled;
};

__device__ __forceinline__ void add_bf16x8(float (&g)[8], const uint4& q) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const float2 x = __bfloat1622float2(h[t]);
    g[2 * t] += x.x;
    g[2 * t + 1] += x.y;
  }
}

// 8 elements per thread. MODE 0: `grads` are the ranks' fp32 gradients (two float4 loads per peer).
// MODE 1: `grads` are the ranks' bf16 wire copies (one 16-byte load per peer) and this rank's own contribution comes
// from `own` (its fp32 gradient). MODE 2: the sum over the ranks is already in `own`, a local fp32 buffer that holds
// this rank's shard only (indexed like master / m / v) - the reduction ran earlier, behind backward. One 16-byte bf16
// store per peer in every mode.
// W: the largest world size this instantiation serves (the peers' vectors of MODE 1 live in W registers-quads; with
// W = 16 for every world size the kernel needed 128 registers and half the resident warps).
template <int MODE, int W>
__global__ void __launch_bounds__(256, (W <= 8 ? 3 : 2)) rs_adamw_ag_kernel(Peers grads, const float* __restrict__ own, Peers models,
                                                         float* __restrict__ master, float* __restrict__ m,
                                                         float* __restrict__ v, long long shard_lo, long long shard_n,
                                                         long long state_off, int rank, int world, AdamArgs a) {
  if (poisoned()) return;
  const long long nv = shard_n >> 3;
  master += state_off; m += state_off; v += state_off;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    // (Issuing the master / moment loads BEFORE the peers' gradients are consumed was tried: it costs ~90 more
    // registers, occupancy drops to one CTA per SM and the kernel takes 7.5 ms instead of 4.6 ms for 0.55 B parameters
    // on two GPUs. Many resident warps hide the NVLink latency better than a few warps with every load in flight.)
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (MODE == 2) {
      const float4* src = reinterpret_cast<const float4*>(own + state_off) + 2 * i;
      const float4 x = src[0], y = src[1];
      g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w;
      g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
    } else if (MODE == 1) {
      uint4 q[W];
#pragma unroll
      for (int k = 1; k < W; ++k)   // all peer loads issued before the first use: their latencies overlap
        if (k < world)
          q[k] = (reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[(rank + k) % world]) +
                                                 shard_lo))[i];
      const float4* src = reinterpret_cast<const float4*>(own + shard_lo) + 2 * i;
      const float4 x = src[0], y = src[1];
      g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w;
      g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
#pragma unroll
      for (int k = 1; k < W; ++k)
        if (k < world) add_bf16x8(g, q[k]);
    } else {
      for (int k = 0; k < world; ++k) {
        const int p = (rank + k) % world;  // start with the local copy, spread peers over time
        const float4* src =
            reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[p]) + shard_lo) + 2 * i;
        const float4 x = src[0], y = src[1];
        g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w;
        g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
      }
    }
    float pm[8], mm[8], vv[8];
    *reinterpret_cast<float4*>(pm) = reinterpret_cast<float4*>(master)[2 * i];
    *reinterpret_cast<float4*>(pm + 4) = reinterpret_cast<float4*>(master)[2 * i + 1];
    *reinterpret_cast<float4*>(mm) = reinterpret_cast<float4*>(m)[2 * i];
    *reinterpret_cast<float4*>(mm + 4) = reinterpret_cast<float4*>(m)[2 * i + 1];
    *reinterpret_cast<float4*>(vv) = reinterpret_cast<float4*>(v)[2 * i];
    *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<float4*>(v)[2 * i + 1];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gj = g[j] * a.grad_scale;
      if (a.decoupled) pm[j] *= (1.f - a.lr * a.weight_decay);
      else gj += a.weight_decay * pm[j];
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
      pm[j] -= (a.lr / a.bias1) * mm[j] / (sqrtf(vv[j] / a.bias2) + a.eps);
    }
    reinterpret_cast<float4*>(master)[2 * i] = *reinterpret_cast<float4*>(pm);
    reinterpret_cast<float4*>(master)[2 * i + 1] = *reinterpret_cast<float4*>(pm + 4);
    reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(mm);
    reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(mm + 4);
    reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(vv);
    reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(vv + 4);
    uint4 o;
    o.x = pack_bf16x2(pm[0], pm[1]);
    o.y = pack_bf16x2(pm[2], pm[3]);
    o.z = pack_bf16x2(pm[4], pm[5]);
    o.w = pack_bf16x2(pm[6], pm[7]);
    for (int k = 0; k < world; ++k) {
      const int p = (rank + k) % world;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(models.p[p]) + shard_lo)[i] = o;
    }
  }
  __threadfence_system();
}

// Full sharding, last micro-batch of a step: g = acc + sum_p grads_p[grad_lo + i] (acc: what earlier micro-batches left
// in the local shard gradient, may be null), AdamW on the local piece of master / m / v, new bf16 weights into the
// local weight piece (peers pull it when they next gather the unit). 8 elements per thread.
__global__ void __launch_bounds__(256) rs_adamw_piece_kernel(Peers grads, long long grad_lo, const float* __restrict__ acc,
                                                            __nv_bfloat16* __restrict__ model, float* __restrict__ master,
                                                            float* __restrict__ m, float* __restrict__ v, long long n,
                                                            int rank, int world, AdamArgs a) {
  if (poisoned()) return;
  const long long nv = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (acc) {
      *reinterpret_cast<float4*>(g) = reinterpret_cast<const float4*>(acc)[2 * i];
      *reinterpret_cast<float4*>(g + 4) = reinterpret_cast<const float4*>(acc)[2 * i + 1];
    }
#pragma unroll 4
    for (int k = 0; k < world; ++k) {
      const int p = (rank + k) % world;
      const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[p]) + grad_lo) + 2 * i;
      const float4 x = src[0], y = src[1];
      g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w;
      g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
    }
    float pm[8], mm[8], vv[8];
    *reinterpret_cast<float4*>(pm) = reinterpret_cast<float4*>(master)[2 * i];
    *reinterpret_cast<float4*>(pm + 4) = reinterpret_cast<float4*>(master)[2 * i + 1];
    *reinterpret_cast<float4*>(mm) = reinterpret_cast<float4*>(m)[2 * i];
    *reinterpret_cast<float4*>(mm + 4) = reinterpret_cast<float4*>(m)[2 * i + 1];
    *reinterpret_cast<float4*>(vv) = reinterpret_cast<float4*>(v)[2 * i];
    *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<float4*>(v)[2 * i + 1];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gj = g[j] * a.grad_scale;
      if (a.decoupled) pm[j] *= (1.f - a.lr * a.weight_decay);
      else gj += a.weight_decay * pm[j];
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
      pm[j] -= (a.lr / a.bias1) * mm[j] / (sqrtf(vv[j] / a.bias2) + a.eps);
    }
    reinterpret_cast<float4*>(master)[2 * i] = *reinterpret_cast<float4*>(pm);
    reinterpret_cast<float4*>(master)[2 * i + 1] = *reinterpret_cast<float4*>(pm + 4);
    reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(mm);
    reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(mm + 4);
    reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(vv);
    reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(vv + 4);
    uint4 o;
    o.x = pack_bf16x2(pm[0], pm[1]);
    o.y = pack_bf16x2(pm[2], pm[3]);
    o.z = pack_bf16x2(pm[4], pm[5]);
    o.w = pack_bf16x2(pm[6], pm[7]);
    reinterpret_cast<uint4*>(model)[i] = o;
  }
  __threadfence_system();
}

// out[i] = scale * sum_p src_p[lo + i]   (fp32), i < n, n % 4 == 0. A thread works on U 16-byte vectors at a time and
// issues all world * U loads before the first addition: a peer load takes microseconds, and with one load in flight
// per thread a small grid (the reduction that runs beside backward) moved 10 GB/s. U is chosen so that world * U
// vectors (<= 16) are in flight per thread. The order of the additions is fixed: own copy first, then rank + 1, ...
template <int U>
__global__ void __launch_bounds__(256) reduce_scatter_kernel(Peers src, float* __restrict__ out, long long lo,
                                                            long long n, int rank, int world, float scale) {
  if (poisoned()) return;
  constexpr int W = 16 / U;                 // ranks this instantiation serves
  const long long nv = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nv; i0 += stride * U) {
    float4 x[W][U];
#pragma unroll
    for (int k = 0; k < W; ++k) {
      if (k < world) {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src.p[(rank + k) % world]) + lo);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long i = i0 + u * stride;
          if (i < nv) x[k][u] = p[i];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nv) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < W; ++k)
          if (k < world) { s.x += x[k][u].x; s.y += x[k][u].y; s.z += x[k][u].z; s.w += x[k][u].w; }
        s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
        reinterpret_cast<float4*>(out)[i] = s;
      }
    }
  }
}

// dst_p[lo_bytes + ...] = local[...] for every rank p: all-gather by peer stores, 16-byte granules
__global__ void __launch_bounds__(256) allgather_kernel(Peers dst, const uint4* __restrict__ local, long long lo_vec,
                                                       long long nvec, int rank, int world, int skip_self) {
  if (poisoned()) return;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 x = local[i];
    for (int k = skip_self ? 1 : 0; k < world; ++k) {
      const int p = (rank + k) % world;
      (reinterpret_cast<uint4*>(dst.p[p]) + lo_vec)[i] = x;
    }
  }
  __threadfence_system();
}

// dst[p * piece + i] = src_p[src_off + i] for every rank p (16-byte granules): all-gather by peer LOADS. The sources
// are read-only while this runs (weights between two optimizer steps), so no flags are exchanged. Eight loads per
// thread are in flight before the first store: NVLink latency is hidden by independent requests, not by occupancy.
__global__ void __launch_bounds__(256) gather_pull_kernel(Peers src, uint4* __restrict__ dst, long long src_off_vec,
                                                         long long piece_vec, int rank, int world) {
  if (poisoned()) return;
  constexpr int U = 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int k = 0; k < world; ++k) {
    // CTAs start at different sources, so the local copy and the loads from every peer run side by side
    const int p = (rank + k + (int)(blockIdx.x % (unsigned)world)) % world;
    const uint4* __restrict__ s = reinterpret_cast<const uint4*>(src.p[p]) + src_off_vec;
    uint4* __restrict__ d = dst + (long long)p * piece_vec;
    for (long long base = blockIdx.x * (long long)blockDim.x + threadIdx.x; base < piece_vec; base += stride * U) {
      uint4 x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + u * stride;
        if (i < piece_vec) x[u] = s[i];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + u * stride;
        if (i < piece_vec) d[i] = x[u];
      }
    }
  }
}

// out[i] (+)= sum_p src_p[lo + i]   (fp32), i < n, n % 4 == 0: reduce-scatter by peer loads into (or onto) a local slice
__global__ void __launch_bounds__(256) reduce_scatter_acc_kernel(Peers src, float* __restrict__ out, long long lo,
                                                                long long n, int rank, int world, int accumulate) {
  if (poisoned()) return;
  const long long nv = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 s = accumulate ? reinterpret_cast<const float4*>(out)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int k = 0; k < world; ++k) {
      const int p = (rank + k) % world;
      const float4 x = (reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src.p[p]) + lo))[i];
      s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
    }
    reinterpret_cast<float4*>(out)[i] = s;
  }
}

static int grid_for(long long items) {
  long long b = (items + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}
static bool fill(Peers& P, const void* const* ptrs, int world) {
  if (!ptrs || world < 1 || world > MAX_RANKS) return false;
  for (int i = 0; i < MAX_RANKS; ++i) P.p[i] = i < world ? const_cast<void*>(ptrs[i]) : nullptr;
  for (int i = 0; i < world; ++i)
    if (!P.p[i]) return false;
  return true;
}

}  // namespace comm
}  // namespace b200

extern "C" {
using namespace b200;
using namespace b200::comm;

int b200_p2p_max_ranks() { return MAX_RANKS; }

// sig_ptrs[r]: rank r's flag array (>= 16 uint32, zero-initialised once). epoch must grow by one per barrier.
int b200_p2p_barrier(const void* const* sig_ptrs, int rank, int world, unsigned int epoch, cudaStream_t st) {
  Peers S;
  if (!fill(S, sig_ptrs, world) || rank < 0 || rank >= world) return B200_ERR_ARG;
  barrier_kernel<<<1, 32, 0, st>>>(S, rank, world, epoch, device_err_word());
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// Clears the poison word of the current device (after the host has read the error word and decided to go on).
int b200_p2p_clear_poison(cudaStream_t st) {
  clear_poison_kernel<<<1, 1, 0, st>>>();
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_p2p_mark_step(unsigned int* counter, cudaStream_t st) {
  if (!counter) return B200_ERR_ARG;
  mark_step_kernel<<<1, 1, 0, st>>>(counter);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// wire[lo, lo + n) = bf16(grad[lo, lo + n)): this rank's gradient in the format the peers read. n, lo multiples of 8.
int b200_p2p_cast_wire(const float* grad, void* wire, long long lo, long long n, cudaStream_t st) {
  if (!grad || !wire || n <= 0 || (n & 7) || (lo & 7) || lo < 0) return B200_ERR_ARG;
  cast_wire_kernel<<<grid_for(n >> 3), 256, 0, st>>>(grad, (__nv_bfloat16*)wire, lo, n);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// The data-parallel optimizer step on flat offsets [lo, lo + n) (inside this rank's shard):
//   grad_mode      0: grad_ptrs[r] is rank r's fp32 gradient; 1: grad_ptrs[r] is rank r's bf16 wire copy and own_grad this
//                  rank's fp32 gradient (its own wire copy is never read); 2: own_grad is a local fp32 buffer of the
//                  shard's size that already holds the sum over the ranks (grad_ptrs is not read)
//   model_ptrs[r]  rank r's full bf16 weights
//   master/m/v     local shard; state_off = lo - shard start
//   max_ctas       > 0 caps the grid: a launch that runs beside the backward pass takes a few CTAs, not every SM
int b200_p2p_rs_adamw_ag(const void* const* grad_ptrs, const float* own_grad, int grad_mode, const void* const* model_ptrs,
                         float* master, float* m, float* v, long long lo, long long n, long long state_off, int rank,
                         int world, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                         float grad_scale, int decoupled, int max_ctas, cudaStream_t st) {
  Peers G, M;
  if (grad_mode < 0 || grad_mode > 2 || !fill(M, model_ptrs, world) || !master || !m || !v || n <= 0 || (n & 7) ||
      (lo & 7) || (state_off & 7) || state_off < 0 || step < 1 || (grad_mode && !own_grad))
    return B200_ERR_ARG;
  if (grad_mode == 2) G = M;   // the table is not read in this mode
  else if (!fill(G, grad_ptrs, world)) return B200_ERR_ARG;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
             grad_scale, decoupled};
  int grid = grid_for(n >> 3);
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
#define B200_RS_LAUNCH(MODE, WW) \
  rs_adamw_ag_kernel<MODE, WW><<<grid, 256, 0, st>>>(G, own_grad, M, master, m, v, lo, n, state_off, rank, world, a)
  if (grad_mode == 2) B200_RS_LAUNCH(2, 2);
  else if (grad_mode == 0) B200_RS_LAUNCH(0, 2);
  else if (world <= 2) B200_RS_LAUNCH(1, 2);
  else if (world <= 4) B200_RS_LAUNCH(1, 4);
  else if (world <= 8) B200_RS_LAUNCH(1, 8);
  else B200_RS_LAUNCH(1, 16);
#undef B200_RS_LAUNCH
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// max_ctas > 0 caps the grid (a reduction that runs beside the backward pass takes a few CTAs, not every SM)
int b200_p2p_reduce_scatter_f32(const void* const* src_ptrs, float* out, long long lo, long long n, int rank, int world,
                                float scale, int max_ctas, cudaStream_t st) {
  Peers S;
  if (!fill(S, src_ptrs, world) || !out || n <= 0 || (n & 3) || (lo & 3)) return B200_ERR_ARG;
  const int U = world <= 2 ? 8 : (world <= 4 ? 4 : (world <= 8 ? 2 : 1));
  int grid = grid_for(ceil_div_ll(n >> 2, (long long)U));
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (U == 8) reduce_scatter_kernel<8><<<grid, 256, 0, st>>>(S, out, lo, n, rank, world, scale);
  else if (U == 4) reduce_scatter_kernel<4><<<grid, 256, 0, st>>>(S, out, lo, n, rank, world, scale);
  else if (U == 2) reduce_scatter_kernel<2><<<grid, 256, 0, st>>>(S, out, lo, n, rank, world, scale);
  else reduce_scatter_kernel<1><<<grid, 256, 0, st>>>(S, out, lo, n, rank, world, scale);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// dst (world * piece_bytes, local) = concatenation over ranks p of src_ptrs[p][src_off_bytes .. + piece_bytes).
int b200_p2p_gather_pull(const void* const* src_ptrs, void* dst, long long src_off_bytes, long long piece_bytes, int rank,
                         int world, cudaStream_t st) {
  Peers S;
  if (!fill(S, src_ptrs, world) || !dst || piece_bytes <= 0 || (piece_bytes & 15) || (src_off_bytes & 15) || rank < 0 ||
      rank >= world)
    return B200_ERR_ARG;
  long long blocks = ((piece_bytes >> 4) + 256 * 8 - 1) / (256 * 8);
  const long long cap = (long long)sm_count() * 2;
  if (blocks > cap) blocks = cap;
  gather_pull_kernel<<<(int)blocks, 256, 0, st>>>(S, (uint4*)dst, src_off_bytes >> 4, piece_bytes >> 4, rank, world);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// grad_ptrs[r]: rank r's unit-sized fp32 gradient buffer; this rank's slice of it starts at grad_lo. acc (nullable),
// model (bf16), master, m, v: this rank's piece of the unit, n elements (multiple of 8).
int b200_p2p_rs_adamw_piece(const void* const* grad_ptrs, long long grad_lo, const float* acc, void* model, float* master,
                            float* m, float* v, long long n, int rank, int world, float lr, float beta1, float beta2,
                            float eps, float weight_decay, int step, float grad_scale, int decoupled, cudaStream_t st) {
  Peers G;
  if (!fill(G, grad_ptrs, world) || !model || !master || !m || !v || n <= 0 || (n & 7) || (grad_lo & 7) || step < 1)
    return B200_ERR_ARG;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
             grad_scale, decoupled};
  rs_adamw_piece_kernel<<<grid_for(n >> 3), 256, 0, st>>>(G, grad_lo, acc, (__nv_bfloat16*)model, master, m, v, n, rank,
                                                         world, a);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_p2p_reduce_scatter_acc_f32(const void* const* src_ptrs, float* out, long long lo, long long n, int rank,
                                    int world, int accumulate, cudaStream_t st) {
  Peers S;
  if (!fill(S, src_ptrs, world) || !out || n <= 0 || (n & 3) || (lo & 3)) return B200_ERR_ARG;
  reduce_scatter_acc_kernel<<<grid_for(n >> 2), 256, 0, st>>>(S, out, lo, n, rank, world, accumulate);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// Copies nbytes (multiple of 16) from `local` into every rank's buffer at byte offset lo_bytes.
int b200_p2p_allgather(const void* const* dst_ptrs, const void* local, long long lo_bytes, long long nbytes, int rank,
                       int world, int skip_self, cudaStream_t st) {
  Peers D;
  if (!fill(D, dst_ptrs, world) || !local || nbytes <= 0 || (nbytes & 15) || (lo_bytes & 15)) return B200_ERR_ARG;
  allgather_kernel<<<grid_for(nbytes >> 4), 256, 0, st>>>(D, (const uint4*)local, lo_bytes >> 4, nbytes >> 4, rank, world,
                                                         skip_self);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
}
