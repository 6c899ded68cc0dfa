// Exact per-row top-K of log_softmax(logits[:, :V]) for teacher collection, and the multi-teacher top-K merge.
//
// topk_logprob: one CTA per row over fp32 logits (the row chunk just written by the LM-head GEMM, L2 resident):
//   1. one read: max, sum-exp -> lse, and a histogram of the upper 11 bits of the order-preserving keys
//   2. second read: everything above the K-th element's bin is selected, the bin itself becomes a candidate list in
//      shared memory, which three small radix passes narrow to the exact K-th value and the number of ties to keep
//   3. the lowest-index ties complete the selection
//   4. bitonic sort in shared memory by (value desc, index asc) - the order torch.topk users expect
//   5. write fp16 log-probs (value - lse) and int32 ids
// Output layout matches the HDF5 datasets: [rows, K] fp16 + [rows, K] int32.
//
// topk_merge: per row, union of two top-K lists with probabilities of equal ids summed, best K kept, log stored
// (the multi-teacher rule of the data store), sorted by value.
#include "../common/ptx.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace topk {

constexpr int NT = 256;
constexpr int MAX_K = 1024;
constexpr int TIE_CAP = 1024;

__device__ __forceinline__ uint32_t fkey(float x) {
  uint32_t k = __float_as_uint(x);
  return (k & 0x80000000u) ? ~k : (k | 0x80000000u);
}
__device__ __forceinline__ float kfloat(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// descending bitonic sort of n (power of two) 64-bit keys in shared memory
__device__ void bitonic_desc(unsigned long long* s, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const unsigned long long a = s[i], b = s[ixj];
          const bool desc = ((i & k) == 0);
          if (desc ? (a < b) : (a > b)) { s[i] = b; s[ixj] = a; }
        }
      }
      __syncthreads();
    }
  }
}

// Block-wide search in a histogram whose bins are ordered by value: the bin that holds the `want`-th largest element
// (want >= 1, and the histogram holds at least `want` elements). Thread t owns the PER bins just below those of thread
// t - 1, thread 0 the highest ones; an inclusive scan over the threads gives every thread the number of elements above
// its bins. Results go to shared memory: the bin, how many elements lie in higher bins, how many in the bin itself.
// Ends with a block-wide barrier.
template <int PER>
__device__ __forceinline__ void find_kth_bin(const unsigned int* hist, unsigned want, unsigned int* redu,
                                             unsigned int* s_bin, unsigned int* s_above, unsigned int* s_inbin) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int base = NT * PER - PER * (tid + 1);
  unsigned loc = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) loc += hist[base + j];
  unsigned inc = loc;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  if (lane == 31) redu[warp] = inc;
  __syncthreads();
  for (int w = 0; w < warp; ++w) inc += redu[w];
  const unsigned above = inc - loc;
  if (above < want && want <= inc) {
    unsigned cum = above;
    int bin = base + PER - 1;
    for (; bin > base; --bin) {
      if (cum + hist[bin] >= want) break;
      cum += hist[bin];
    }
    *s_bin = (unsigned)bin; *s_above = cum; *s_inbin = hist[bin];
  }
  __syncthreads();
}

// f(value, index) for every index in [lo, hi) of a row, the block's threads striding over it; 16-byte loads when the
// row pointer allows (lo must be a multiple of 4 then, which the callers' constants are).
template <class F>
__device__ __forceinline__ void for_row(const float* __restrict__ x, int lo, int hi, F f) {
  const int tid = threadIdx.x;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (lo & 3) == 0) {
    const int hi4 = lo + ((hi - lo) & ~3);
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int i = (lo >> 2) + tid; i < (hi4 >> 2); i += NT) {
      const float4 v = x4[i];
      f(v.x, 4 * i); f(v.y, 4 * i + 1); f(v.z, 4 * i + 2); f(v.w, 4 * i + 3);
    }
    for (int i = hi4 + tid; i < hi; i += NT) f(x[i], i);
  } else {
    for (int i = lo + tid; i < hi; i += NT) f(x[i], i);
  }
}

constexpr int HB = 11;               // bits of the first histogram: sign, exponent, two bits of the mantissa
constexpr int NBIN = 1 << HB;        // = NT * 8
constexpr int CAND_CAP = 1024;       // elements of the threshold bin that are kept in shared memory
constexpr int SAMPLE = 4096;         // leading elements whose K-th largest bounds the row's K-th largest from below

// Two reads of the row. Read 1: running (max, sum-exp) per thread and a histogram of the upper 11 key bits; the first
// 4096 elements go first, and since the K-th largest of a subset is a lower bound of the K-th largest of the row, the
// rest of the row only enters the histogram from that bin up (a few per cent of it: the shared-memory atomics were
// the cost of the one-pass histogram). The histogram gives the bin b of the K-th largest element. Read 2: elements of
// higher bins are selected, those of bin b (typically 100-200) become candidates in shared memory, and three small
// radix passes over the candidates' remaining 21 key bits give the exact threshold and the number of ties to keep.
// A bin with more than CAND_CAP elements falls back to radix passes over the row.
//
// Vocabulary-shard mode (out_raw != null): the row is one rank's slice of the vocabulary; the kernel writes the raw
// fp32 logits of the slice's top K, their GLOBAL ids (index + id_offset) and the slice's log-sum-exp, which
// topk_combine_kernel turns into the exact top-K log-probs of the whole vocabulary.
__global__ void __launch_bounds__(NT) topk_logprob_kernel(const float* __restrict__ logits, long long ld, int V, int K,
                                                         __half* __restrict__ out_logp, int* __restrict__ out_idx,
                                                         float* __restrict__ out_raw, float* __restrict__ out_lse,
                                                         int id_offset) {
  static_assert(NBIN == NT * 8, "find_kth_bin<8> covers the first histogram");
  __shared__ unsigned long long sel[MAX_K];
  __shared__ unsigned long long cand[CAND_CAP];
  __shared__ unsigned int hist[NBIN];
  __shared__ unsigned int ties[TIE_CAP];
  __shared__ float redm[NT / 32], reds[NT / 32];
  __shared__ unsigned int redu[NT / 32];
  __shared__ unsigned int s_bin, s_above, s_inbin, s_nsel, s_ncand, s_nties;
  __shared__ float s_lse;
  const long long row = blockIdx.x;
  const float* x = logits + row * ld;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < NBIN; i += NT) hist[i] = 0;
  if (tid == 0) { s_nsel = 0; s_ncand = 0; s_nties = 0; }
  __syncthreads();

  // ---- read 1: max, sum-exp, histogram
  float m = -INFINITY, sum = 0.f;
  auto stat = [&](float v) {
    if (v > m) { sum *= __expf(m - v); m = v; }
    if (v > -INFINITY) sum += __expf(v - m);
  };
  const int n_sample = V >= 4 * SAMPLE ? SAMPLE : 0;
  unsigned lb_bin = 0;
  if (n_sample) {
    for_row(x, 0, n_sample, [&](float v, int) {
      stat(v);
      atomicAdd(&hist[fkey(v) >> (32 - HB)], 1u);
    });
    __syncthreads();
    find_kth_bin<8>(hist, (unsigned)K, redu, &s_bin, &s_above, &s_inbin);
    lb_bin = s_bin;
    __syncthreads();
  }
  for_row(x, n_sample, V, [&](float v, int) {
    stat(v);
    const unsigned bin = fkey(v) >> (32 - HB);
    if (bin >= lb_bin) atomicAdd(&hist[bin], 1u);
  });
  {
    const float wm = warp_max(m);
    const float part = (m > -INFINITY) ? sum * __expf(m - wm) : 0.f;
    const float ws = warp_sum(part);
    if (lane == 0) { redm[warp] = wm; reds[warp] = ws; }
  }
  __syncthreads();
  if (tid == 0) {
    float M = redm[0];
    for (int w = 1; w < NT / 32; ++w) M = fmaxf(M, redm[w]);
    float t = 0.f;
    for (int w = 0; w < NT / 32; ++w)
      if (redm[w] > -INFINITY) t += reds[w] * __expf(redm[w] - M);
    s_lse = M + __logf(t);
  }
  find_kth_bin<8>(hist, (unsigned)K, redu, &s_bin, &s_above, &s_inbin);
  const unsigned bstar = s_bin;
  const unsigned n_inbin = s_inbin;
  unsigned remaining = (unsigned)K - s_above;       // how many elements of bin bstar belong to the top K (>= 1)
  const bool in_smem = n_inbin <= (unsigned)CAND_CAP;

  // ---- read 2: higher bins are in; bin bstar becomes the candidate list
  for_row(x, 0, V, [&](float v, int i) {
    const uint32_t k = fkey(v);
    const unsigned bin = k >> (32 - HB);
    if (bin > bstar) {
      sel[atomicAdd(&s_nsel, 1u)] = ((unsigned long long)k << 32) | (0xffffffffu - (uint32_t)i);
    } else if (bin == bstar && in_smem) {
      cand[atomicAdd(&s_ncand, 1u)] = ((unsigned long long)k << 32) | (0xffffffffu - (uint32_t)i);
    }
  });
  __syncthreads();

  // f(key, index) for every element of bin bstar
  auto for_bin = [&](auto f) {
    if (in_smem) {
      for (unsigned c = tid; c < n_inbin; c += NT) {
        const unsigned long long e = cand[c];
        f((uint32_t)(e >> 32), 0xffffffffu - (uint32_t)(e & 0xffffffffu));
      }
    } else {
      for_row(x, 0, V, [&](float v, int i) {
        const uint32_t k = fkey(v);
        if ((k >> (32 - HB)) == bstar) f(k, (uint32_t)i);
      });
    }
  };

  // ---- the remaining 21 key bits: 8 + 8 + 5
  uint32_t prefix = bstar << (32 - HB), mask = 0xffffffffu << (32 - HB);
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 13 : (pass == 1 ? 5 : 0);
    const uint32_t digit = pass == 2 ? 0x1fu : 0xffu;
    hist[tid] = 0;
    __syncthreads();
    for_bin([&](uint32_t k, uint32_t) {
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & digit], 1u);
    });
    __syncthreads();
    find_kth_bin<1>(hist, remaining, redu, &s_bin, &s_above, &s_inbin);
    prefix |= s_bin << shift;
    mask |= digit << shift;
    remaining -= s_above;
    __syncthreads();
  }
  const uint32_t thr = prefix;            // key of the K-th largest element
  const unsigned need_eq = remaining;     // how many elements equal to it belong to the top K

  // ---- gather from bin bstar
  for_bin([&](uint32_t k, uint32_t i) {
    if (k > thr) {
      sel[atomicAdd(&s_nsel, 1u)] = ((unsigned long long)k << 32) | (0xffffffffu - i);
    } else if (k == thr) {
      const unsigned p = atomicAdd(&s_nties, 1u);
      if (p < TIE_CAP) ties[p] = i;
    }
  });
  __syncthreads();
  const unsigned ngt = s_nsel;
  const unsigned nt = s_nties;
  if (nt > TIE_CAP) {
    // pathological row (more than TIE_CAP equal values at the threshold): ordered sequential pick
    if (tid == 0) {
      unsigned got = 0;
      for (int i = 0; i < V && got < need_eq; ++i)
        if (fkey(x[i]) == thr) sel[ngt + got++] = ((unsigned long long)thr << 32) | (0xffffffffu - (uint32_t)i);
    }
  } else {
    // keep the need_eq lowest indices among the ties: rank each tie by counting smaller indices
    for (unsigned t = tid; t < nt; t += NT) {
      const uint32_t me = ties[t];
      unsigned rank = 0;
      for (unsigned u = 0; u < nt; ++u) rank += (ties[u] < me) ? 1u : 0u;
      if (rank < need_eq) sel[ngt + rank] = ((unsigned long long)thr << 32) | (0xffffffffu - me);
    }
  }
  __syncthreads();

  // ---- sort (pad to a power of two with zeros, which sort last) and write
  int n2 = 1;
  while (n2 < K) n2 <<= 1;
  for (int i = K + tid; i < n2; i += NT) sel[i] = 0ull;
  __syncthreads();
  bitonic_desc(sel, n2);

  const float lse = s_lse;
  for (int i = tid; i < K; i += NT) {
    const unsigned long long e = sel[i];
    const float z = kfloat((uint32_t)(e >> 32));
    if (out_raw) out_raw[row * K + i] = z;
    else out_logp[row * K + i] = __float2half(z - lse);
    out_idx[row * K + i] = (int)(0xffffffffu - (uint32_t)(e & 0xffffffffu)) + id_offset;
  }
  if (out_lse && tid == 0) out_lse[row] = lse;
}

// Per row: `parts` vocabulary shards each delivered K (raw logit, global id) candidates and the shard's log-sum-exp
// (layout [parts][rows][K] and [parts][rows], part stride given in elements). Output: the K best of the parts*K
// candidates as fp16 log-probs under the whole-vocabulary log-sum-exp, ids int32; ties by lower id.
__global__ void __launch_bounds__(NT) topk_combine_kernel(const float* __restrict__ z, const int* __restrict__ ids,
                                                         const float* __restrict__ lse, long long zk_stride,
                                                         long long lse_stride, int parts, int K,
                                                         __half* __restrict__ out_logp, int* __restrict__ out_idx) {
  extern __shared__ unsigned long long cs[];
  __shared__ float s_glse;
  const long long row = blockIdx.x;
  const int n = parts * K;
  int n2 = 1;
  while (n2 < n) n2 <<= 1;
  if (threadIdx.x == 0) {
    float m = -INFINITY;
    for (int q = 0; q < parts; ++q) m = fmaxf(m, lse[q * lse_stride + row]);
    float t = 0.f;
    for (int q = 0; q < parts; ++q) t += __expf(lse[q * lse_stride + row] - m);
    s_glse = m + __logf(t);
  }
  for (int i = threadIdx.x; i < n2; i += NT) {
    unsigned long long e = 0ull;
    if (i < n) {
      const int q = i / K, j = i - q * K;
      const float v = z[q * zk_stride + row * K + j];
      const int id = ids[q * zk_stride + row * K + j];
      e = ((unsigned long long)fkey(v) << 32) | (0xffffffffu - (uint32_t)id);
    }
    cs[i] = e;
  }
  __syncthreads();
  bitonic_desc(cs, n2);
  const float g = s_glse;
  for (int i = threadIdx.x; i < K; i += NT) {
    const unsigned long long e = cs[i];
    out_logp[row * K + i] = __float2half(kfloat((uint32_t)(e >> 32)) - g);
    out_idx[row * K + i] = (int)(0xffffffffu - (uint32_t)(e & 0xffffffffu));
  }
}

// ---------------------------------------------------------------------------------------------- merge
// a_*, b_*: [rows, K] (log-prob fp32, id int32). out: union with summed probabilities, best K, sorted by value desc.
__global__ void __launch_bounds__(NT) topk_merge_kernel(const float* __restrict__ a_lp, const int* __restrict__ a_id,
                                                       const float* __restrict__ b_lp, const int* __restrict__ b_id,
                                                       int K, float* __restrict__ o_lp, int* __restrict__ o_id) {
  __shared__ unsigned long long s[2 * MAX_K];
  __shared__ float pv[2 * MAX_K];
  const long long row = blockIdx.x;
  const int n = 2 * K;
  int n2 = 1;
  while (n2 < n) n2 <<= 1;
  // sort by id (key = id << 32 | slot), carrying probabilities in pv[slot]
  for (int i = threadIdx.x; i < n2; i += NT) {
    if (i < n) {
      const bool first = i < K;
      int id = first ? a_id[row * K + i] : b_id[row * K + i - K];
      pv[i] = __expf(first ? a_lp[row * K + i] : b_lp[row * K + i - K]);
      // an empty slot (log-prob -inf, id 0) carries no mass; it gets an id of its own above every vocabulary so that
      // it never sits between a real token 0 of one list and of the other (equal ids are summed in PAIRS below)
      if (!(pv[i] > 0.f)) id = 0x7f000000 + i;
      s[i] = ((unsigned long long)(uint32_t)id << 32) | (uint32_t)i;
    } else {
      s[i] = 0ull;
    }
  }
  __syncthreads();
  bitonic_desc(s, n2);  // equal ids are now adjacent (descending id), padding zeros last... id 0 handled via slot
  __syncthreads();
  // combine duplicates: the first of an equal-id pair takes the sum, the second is dropped
  __shared__ float comb[2 * MAX_K];
  for (int i = threadIdx.x; i < n; i += NT) {
    const uint32_t id = (uint32_t)(s[i] >> 32);
    const float p = pv[(uint32_t)s[i]];
    const bool dup_prev = (i > 0) && ((uint32_t)(s[i - 1] >> 32) == id);
    const bool dup_next = (i + 1 < n) && ((uint32_t)(s[i + 1] >> 32) == id);
    comb[i] = dup_prev ? -1.f : (dup_next ? p + pv[(uint32_t)s[i + 1]] : p);
  }
  __syncthreads();
  // re-key by probability (desc), tie-break by lower id
  for (int i = threadIdx.x; i < n2; i += NT) {
    if (i < n && comb[i] >= 0.f) {
      const uint32_t id = (uint32_t)(s[i] >> 32);
      s[i] = ((unsigned long long)fkey(comb[i]) << 32) | (0xffffffffu - id);
    } else {
      s[i] = 0ull;
    }
  }
  __syncthreads();
  bitonic_desc(s, n2);
  for (int i = threadIdx.x; i < K; i += NT) {
    const unsigned long long e = s[i];
    const float p = e ? kfloat((uint32_t)(e >> 32)) : 0.f;
    o_lp[row * K + i] = __logf(p);
    const int oid = e ? (int)(0xffffffffu - (uint32_t)e) : 0;
    o_id[row * K + i] = (p > 0.f && oid < 0x7f000000) ? oid : 0;
  }
}

static int launch_topk(const float* logits, long long ld, int rows, int V, int K, __half* out_logp, int* out_idx,
                       float* out_raw, float* out_lse, int id_offset, cudaStream_t st) {
  topk_logprob_kernel<<<rows, NT, 0, st>>>(logits, ld, V, K, out_logp, out_idx, out_raw, out_lse, id_offset);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

}  // namespace topk
}  // namespace b200

extern "C" {
using namespace b200;

// logits: fp32 [rows, >=V] with row stride ld (elements). out_logp fp16 [rows, K], out_idx int32 [rows, K].
int b200_topk_logprob(const float* logits, long long ld, int rows, int V, int K, void* out_logp, int* out_idx,
                      cudaStream_t st) {
  if (!logits || !out_logp || !out_idx || rows <= 0 || V <= 0 || K <= 0 || K > topk::MAX_K || K > V)
    return K > topk::MAX_K ? B200_ERR_TOO_BIG : B200_ERR_ARG;
  return topk::launch_topk(logits, ld, rows, V, K, (__half*)out_logp, out_idx, nullptr, nullptr, 0, st);
}

// One vocabulary shard of a vocabulary-parallel LM head: raw top-K logits fp32 [rows, K], global ids, shard lse [rows].
int b200_topk_partial(const float* logits, long long ld, int rows, int V, int K, int id_offset, float* out_raw,
                      int* out_idx, float* out_lse, cudaStream_t st) {
  if (!logits || !out_raw || !out_idx || !out_lse || rows <= 0 || V <= 0 || K <= 0 || K > topk::MAX_K || K > V)
    return K > topk::MAX_K ? B200_ERR_TOO_BIG : B200_ERR_ARG;
  return topk::launch_topk(logits, ld, rows, V, K, nullptr, out_idx, out_raw, out_lse, id_offset, st);
}

// Merge of `parts` shard results (see topk_combine_kernel). zk_stride / lse_stride: elements between parts.
int b200_topk_combine(const float* z, const int* ids, const float* lse, long long zk_stride, long long lse_stride,
                      int parts, int rows, int K, void* out_logp, int* out_idx, cudaStream_t st) {
  if (!z || !ids || !lse || !out_logp || !out_idx || parts <= 0 || rows <= 0 || K <= 0) return B200_ERR_ARG;
  int n2 = 1;
  while (n2 < parts * K) n2 <<= 1;
  const int smem = n2 * 8;
  if (smem > 200 * 1024) return B200_ERR_TOO_BIG;
  if (smem > 48 * 1024)
    B200_CUDA_CHECK(cudaFuncSetAttribute(topk::topk_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  topk::topk_combine_kernel<<<rows, topk::NT, smem, st>>>(z, ids, lse, zk_stride, lse_stride, parts, K,
                                                         (__half*)out_logp, out_idx);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_topk_merge(const float* a_lp, const int* a_id, const float* b_lp, const int* b_id, int rows, int K,
                    float* o_lp, int* o_id, cudaStream_t st) {
  if (!a_lp || !a_id || !b_lp || !b_id || !o_lp || !o_id || rows <= 0 || K <= 0 || K > topk::MAX_K)
    return K > topk::MAX_K ? B200_ERR_TOO_BIG : B200_ERR_ARG;
  topk::topk_merge_kernel<<<rows, topk::NT, 0, st>>>(a_lp, a_id, b_lp, b_id, K, o_lp, o_id);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
}

namespace b200 {
namespace topk {
// out[row, j] = fp16(x[row, j] - lse(row))  for j < V : full-vocabulary log-probabilities (top-K storage disabled)
__global__ void __launch_bounds__(NT) logprob_full_kernel(const float* __restrict__ logits, long long ld, int V,
                                                         __half* __restrict__ out, long long ldo) {
  __shared__ float redf[NT / 32];
  __shared__ float s_max, s_lse;
  const long long row = blockIdx.x;
  const float* x = logits + row * ld;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float mx = -INFINITY;
  for (int i = tid; i < V; i += NT) mx = fmaxf(mx, x[i]);
  mx = warp_max(mx);
  if (lane == 0) redf[warp] = mx;
  __syncthreads();
  if (tid == 0) { float m = redf[0]; for (int w = 1; w < NT / 32; ++w) m = fmaxf(m, redf[w]); s_max = m; }
  __syncthreads();
  mx = s_max;
  float sm = 0.f;
  for (int i = tid; i < V; i += NT) sm += __expf(x[i] - mx);
  sm = warp_sum(sm);
  __syncthreads();
  if (lane == 0) redf[warp] = sm;
  __syncthreads();
  if (tid == 0) { float t = 0.f; for (int w = 0; w < NT / 32; ++w) t += redf[w]; s_lse = mx + __logf(t); }
  __syncthreads();
  const float lse = s_lse;
  for (int i = tid; i < V; i += NT) out[row * ldo + i] = __float2half(x[i] - lse);
}
}  // namespace topk
}  // namespace b200

extern "C" int b200_logprob_full(const float* logits, long long ld, int rows, int V, void* out, long long ldo,
                                 cudaStream_t st) {
  using namespace b200;
  if (!logits || !out || rows <= 0 || V <= 0) return B200_ERR_ARG;
  topk::logprob_full_kernel<<<rows, topk::NT, 0, st>>>(logits, ld, V, (__half*)out, ldo);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// ---------------------------------------------------------------------------------------------- vocabulary remap
// Cross-tokenizer marginalisation of one teacher's top-K rows onto the student vocabulary: every teacher id is
// sent through `table` (teacher id -> student id, -1 = no image), probabilities that land on the same student id
// are summed, the best K_out are kept and written as (log-prob, id) sorted by probability. Entries without an image
// (or with a non-finite log-prob) drop out; unused output slots get -inf and id 0.
namespace b200 {
namespace topk {
__global__ void __launch_bounds__(NT) remap_topk_kernel(const float* __restrict__ lp, const int* __restrict__ ids,
                                                       const int* __restrict__ table, int table_size, int K, int K_out,
                                                       float* __restrict__ o_lp, int* __restrict__ o_id) {
  __shared__ unsigned long long s[MAX_K];
  __shared__ float pv[MAX_K];
  __shared__ float comb[MAX_K];
  const long long row = blockIdx.x;
  int n2 = 1;
  while (n2 < K) n2 <<= 1;
  for (int i = threadIdx.x; i < n2; i += NT) {
    unsigned long long key = 0ull;
    if (i < K) {
      const int t = ids[row * K + i];
      const float l = lp[row * K + i];
      const int sid = (t >= 0 && t < table_size) ? table[t] : -1;
      pv[i] = (sid >= 0 && l > -1e30f) ? __expf(l) : 0.f;
      // key: (student id + 1) so that "no image" (0) sorts last together with the padding
      key = (sid >= 0 && l > -1e30f) ? (((unsigned long long)(uint32_t)(sid + 1) << 32) | (uint32_t)i) : 0ull;
    }
    s[i] = key;
  }
  __syncthreads();
  bitonic_desc(s, n2);
  // run heads take the sum of their run (runs can be longer than two here)
  for (int i = threadIdx.x; i < n2; i += NT) {
    const unsigned long long e = s[i];
    float c = -1.f;
    if (e != 0ull) {
      const uint32_t id = (uint32_t)(e >> 32);
      if (i == 0 || (uint32_t)(s[i - 1] >> 32) != id) {
        c = 0.f;
        for (int j = i; j < n2 && (uint32_t)(s[j] >> 32) == id; ++j) c += pv[(uint32_t)s[j]];
      }
    }
    comb[i] = c;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n2; i += NT) {
    const unsigned long long e = s[i];
    const float c = comb[i];
    __syncwarp();
    s[i] = (c >= 0.f) ? (((unsigned long long)fkey(c) << 32) | (0xffffffffu - ((uint32_t)(e >> 32) - 1u))) : 0ull;
  }
  __syncthreads();
  bitonic_desc(s, n2);
  for (int i = threadIdx.x; i < K_out; i += NT) {
    const unsigned long long e = i < n2 ? s[i] : 0ull;
    o_lp[row * K_out + i] = e ? __logf(kfloat((uint32_t)(e >> 32))) : -INFINITY;
    o_id[row * K_out + i] = e ? (int)(0xffffffffu - (uint32_t)e) : 0;
  }
}
}  // namespace topk
}  // namespace b200

extern "C" int b200_remap_topk(const float* lp, const int* ids, const int* table, int table_size, int rows, int K,
                               int K_out, float* o_lp, int* o_id, cudaStream_t st) {
  using namespace b200;
  if (!lp || !ids || !table || !o_lp || !o_id || rows <= 0 || K <= 0 || K_out <= 0 || table_size <= 0)
    return B200_ERR_ARG;
  if (K > topk::MAX_K || K_out > topk::MAX_K) return B200_ERR_TOO_BIG;
  topk::remap_topk_kernel<<<rows, topk::NT, 0, st>>>(lp, ids, table, table_size, K, K_out, o_lp, o_id);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
