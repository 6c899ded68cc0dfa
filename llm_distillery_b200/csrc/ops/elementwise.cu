// Bandwidth-bound transformer ops for sm_100a: RMSNorm (+ fused residual add) fwd/bwd, rotary
// embedding fwd/bwd (in place), SwiGLU fwd/bwd, embedding gather / scatter-add, dtype casts.
// All tensors are bf16 unless stated; statistics and weight gradients are fp32.
// Every kernel moves 16-byte vectors and keeps the row it works on in registers between passes,
// so each element crosses HBM once per direction.
#include "../common/ptx.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace ew {

constexpr int NT = 256;
constexpr int MAX_VEC = 4;  // 16-byte vectors cached per thread: rows up to NT*MAX_VEC*8 = 8192 elements

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (NT / 32)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    float2 x = __bfloat1622float2(h[t]);
    f[2 * t] = x.x;
    f[2 * t + 1] = x.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  return o;
}

// y = rmsnorm(x (+ res)) * w ; if res != null also writes h = x + res to `hout`. rstd[row] saved for backward.
__global__ void __launch_bounds__(NT) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ res,
                                                        const __nv_bfloat16* __restrict__ w,
                                                        __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ hout,
                                                        float* __restrict__ rstd, int rows, int h, float eps) {
  __shared__ float red[NT / 32];
  const int nvec = h >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * h);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * h) : nullptr;
    float vals[MAX_VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NT;
      if (v < nvec) {
        unpack8(xr[v], vals[i]);
        if (rr) {
          float r8[8];
          unpack8(rr[v], r8);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += r8[j];
          if (hout) {
            // the residual stream is stored in bf16: normalise what is stored, not the fp32 sum
            uint4 hq = pack8(vals[i]);
            reinterpret_cast<uint4*>(hout + (size_t)row * h)[v] = hq;
            unpack8(hq, vals[i]);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    const float tot = block_sum(ss, red);
    const float rs = rsqrtf(tot / (float)h + eps);
    if (threadIdx.x == 0 && rstd) rstd[row] = rs;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NT;
      if (v < nvec) {
        float w8[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(w)[v], w8);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rs * w8[j];
        reinterpret_cast<uint4*>(y + (size_t)row * h)[v] = pack8(o);
      }
    }
  }
}

// 16-byte read-only load that the compiler may not hoist out of a loop (keeps loop-invariant vectors in L1, not in
// registers).
__device__ __forceinline__ uint4 ld_nc_v4_nohoist(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// One WARP per row (h = VPL * 256): the row stays in registers, the reduction is a warp shuffle, no block barrier.
template <int VPL>
__global__ void __launch_bounds__(128) rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x,
                                                              const __nv_bfloat16* __restrict__ res,
                                                              const __nv_bfloat16* __restrict__ w,
                                                              __nv_bfloat16* __restrict__ y,
                                                              __nv_bfloat16* __restrict__ hout,
                                                              float* __restrict__ rstd, int rows, float eps) {
  constexpr int h = VPL * 256;
  const int lane = threadIdx.x & 31;
  const int nwarps = gridDim.x * 4;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x * 4 + (threadIdx.x >> 5); row < rows; row += nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * h);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * h) : nullptr;
    uint4 q[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) q[i] = xr[lane + 32 * i];
    if (rr) {
      uint4 r[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) r[i] = rr[lane + 32 * i];
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        float a[8], b[8];
        unpack8(q[i], a);
        unpack8(r[i], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] += b[j];
        q[i] = pack8(a);  // the residual stream is stored in bf16: normalise what is stored, not the fp32 sum
        if (hout) reinterpret_cast<uint4*>(hout + (size_t)row * h)[lane + 32 * i] = q[i];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float a[8];
      unpack8(q[i], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += a[j] * a[j];
    }
    const float rs = rsqrtf(warp_sum(ss) * (1.f / (float)h) + eps);
    if (lane == 0 && rstd) rstd[row] = rs;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * h);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float a[8], w8[8], o[8];
      unpack8(q[i], a);
      unpack8(ld_nc_v4_nohoist(wv + lane + 32 * i), w8);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = a[j] * rs * w8[j];
      yr[lane + 32 * i] = pack8(o);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres) ; dw partial sums per block in fp32.
__global__ void __launch_bounds__(NT) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                        const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ w,
                                                        const float* __restrict__ rstd,
                                                        const __nv_bfloat16* __restrict__ dres,
                                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial,
                                                        int rows, int h) {
  __shared__ float red[NT / 32];
  const int nvec = h >> 3;
  float dwacc[MAX_VEC][8];
  float w8[MAX_VEC][8];
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int v = threadIdx.x + i * NT;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (v < nvec) unpack8(reinterpret_cast<const uint4*>(w)[v], w8[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    float xh[MAX_VEC][8], g[MAX_VEC][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NT;
      if (v < nvec) {
        float d8[8];
        unpack8(reinterpret_cast<const uint4*>(x + (size_t)row * h)[v], xh[i]);
        unpack8(reinterpret_cast<const uint4*>(dy + (size_t)row * h)[v], d8);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rs;
          dwacc[i][j] += d8[j] * xh[i][j];
          g[i][j] = d8[j] * w8[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    const float c = block_sum(dot, red) / (float)h;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NT;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - xh[i][j] * c);
        if (dres) {
          float r8[8];
          unpack8(reinterpret_cast<const uint4*>(dres + (size_t)row * h)[v], r8);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r8[j];
        }
        reinterpret_cast<uint4*>(dx + (size_t)row * h)[v] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int v = threadIdx.x + i * NT;
    if (v < nvec) {
      float* p = dw_partial + (size_t)blockIdx.x * h + (size_t)v * 8;
      *reinterpret_cast<float4*>(p) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// Second read of a vector this thread loaded a moment ago (volatile: the compiler may not merge it with the first).
__device__ __forceinline__ uint4 ld_cg_v4_again(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Same computation with one WARP per row (h = VPL * 256): no block barriers, 2 * VPL 16-byte loads in flight per
// lane, the second sweep re-reading the row through the caches, and the warp's running weight-gradient sums
// in shared memory (h floats per warp, split into two planes so that every access is a conflict-free float4).
// At the end the CTA's four warps add their sums and the CTA writes ONE row of dw_partial (the column-sum kernel
// behind it then reads a quarter of the bytes: it has only h / 32 CTAs and was 1.5 % of a training step).
template <int VPL>
__global__ void __launch_bounds__(128, 5) rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy,
                                                              const __nv_bfloat16* __restrict__ x,
                                                              const __nv_bfloat16* __restrict__ w,
                                                              const float* __restrict__ rstd,
                                                              const __nv_bfloat16* __restrict__ dres,
                                                              __nv_bfloat16* __restrict__ dx,
                                                              float* __restrict__ dw_partial, int rows, int nwarps) {
  constexpr int h = VPL * 256;
  extern __shared__ float4 sdw_all[];
  const int lane = threadIdx.x & 31;
  const int gw = blockIdx.x * 4 + (threadIdx.x >> 5);
  float4* lo = sdw_all + (threadIdx.x >> 5) * (h / 4);  // plane 0: elements 0-3 of every 8-vector
  float4* hi = lo + h / 8;                                // plane 1: elements 4-7
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    lo[lane + 32 * i] = make_float4(0.f, 0.f, 0.f, 0.f);
    hi[lane + 32 * i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  for (int row = gw < nwarps ? gw : rows; row < rows; row += nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * h);
    const uint4* dr = reinterpret_cast<const uint4*>(dy + (size_t)row * h);
    const float rs = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float xf[8], df[8], wf[8];
      unpack8(xr[lane + 32 * i], xf);
      unpack8(dr[lane + 32 * i], df);
      unpack8(ld_nc_v4_nohoist(wv + lane + 32 * i), wf);
      float4 a = lo[lane + 32 * i], b = hi[lane + 32 * i];
      float t[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = xf[j] * rs;
        t[j] = df[j] * xh;
        dot += df[j] * wf[j] * xh;
      }
      a.x += t[0]; a.y += t[1]; a.z += t[2]; a.w += t[3];
      b.x += t[4]; b.y += t[5]; b.z += t[6]; b.w += t[7];
      lo[lane + 32 * i] = a;
      hi[lane + 32 * i] = b;
    }
    const float c = warp_sum(dot) * (1.f / (float)h);
    // second sweep: the row comes back from L1/L2 (it was read a moment ago), which costs no HBM traffic and keeps
    // the register count low enough for many rows in flight per SM
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + (size_t)row * h) : nullptr;
    uint4* outr = reinterpret_cast<uint4*>(dx + (size_t)row * h);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float xf[8], df[8], wf[8], o[8];
      unpack8(ld_cg_v4_again(xr + lane + 32 * i), xf);
      unpack8(ld_cg_v4_again(dr + lane + 32 * i), df);
      unpack8(ld_nc_v4_nohoist(wv + lane + 32 * i), wf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (df[j] * wf[j] - xf[j] * rs * c);
      if (rr) {
        float r8[8];
        unpack8(rr[lane + 32 * i], r8);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r8[j];
      }
      outr[lane + 32 * i] = pack8(o);
    }
  }
  __syncthreads();
  // q < h/8: plane 0 (elements 8q .. 8q+3); q >= h/8: plane 1 (elements 8(q - h/8) + 4 .. + 7)
  for (int q = threadIdx.x; q < h / 4; q += 128) {
    float4 s4 = sdw_all[q];
#pragma unroll
    for (int wi = 1; wi < 4; ++wi) {
      const float4 t = sdw_all[wi * (h / 4) + q];
      s4.x += t.x; s4.y += t.y; s4.z += t.z; s4.w += t.w;
    }
    const int col = q < h / 8 ? 8 * q : 8 * (q - h / 8) + 4;
    *reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * h + col) = s4;
  }
}

// out[j] (+)= sum_b partial[b][j]; block = 32 columns x 8 row groups, reduced through shared memory
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                     int nblk, int h, int accumulate) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (j < h)
    for (int b = ty; b < nblk; b += 8) s += partial[(size_t)b * h + j];
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < h) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][tx];
    out[j] = accumulate ? out[j] + t : t;
  }
}

// Per-head RMSNorm of the query and key heads of a fused qkv row (Qwen3: q_norm / k_norm, applied before the rotary
// embedding): y = x * rsqrt(mean_d x^2 + eps) * w, with one weight vector of d elements for all query heads and one
// for all key heads; value heads are copied. One warp per (token, head), EPL = d / 32 elements per lane, so a head is
// one 64- or 128-... byte access per lane pair and the reduction over d is a butterfly. rstd [T, H + Hkv] is kept
// for the backward pass.
template <int EPL>
__global__ void __launch_bounds__(256) headnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          __nv_bfloat16* __restrict__ y,
                                                          const __nv_bfloat16* __restrict__ wq,
                                                          const __nv_bfloat16* __restrict__ wk,
                                                          float* __restrict__ rstd, long long T, int H, int Hkv,
                                                          long long ld, float eps) {
  constexpr int d = EPL * 32;
  const int lane = threadIdx.x & 31;
  const int nh = H + 2 * Hkv, nn = H + Hkv;
  const long long items = T * nh;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long it = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; it < items; it += warps) {
    const long long t = it / nh;
    const int hd = (int)(it - t * nh);
    const __nv_bfloat16* xp = x + t * ld + (long long)hd * d + lane * EPL;
    __nv_bfloat16* yp = y + t * ld + (long long)hd * d + lane * EPL;
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; j += 2) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xp + j));
      v[j] = f.x; v[j + 1] = f.y;
    }
    if (hd < nn) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) ss += v[j] * v[j];
      ss = warp_sum(ss);
      const float rs = rsqrtf(ss * (1.f / (float)d) + eps);
      if (lane == 0) rstd[t * nn + hd] = rs;
      const __nv_bfloat16* w = (hd < H ? wq : wk) + lane * EPL;
#pragma unroll
      for (int j = 0; j < EPL; ++j) v[j] = v[j] * rs * __bfloat162float(w[j]);
    }
#pragma unroll
    for (int j = 0; j < EPL; j += 2)
      *reinterpret_cast<uint32_t*>(yp + j) = pack_bf16x2(v[j], v[j + 1]);
  }
}

// Backward of the above, in place on the gradient g of the normalised (un-rotated) qkv row: for query and key heads
// g <- rstd * (g w - xhat * mean_d(g w xhat)), xhat = x * rstd; value heads are left alone. The weight gradients
// sum_{token, head} g * xhat stay in registers over the warp's items (a lane always owns the same EPL elements),
// the block's warps add theirs through shared memory, and every block writes one row [dwq | dwk] of `partial`.
template <int EPL>
__global__ void __launch_bounds__(256) headnorm_bwd_kernel(__nv_bfloat16* __restrict__ g,
                                                          const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ wq,
                                                          const __nv_bfloat16* __restrict__ wk,
                                                          const float* __restrict__ rstd,
                                                          float* __restrict__ partial, long long T, int H, int Hkv,
                                                          long long ld) {
  constexpr int d = EPL * 32;
  __shared__ float sdw[8][2 * d];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nn = H + Hkv;
  const long long items = T * nn;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  float aq[EPL], ak[EPL], wqf[EPL], wkf[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    aq[j] = 0.f; ak[j] = 0.f;
    wqf[j] = __bfloat162float(wq[lane * EPL + j]);
    wkf[j] = __bfloat162float(wk[lane * EPL + j]);
  }
  for (long long it = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; it < items; it += warps) {
    const long long t = it / nn;
    const int hd = (int)(it - t * nn);
    const bool isq = hd < H;
    const __nv_bfloat16* xp = x + t * ld + (long long)hd * d + lane * EPL;
    __nv_bfloat16* gp = g + t * ld + (long long)hd * d + lane * EPL;
    const float rs = rstd[it];
    float xh[EPL], gw[EPL], gy[EPL];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; j += 2) {
      const float2 fx = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xp + j));
      const float2 fg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp + j));
      xh[j] = fx.x * rs; xh[j + 1] = fx.y * rs;
      gy[j] = fg.x; gy[j + 1] = fg.y;
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      gw[j] = gy[j] * (isq ? wqf[j] : wkf[j]);
      dot += gw[j] * xh[j];
      if (isq) aq[j] += gy[j] * xh[j]; else ak[j] += gy[j] * xh[j];
    }
    const float c = warp_sum(dot) * (1.f / (float)d);
    float o[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) o[j] = rs * (gw[j] - xh[j] * c);
#pragma unroll
    for (int j = 0; j < EPL; j += 2) *reinterpret_cast<uint32_t*>(gp + j) = pack_bf16x2(o[j], o[j + 1]);
  }
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    sdw[warp][lane * EPL + j] = aq[j];
    sdw[warp][d + lane * EPL + j] = ak[j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * d; c += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) t += sdw[w8][c];
    partial[(size_t)blockIdx.x * (2 * d) + c] = t;
  }
}

// Rotary embedding, HF Llama convention (pairs (i, i + d/2)), in place on x[T, nh, d].
// cos/sin tables are fp32 [max_pos, rot/2]; pos[t] gives the position of token t. sign = -1 runs the inverse rotation
// (the backward pass). rot <= d: only the first rot elements of a head rotate (partial rotary embeddings), element j
// pairing with j + rot/2; the rest of the head is left as it is.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ cs,
                            const float* __restrict__ sn, long long T, int nh, int d, int rot, long long row_stride,
                            float sign) {
  // one thread rotates 8 pairs: a 16-byte vector from each half of the rotated part
  const int half = rot >> 1;
  const int vecs_per_head = half >> 3;
  const int vecs_per_tok = nh * vecs_per_head;
  const long long total = T * vecs_per_tok;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vecs_per_tok;
    const int r = (int)(i - t * vecs_per_tok);
    const int hd = r / vecs_per_head;
    const int j = (r - hd * vecs_per_head) * 8;
    const int p = pos[t];
    __nv_bfloat16* base = x + t * row_stride + (long long)hd * d;
    float fa[8], fb[8], oa[8], ob[8];
    unpack8(*reinterpret_cast<const uint4*>(base + j), fa);
    unpack8(*reinterpret_cast<const uint4*>(base + j + half), fb);
    const float4 c0 = *reinterpret_cast<const float4*>(cs + (size_t)p * half + j);
    const float4 c1 = *reinterpret_cast<const float4*>(cs + (size_t)p * half + j + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sn + (size_t)p * half + j);
    const float4 s1 = *reinterpret_cast<const float4*>(sn + (size_t)p * half + j + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sg[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      // explicit roundings: the q/k/v GEMM's rotary epilogue (csrc/gemm/gemm.cu) evaluates the same expressions
      const float sk = sg[k] * sign;
      oa[k] = __fmaf_rn(fa[k], c[k], -__fmul_rn(fb[k], sk));
      ob[k] = __fmaf_rn(fb[k], c[k], __fmul_rn(fa[k], sk));
    }
    *reinterpret_cast<uint4*>(base + j) = pack8(oa);
    *reinterpret_cast<uint4*>(base + j + half) = pack8(ob);
  }
}

// x[t, j] += bias[j] in place (bf16, 16-byte vectors): the q/k/v projection bias of Qwen2-style attention
__global__ void bias_add_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias, long long T,
                                int N, long long ld) {
  const int nv = N >> 3;
  const long long total = T * nv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / nv;
    const int v = (int)(i - t * nv);
    uint4* px = reinterpret_cast<uint4*>(x + t * ld) + v;
    float a[8], b8[8];
    unpack8(*px, a);
    unpack8(reinterpret_cast<const uint4*>(bias)[v], b8);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += b8[j];
    *px = pack8(a);
  }
}

// out[j] += sum_t dy[t, j]  (fp32 atomics; the launcher zeroes `out` first when it must not accumulate).
// Block = 32 column vectors (256 columns) x 8 row lanes; grid.y row groups stride over the rows.
__global__ void __launch_bounds__(256) bias_grad_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ out,
                                                        long long T, int N, long long ld) {
  __shared__ float red[8][32][9];
  const int cv = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int v = blockIdx.x * 32 + cv;  // column vector index
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (v * 8 < N) {
    for (long long t = (long long)blockIdx.y * 8 + rl; t < T; t += (long long)gridDim.y * 8) {
      float a[8];
      unpack8(reinterpret_cast<const uint4*>(dy + t * ld)[v], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += a[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[rl][cv][j] = acc[j];
  __syncthreads();
  if (rl == 0 && v * 8 < N) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) s += red[k][cv][j];
      atomicAdd(out + v * 8 + j, s);
    }
  }
}

// act[t, j] = silu(gu[t, j]) * gu[t, f + j]      gu is [T, 2f]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, long long T,
                                  int f) {
  const int fv = f >> 3;
  const long long total = T * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int v = (int)(i - t * fv);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * f);
    float g[8], u[8], o[8];
    unpack8(row[v], g);
    unpack8(row[fv + v], u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = __fdividef(g[j], 1.f + __expf(-g[j])) * u[j];
    reinterpret_cast<uint4*>(act + t * f)[v] = pack8(o);
  }
}

// dgu[t, j] = dact * u * dsilu(g) ; dgu[t, f + j] = dact * silu(g)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int f) {
  const int fv = f >> 3;
  const long long total = T * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int v = (int)(i - t * fv);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * f);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[v], g);
    unpack8(row[fv + v], u);
    unpack8(reinterpret_cast<const uint4*>(dact + t * f)[v], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = __fdividef(1.f, 1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
      du[j] = d[j] * silu;
    }
    uint4* orow = reinterpret_cast<uint4*>(dgu + t * 2 * f);
    orow[v] = pack8(dg);
    orow[fv + v] = pack8(du);
  }
}

__global__ void embed_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ W,
                                 __nv_bfloat16* __restrict__ out, long long T, int h, int vocab) {
  const int hv = h >> 3;
  const long long total = T * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / hv;
    const int v = (int)(i - t * hv);
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    reinterpret_cast<uint4*>(out + t * h)[v] = reinterpret_cast<const uint4*>(W + id * h)[v];
  }
}

// dW[ids[t], :] += dout[t, :]   (fp32 gradient buffer, atomics: rows repeat)
__global__ void embed_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                 float* __restrict__ dW, long long T, int h, int vocab) {
  const int hv = h >> 3;
  const long long total = T * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / hv;
    const int v = (int)(i - t * hv);
    long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float d[8];
    unpack8(reinterpret_cast<const uint4*>(dout + t * h)[v], d);
    float* dst = dW + id * h + (long long)v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, d[j]);
  }
}

// dst[rows[i], :] = src[i, :]   (rows unique; dst pre-zeroed by the launcher). Backward of a row gather.
__global__ void scatter_rows_kernel(const long long* __restrict__ rows, const __nv_bfloat16* __restrict__ src,
                                    __nv_bfloat16* __restrict__ dst, long long n, int h, long long dst_rows) {
  const int hv = h >> 3;
  const long long total = n * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / hv;
    const int v = (int)(i - t * hv);
    const long long r = rows[t];
    if (r < 0 || r >= dst_rows) continue;
    reinterpret_cast<uint4*>(dst + r * h)[v] = reinterpret_cast<const uint4*>(src + t * h)[v];
  }
}

// bf16 <-> fp32 conversions over flat buffers (n elements), with optional scale / accumulate.
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n,
                                        float scale) {
  const long long nv = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(in)[2 * i];
    const float4 b = reinterpret_cast<const float4*>(in)[2 * i + 1];
    float f[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale, b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    reinterpret_cast<uint4*>(out)[i] = pack8(f);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nv << 3; i < n; ++i) out[i] = __float2bfloat16(in[i] * scale);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, long long n,
                                        float scale, int accumulate) {
  const long long nv = n >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(in)[i], f);
    float4 a = make_float4(f[0] * scale, f[1] * scale, f[2] * scale, f[3] * scale);
    float4 b = make_float4(f[4] * scale, f[5] * scale, f[6] * scale, f[7] * scale);
    if (accumulate) {
      const float4 oa = reinterpret_cast<float4*>(out)[2 * i], ob = reinterpret_cast<float4*>(out)[2 * i + 1];
      a.x += oa.x; a.y += oa.y; a.z += oa.z; a.w += oa.w;
      b.x += ob.x; b.y += ob.y; b.z += ob.z; b.w += ob.w;
    }
    reinterpret_cast<float4*>(out)[2 * i] = a;
    reinterpret_cast<float4*>(out)[2 * i + 1] = b;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = nv << 3; i < n; ++i) {
      const float v = __bfloat162float(in[i]) * scale;
      out[i] = accumulate ? out[i] + v : v;
    }
}

static inline int grid_for(long long work_items, int threads, int per_sm = 8) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = (long long)sm_count() * per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace ew
}  // namespace b200

extern "C" {
using namespace b200;
using namespace b200::ew;

// Number of fp32 partial rows rmsnorm_bwd needs in `dw_partial` ([blocks, h]).
int b200_rmsnorm_bwd_blocks(int rows) {
  const int cap = sm_count() * 16;  // enough rows in flight per SM to keep HBM busy; partial rows stay small
  return rows < cap ? rows : cap;
}

int b200_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* hout, float* rstd, int rows, int h,
                     float eps, cudaStream_t st) {
  if (!x || !w || !y || rows <= 0 || (h & 7) || h > NT * MAX_VEC * 8) return B200_ERR_ARG;
  const int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
  const int wblocks = ceil_div(rows, 4) < sm_count() * 5 ? ceil_div(rows, 4) : sm_count() * 5;  // 4 rows per 128-thread CTA
#define B200_RMS_FWD_WARP(VPL)                                                                                        \
  rmsnorm_fwd_warp_kernel<VPL><<<wblocks, 128, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res,            \
                                                        (const __nv_bfloat16*)w, (__nv_bfloat16*)y,                   \
                                                        (__nv_bfloat16*)hout, rstd, rows, eps)
  if (h == 2048) B200_RMS_FWD_WARP(8);
  else if (h == 1024) B200_RMS_FWD_WARP(4);
  else if (h == 512) B200_RMS_FWD_WARP(2);
  else if (h == 256) B200_RMS_FWD_WARP(1);
  else
    rmsnorm_fwd_kernel<<<grid, NT, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w,
                                            (__nv_bfloat16*)y, (__nv_bfloat16*)hout, rstd, rows, h, eps);
#undef B200_RMS_FWD_WARP
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// dw_out (+)= column sums; dw_partial is scratch of b200_rmsnorm_bwd_blocks(rows) * h floats.
int b200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                     float* dw_partial, float* dw_out, int dw_accumulate, int rows, int h, cudaStream_t st) {
  if (!dy || !x || !w || !rstd || !dx || !dw_partial || !dw_out || rows <= 0 || (h & 7) || h > NT * MAX_VEC * 8)
    return B200_ERR_ARG;
  const int grid = b200_rmsnorm_bwd_blocks(rows);  // partial rows: one per block, or one per warp in the warp kernels
#define B200_RMS_BWD_WARP(VPL)                                                                                       \
  rmsnorm_bwd_warp_kernel<VPL><<<ceil_div(grid, 4), 128, 4 * (VPL) * 256 * 4, st>>>(                                                   \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,   \
      (__nv_bfloat16*)dx, dw_partial, rows, grid)
  if (h == 2048) B200_RMS_BWD_WARP(8);
  else if (h == 1024) B200_RMS_BWD_WARP(4);
  else if (h == 512) B200_RMS_BWD_WARP(2);
  else if (h == 256) B200_RMS_BWD_WARP(1);
  else
    rmsnorm_bwd_kernel<<<grid, NT, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                            rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dw_partial, rows, h);
#undef B200_RMS_BWD_WARP
  B200_CUDA_CHECK(cudaGetLastError());
  const bool warp_kernel = h == 2048 || h == 1024 || h == 512 || h == 256;    // one partial row per 4-warp CTA there
  colsum_kernel<<<ceil_div(h, 32), 256, 0, st>>>(dw_partial, dw_out, warp_kernel ? ceil_div(grid, 4) : grid, h,
                                                 dw_accumulate);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// Per-head RMSNorm of the q and k heads of qkv rows [T, (H + 2 Hkv) d] with row stride ld (Qwen3 q_norm / k_norm):
// y gets the normalised q and k heads and a copy of the v heads, rstd [T, H + Hkv] the inverse norms. d = 64 or 128.
int b200_headnorm_fwd(const void* x, void* y, const void* wq, const void* wk, float* rstd, long long T, int H, int Hkv,
                      int d, long long ld, float eps, cudaStream_t st) {
  if (!x || !y || !wq || !wk || !rstd || T <= 0 || H <= 0 || Hkv <= 0 || (d != 64 && d != 128) || (ld & 7))
    return B200_ERR_ARG;
  const long long items = T * (H + 2 * Hkv);
  const int grid = grid_for(items * 32, 256);
  if (d == 128)
    headnorm_fwd_kernel<4><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (const __nv_bfloat16*)wq,
                                                 (const __nv_bfloat16*)wk, rstd, T, H, Hkv, ld, eps);
  else
    headnorm_fwd_kernel<2><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (const __nv_bfloat16*)wq,
                                                 (const __nv_bfloat16*)wk, rstd, T, H, Hkv, ld, eps);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_headnorm_bwd_blocks(long long T, int H, int Hkv) {
  const long long items = T * (H + Hkv);
  long long b = (items + 7) / 8;             // 8 warps per block
  const long long cap = (long long)sm_count() * 8;
  return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

// In place on g (the gradient of the normalised, un-rotated qkv rows); dw_partial is scratch of
// b200_headnorm_bwd_blocks(T, H, Hkv) * 2 d floats; dw_out [2 d] = [dwq | dwk] is written or accumulated.
int b200_headnorm_bwd(void* g, const void* x, const void* wq, const void* wk, const float* rstd, float* dw_partial,
                      float* dw_out, int dw_accumulate, long long T, int H, int Hkv, int d, long long ld,
                      cudaStream_t st) {
  if (!g || !x || !wq || !wk || !rstd || !dw_partial || !dw_out || T <= 0 || H <= 0 || Hkv <= 0 ||
      (d != 64 && d != 128) || (ld & 7))
    return B200_ERR_ARG;
  const int grid = b200_headnorm_bwd_blocks(T, H, Hkv);
  if (d == 128)
    headnorm_bwd_kernel<4><<<grid, 256, 0, st>>>((__nv_bfloat16*)g, (const __nv_bfloat16*)x, (const __nv_bfloat16*)wq,
                                                 (const __nv_bfloat16*)wk, rstd, dw_partial, T, H, Hkv, ld);
  else
    headnorm_bwd_kernel<2><<<grid, 256, 0, st>>>((__nv_bfloat16*)g, (const __nv_bfloat16*)x, (const __nv_bfloat16*)wq,
                                                 (const __nv_bfloat16*)wk, rstd, dw_partial, T, H, Hkv, ld);
  B200_CUDA_CHECK(cudaGetLastError());
  colsum_kernel<<<ceil_div(2 * d, 32), 256, 0, st>>>(dw_partial, dw_out, grid, 2 * d, dw_accumulate);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// rot: how many leading elements of each head rotate (a multiple of 16, at most d); the tables are [max_pos, rot/2]
int b200_rope_partial(void* x, const int* pos, const float* cos_tab, const float* sin_tab, long long T, int nh, int d,
                      int rot, long long row_stride, int inverse, cudaStream_t st) {
  if (!x || !pos || !cos_tab || !sin_tab || T <= 0 || nh <= 0 || (d & 7) || rot <= 0 || rot > d || (rot & 15) ||
      (row_stride & 7))
    return B200_ERR_ARG;
  const long long total = T * nh * (rot >> 4);
  rope_kernel<<<grid_for(total, 256), 256, 0, st>>>((__nv_bfloat16*)x, pos, cos_tab, sin_tab, T, nh, d, rot,
                                                   row_stride, inverse ? -1.f : 1.f);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_rope(void* x, const int* pos, const float* cos_tab, const float* sin_tab, long long T, int nh, int d,
              long long row_stride, int inverse, cudaStream_t st) {
  return b200_rope_partial(x, pos, cos_tab, sin_tab, T, nh, d, d, row_stride, inverse, st);
}

int b200_bias_add(void* x, const void* bias, long long T, int N, long long ld, cudaStream_t st) {
  if (!x || !bias || T <= 0 || N <= 0 || (N & 7) || (ld & 7)) return B200_ERR_ARG;
  bias_add_kernel<<<grid_for(T * (N >> 3), 256), 256, 0, st>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)bias, T, N, ld);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

// out[N] (fp32) (+)= column sums of dy[T, N] (bf16, row stride ld)
int b200_bias_grad(const void* dy, float* out, long long T, int N, long long ld, int accumulate, cudaStream_t st) {
  if (!dy || !out || T <= 0 || N <= 0 || (N & 7) || (ld & 7)) return B200_ERR_ARG;
  if (!accumulate) B200_CUDA_CHECK(cudaMemsetAsync(out, 0, sizeof(float) * N, st));
  long long gy = (T + 511) / 512;
  if (gy > 64) gy = 64;
  if (gy < 1) gy = 1;
  dim3 grid((unsigned)ceil_div(N, 256), (unsigned)gy);
  bias_grad_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy, out, T, N, ld);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_swiglu_fwd(const void* gu, void* act, long long T, int f, cudaStream_t st) {
  if (!gu || !act || T <= 0 || (f & 7)) return B200_ERR_ARG;
  swiglu_fwd_kernel<<<grid_for(T * (f >> 3), 256), 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)act, T, f);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_swiglu_bwd(const void* gu, const void* dact, void* dgu, long long T, int f, cudaStream_t st) {
  if (!gu || !dact || !dgu || T <= 0 || (f & 7)) return B200_ERR_ARG;
  swiglu_bwd_kernel<<<grid_for(T * (f >> 3), 256), 256, 0, st>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dact,
                                                                (__nv_bfloat16*)dgu, T, f);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_embed_fwd(const long long* ids, const void* W, void* out, long long T, int h, int vocab, cudaStream_t st) {
  if (!ids || !W || !out || T <= 0 || (h & 7)) return B200_ERR_ARG;
  embed_fwd_kernel<<<grid_for(T * (h >> 3), 256), 256, 0, st>>>(ids, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, T, h,
                                                               vocab);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_embed_bwd(const long long* ids, const void* dout, float* dW, long long T, int h, int vocab, cudaStream_t st) {
  if (!ids || !dout || !dW || T <= 0 || (h & 7)) return B200_ERR_ARG;
  embed_bwd_kernel<<<grid_for(T * (h >> 3), 256), 256, 0, st>>>(ids, (const __nv_bfloat16*)dout, dW, T, h, vocab);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_scatter_rows(const long long* rows, const void* src, void* dst, long long n, int h, long long dst_rows,
                      cudaStream_t st) {
  if (!rows || !src || !dst || n <= 0 || (h & 7) || dst_rows <= 0) return B200_ERR_ARG;
  B200_CUDA_CHECK(cudaMemsetAsync(dst, 0, (size_t)dst_rows * h * 2, st));
  scatter_rows_kernel<<<grid_for(n * (h >> 3), 256), 256, 0, st>>>(rows, (const __nv_bfloat16*)src, (__nv_bfloat16*)dst,
                                                                  n, h, dst_rows);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_cast_f32_to_bf16(const float* in, void* out, long long n, float scale, cudaStream_t st) {
  if (!in || !out || n <= 0) return B200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return B200_ERR_ARG;
  cast_f32_to_bf16_kernel<<<grid_for(n >> 3, 256), 256, 0, st>>>(in, (__nv_bfloat16*)out, n, scale);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_cast_bf16_to_f32(const void* in, float* out, long long n, float scale, int accumulate, cudaStream_t st) {
  if (!in || !out || n <= 0) return B200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return B200_ERR_ARG;
  cast_bf16_to_f32_kernel<<<grid_for(n >> 3, 256), 256, 0, st>>>((const __nv_bfloat16*)in, out, n, scale, accumulate);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
}

// ------------------------------------------------------------------------------------------------------------
// Allocation-free RMSNorm backward (declared and documented in rmsnorm_noalloc.h).
#include "rmsnorm_noalloc.h"

#include <mutex>

namespace b200 {
namespace ew {

// Workspace for the per-block weight-gradient partial sums. In host code this name is only a handle for the
// runtime: the kernels get the device address obtained once per device by scratch_for_current_device().
static __device__ __align__(256) float g_rmsnorm_noalloc_scratch[B200_RMSNORM_NOALLOC_MAX_BLOCKS * B200_RMSNORM_NOALLOC_MAX_H];

static float* g_noalloc_ptr[64] = {nullptr};
static std::mutex g_noalloc_mu;

// Device address of the workspace on the current device (looked up on the first call per device).
static int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_last_cuda_error(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) {
    set_last_cuda_error(cudaErrorInvalidDevice, "b200_rmsnorm_bwd_noalloc: device index outside the 64 this library tracks");
    return B200_ERR_ARG;
  }
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_noalloc_scratch);
    if (e != cudaSuccess) return set_last_cuda_error(e, "cudaGetSymbolAddress(g_rmsnorm_noalloc_scratch)");
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return B200_OK;
}

}  // namespace ew
}  // namespace b200

extern "C" int b200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                        const void* dres, void* dx, float* dw_out, int dw_accumulate, int rows, int h,
                                        cudaStream_t st) {
  using namespace b200;
  using namespace b200::ew;
  if (!dy || !x || !w || !rstd || !dx || !dw_out || rows <= 0 || h <= 0 || (h & 7)) return B200_ERR_ARG;
  if (h > B200_RMSNORM_NOALLOC_MAX_H) {
    set_last_cuda_error(cudaErrorInvalidValue,
                        "b200_rmsnorm_bwd_noalloc: h exceeds B200_RMSNORM_NOALLOC_MAX_H (4096); use b200_rmsnorm_bwd "
                        "with a caller-provided workspace");
    return B200_ERR_TOO_BIG;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != B200_OK) return rc;
  const int grid = rows < B200_RMSNORM_NOALLOC_MAX_BLOCKS ? rows : B200_RMSNORM_NOALLOC_MAX_BLOCKS;
  // every block writes its own partial row (all h columns) before the column sum reads rows [0, grid):
  // nothing left over from an earlier call is ever read
  rmsnorm_bwd_kernel<<<grid, NT, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                          rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, scratch, rows, h);
  B200_CUDA_CHECK(cudaGetLastError());
  colsum_kernel<<<ceil_div(h, 32), 256, 0, st>>>(scratch, dw_out, grid, h, dw_accumulate);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
