// Fused optimizer steps over flat parameter shards (one launch per step, fp32 master weights and
// state, bf16 model weights written in the same pass): AdamW / Adam, SGD with momentum (+ Nesterov),
// centred RMSprop, Adagrad, and a block-wise 8-bit-state AdamW. The gradient is read as fp32 and
// may be pre-scaled (1 / (grad_accum * world)) in the same pass.
#include "../common/ptx.cuh"
#include "../common/host.cuh"

namespace b200 {
namespace optim {

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale;
  int decoupled;  // 1: AdamW, 0: Adam with L2 added to the gradient
};

__global__ void __launch_bounds__(256) adam_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ model,
                                                  const float* __restrict__ grad, float* __restrict__ m,
                                                  float* __restrict__ v, long long n, AdamArgs a) {
  const long long nv = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(master)[i];
    float4 g = reinterpret_cast<const float4*>(grad)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* pp = &p.x; float* gp = &g.x; float* mp = &mm.x; float* vp = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = gp[j] * a.grad_scale;
      if (a.decoupled) pp[j] *= (1.f - a.lr * a.weight_decay);
      else gj += a.weight_decay * pp[j];
      mp[j] = a.beta1 * mp[j] + (1.f - a.beta1) * gj;
      vp[j] = a.beta2 * vp[j] + (1.f - a.beta2) * gj * gj;
      const float denom = sqrtf(vp[j] / a.bias2) + a.eps;
      pp[j] -= (a.lr / a.bias1) * mp[j] / denom;
    }
    reinterpret_cast<float4*>(master)[i] = p;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (model) {
      uint2 o;
      o.x = pack_bf16x2(p.x, p.y);
      o.y = pack_bf16x2(p.z, p.w);
      reinterpret_cast<uint2*>(model)[i] = o;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long i = nv << 2; i < n; ++i) {
      float gj = grad[i] * a.grad_scale, pj = master[i];
      if (a.decoupled) pj *= (1.f - a.lr * a.weight_decay);
      else gj += a.weight_decay * pj;
      m[i] = a.beta1 * m[i] + (1.f - a.beta1) * gj;
      v[i] = a.beta2 * v[i] + (1.f - a.beta2) * gj * gj;
      pj -= (a.lr / a.bias1) * m[i] / (sqrtf(v[i] / a.bias2) + a.eps);
      master[i] = pj;
      if (model) model[i] = __float2bfloat16(pj);
    }
  }
}

// kind: 0 SGD(momentum, nesterov) ; 1 RMSprop centred (alpha, eps) ; 2 Adagrad (eps)
struct SimpleArgs {
  float lr, weight_decay, momentum, alpha, eps, grad_scale;
  int kind, nesterov, first_step;
};

__global__ void __launch_bounds__(256) simple_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ model,
                                                    const float* __restrict__ grad, float* __restrict__ s0,
                                                    float* __restrict__ s1, long long n, SimpleArgs a) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float p = master[i];
    float g = grad[i] * a.grad_scale + a.weight_decay * p;
    if (a.kind == 0) {
      float buf = a.first_step ? g : a.momentum * s0[i] + g;
      s0[i] = buf;
      const float upd = a.momentum == 0.f ? g : (a.nesterov ? g + a.momentum * buf : buf);
      p -= a.lr * upd;
    } else if (a.kind == 1) {
      const float sq = a.alpha * s0[i] + (1.f - a.alpha) * g * g;
      const float ga = a.alpha * s1[i] + (1.f - a.alpha) * g;
      s0[i] = sq;
      s1[i] = ga;
      p -= a.lr * g / (sqrtf(fmaxf(sq - ga * ga, 0.f)) + a.eps);
    } else {
      const float acc = s0[i] + g * g;
      s0[i] = acc;
      p -= a.lr * g / (sqrtf(acc) + a.eps);
    }
    master[i] = p;
    if (model) model[i] = __float2bfloat16(p);
  }
}

// Block-wise 8-bit AdamW state: each block of 256 values shares one fp32 absmax per moment; m is stored as a
// signed 8-bit linear code, v as an unsigned 8-bit code of sqrt(v) (keeps small second moments resolvable).
constexpr int QB = 256;
__global__ void __launch_bounds__(QB) adam8_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ model,
                                                  const float* __restrict__ grad, int8_t* __restrict__ mq,
                                                  uint8_t* __restrict__ vq, float* __restrict__ mabs,
                                                  float* __restrict__ vabs, long long n, AdamArgs a) {
  __shared__ float red[QB / 32];
  __shared__ float bcast[2];
  for (long long blk = blockIdx.x; blk * QB < n; blk += gridDim.x) {
    const long long i = blk * QB + threadIdx.x;
    const bool ok = i < n;
    float p = 0.f, g = 0.f, mm = 0.f, vv = 0.f;
    if (ok) {
      p = master[i];
      g = grad[i] * a.grad_scale;
      mm = (float)mq[i] * (mabs[blk] / 127.f);
      const float sv = (float)vq[i] * (vabs[blk] / 255.f);
      vv = sv * sv;
      if (a.decoupled) p *= (1.f - a.lr * a.weight_decay);
      else g += a.weight_decay * p;
      mm = a.beta1 * mm + (1.f - a.beta1) * g;
      vv = a.beta2 * vv + (1.f - a.beta2) * g * g;
      p -= (a.lr / a.bias1) * mm / (sqrtf(vv / a.bias2) + a.eps);
      master[i] = p;
      if (model) model[i] = __float2bfloat16(p);
    }
    // new per-block scales
    float am = warp_max(fabsf(mm)), av = warp_max(sqrtf(vv));
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) red[w] = am;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < QB / 32; ++k) t = fmaxf(t, red[k]);
      bcast[0] = t;
    }
    __syncthreads();
    if (l == 0) red[w] = av;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int k = 0; k < QB / 32; ++k) t = fmaxf(t, red[k]);
      bcast[1] = t;
      mabs[blk] = bcast[0];
      vabs[blk] = t;
    }
    __syncthreads();
    if (ok) {
      const float sm = bcast[0] > 0.f ? 127.f / bcast[0] : 0.f;
      const float sv = bcast[1] > 0.f ? 255.f / bcast[1] : 0.f;
      mq[i] = (int8_t)__float2int_rn(mm * sm);
      vq[i] = (uint8_t)min(255, __float2int_ru(sqrtf(vv) * sv));
    }
  }
}

// sum of squares of a flat fp32 buffer (for gradient-norm logging), atomically added into out[0].
__global__ void sumsq_kernel(const float* __restrict__ x, long long n, float scale, float* __restrict__ out) {
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = x[i] * scale;
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) atomicAdd(out, s);
}

}  // namespace optim
}  // namespace b200

extern "C" {
using namespace b200;
using namespace b200::optim;

static int opt_grid(long long n, int per_thread) {
  long long b = (n / per_thread + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

// step is 1-based. model may be null (no bf16 copy). All buffers hold n elements and are 16-byte aligned.
int b200_adam_step(float* master, void* model, const float* grad, float* m, float* v, long long n, float lr,
                   float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale, int decoupled,
                   cudaStream_t st) {
  if (!master || !grad || !m || !v || n <= 0 || step < 1) return B200_ERR_ARG;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
             grad_scale, decoupled};
  adam_kernel<<<opt_grid(n, 4), 256, 0, st>>>(master, (__nv_bfloat16*)model, grad, m, v, n, a);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_adam8_step(float* master, void* model, const float* grad, void* mq, void* vq, float* mabs, float* vabs,
                    long long n, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                    float grad_scale, int decoupled, cudaStream_t st) {
  if (!master || !grad || !mq || !vq || !mabs || !vabs || n <= 0 || step < 1) return B200_ERR_ARG;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step),
             grad_scale, decoupled};
  long long blocks = (n + QB - 1) / QB;
  const long long cap = (long long)sm_count() * 8;
  adam8_kernel<<<(int)(blocks < cap ? blocks : cap), QB, 0, st>>>(master, (__nv_bfloat16*)model, grad, (int8_t*)mq,
                                                                  (uint8_t*)vq, mabs, vabs, n, a);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_simple_opt_step(float* master, void* model, const float* grad, float* s0, float* s1, long long n, int kind,
                         float lr, float weight_decay, float momentum, float alpha, float eps, int nesterov,
                         int first_step, float grad_scale, cudaStream_t st) {
  if (!master || !grad || !s0 || n <= 0 || kind < 0 || kind > 2 || (kind == 1 && !s1)) return B200_ERR_ARG;
  SimpleArgs a{lr, weight_decay, momentum, alpha, eps, grad_scale, kind, nesterov, first_step};
  simple_kernel<<<opt_grid(n, 1), 256, 0, st>>>(master, (__nv_bfloat16*)model, grad, s0, s1, n, a);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}

int b200_sumsq(const float* x, long long n, float scale, float* out, cudaStream_t st) {
  if (!x || !out || n <= 0) return B200_ERR_ARG;
  sumsq_kernel<<<opt_grid(n, 4), 256, 0, st>>>(x, n, scale, out);
  B200_CUDA_CHECK(cudaGetLastError());
  return B200_OK;
}
}
