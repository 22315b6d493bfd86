// Fused optimizer kernels over flat parameter arenas: Adam / AdamW / SGD with optional fp32 master
// weights for bf16 parameters, gradient-norm clipping, and a device-resident hyper-parameter block so
// that a captured CUDA graph of a training step can be replayed (the step counter advances on the
// device, the host may rewrite the learning rate between replays).
// Math contracts: Source/Private/Oa/Ml/Shader/Compute/Optim/Adam/Adam.slang:28-43,
// Optim/AdamW/Adamw.slang:35-53 (decay first, then the Adam update), Optim/Sgd/SgdMomentum.slang:28-40
// (weight decay is NOT multiplied by the learning rate), Optim/GradClip/*.slang.
// Difference from the reference: the bf16 write-back rounds to nearest even instead of truncating.
#include "common.cuh"
#include "api.h"

namespace oa {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void stf(T* p, long long i, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__global__ void optim_advance_kernel(float* state) {
  if (threadIdx.x == 0 && blockIdx.x == 0) state[0] += 1.f;
}

// One Adam step on element i given fp32 weight w and gradient g; returns the new weight.
struct AdamHyper {
  float lr, b1, b2, eps, wd, bc1, bc2;
  int decoupled;
};
__device__ __forceinline__ AdamHyper load_hyper(const float* state, int decoupled) {
  AdamHyper h;
  float step = state[0];
  h.lr = state[1]; h.b1 = state[2]; h.b2 = state[3]; h.eps = state[4]; h.wd = state[5];
  h.bc1 = 1.f - powf(h.b1, step);
  h.bc2 = 1.f - powf(h.b2, step);
  h.decoupled = decoupled;
  return h;
}
__device__ __forceinline__ float adam_update(const AdamHyper& h, float w, float g, float& m, float& v) {
  if (h.decoupled) w -= h.lr * h.wd * w;
  else g += h.wd * w;
  m = h.b1 * m + (1.f - h.b1) * g;
  v = h.b2 * v + (1.f - h.b2) * g * g;
  float mh = m / h.bc1, vh = v / h.bc2;
  return w - h.lr * mh / (sqrtf(vh) + h.eps);
}

template <typename P, typename G>
__global__ void adam_kernel(P* __restrict__ param, const G* __restrict__ grad, float* __restrict__ master,
                            float* __restrict__ m, float* __restrict__ v, long long n, const float* __restrict__ state,
                            int decoupled, const float* __restrict__ inv_clip) {
  const AdamHyper h = load_hyper(state, decoupled);
  const float gs = state[6] * (inv_clip ? inv_clip[0] : 1.f);
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = ldf<G>(grad, i) * gs;
    float w = master ? master[i] : ldf<P>(param, i);
    float mi = m[i], vi = v[i];
    w = adam_update(h, w, g, mi, vi);
    m[i] = mi; v[i] = vi;
    if (master) master[i] = w;
    stf<P>(param, i, w);
  }
}

// bf16 parameter / bf16 gradient / fp32 master fast path: four elements per thread per trip (8-byte bf16 and 16-byte fp32
// accesses), two trips in flight.  Requires 16-byte aligned arenas (the optimizer's flat arenas are) and n % 4 == 0.
__global__ void __launch_bounds__(256)
adam_bf16_vec4_kernel(__nv_bfloat16* __restrict__ param, const __nv_bfloat16* __restrict__ grad, float* __restrict__ master,
                      float* __restrict__ m, float* __restrict__ v, long long n4, const float* __restrict__ state, int decoupled,
                      const float* __restrict__ inv_clip) {
  const AdamHyper h = load_hyper(state, decoupled);
  const float gs = state[6] * (inv_clip ? inv_clip[0] : 1.f);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += 2 * stride) {
    const long long idx[2] = {i, i + stride};
    uint2 g2[2];
    float4 w4[2], m4[2], v4[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] < n4) {
        g2[u] = reinterpret_cast<const uint2*>(grad)[idx[u]];
        w4[u] = reinterpret_cast<const float4*>(master)[idx[u]];
        m4[u] = reinterpret_cast<const float4*>(m)[idx[u]];
        v4[u] = reinterpret_cast<const float4*>(v)[idx[u]];
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] >= n4) continue;
      const float2 ga = unpack_bf16x2(g2[u].x), gb = unpack_bf16x2(g2[u].y);
      float w[4] = {w4[u].x, w4[u].y, w4[u].z, w4[u].w}, mm[4] = {m4[u].x, m4[u].y, m4[u].z, m4[u].w}, vv[4] = {v4[u].x, v4[u].y, v4[u].z, v4[u].w};
      const float g[4] = {ga.x * gs, ga.y * gs, gb.x * gs, gb.y * gs};
#pragma unroll
      for (int k = 0; k < 4; ++k) w[k] = adam_update(h, w[k], g[k], mm[k], vv[k]);
      reinterpret_cast<float4*>(master)[idx[u]] = make_float4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<float4*>(m)[idx[u]] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      reinterpret_cast<float4*>(v)[idx[u]] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      reinterpret_cast<uint2*>(param)[idx[u]] = make_uint2(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]));
    }
  }
}

template <typename P, typename G>
__global__ void sgd_kernel(P* __restrict__ param, const G* __restrict__ grad, float* __restrict__ master,
                           float* __restrict__ mom, long long n, float lr, float mu, float wd) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = ldf<G>(grad, i);
    float w = master ? master[i] : ldf<P>(param, i);
    float upd = g;
    if (mom) { float mm = mu * mom[i] + g; mom[i] = mm; upd = mm; }
    w -= lr * upd + wd * w;
    if (master) master[i] = w;
    stf<P>(param, i, w);
  }
}

template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = ldf<T>(x, i);
    s += v * v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int nparts, float* out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    out[0] = accumulate ? out[0] + t : t;
  }
}
__global__ void clip_coef_kernel(const float* sumsq, float max_norm, float* coef) {
  float nrm = sqrtf(sumsq[0]);
  coef[0] = nrm > max_norm ? max_norm / (nrm + 1e-6f) : 1.f;
}
template <typename T>
__global__ void scale_inplace_kernel(T* x, long long n, const float* coef) {
  float c = coef[0];
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) stf<T>(x, i, ldf<T>(x, i) * c);
}

static inline int ogrid(long long n) {
  long long b = (n + 255) / 256;
  if (b > 148 * 8) b = 148 * 8;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace oa

using namespace oa;
#define ST ((cudaStream_t)stream)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH)

extern "C" int oa_optim_advance(float* state, void* stream) {
  optim_advance_kernel<<<1, 32, 0, ST>>>(state);
  return CHECK_LAUNCH();
}

extern "C" int oa_adamw(int pd, int gd, void* param, const void* grad, float* master, float* m, float* v, long long n,
                        const float* state, int decoupled, const float* inv_clip, void* stream) {
  if (n <= 0) return OA_OK;
  int g = ogrid(n);
  const uintptr_t al = reinterpret_cast<uintptr_t>(param) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(master) |
                       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v);
  if (pd == OA_BF16 && gd == OA_BF16 && master && (n & 3) == 0 && (al & 15) == 0) {
    adam_bf16_vec4_kernel<<<ogrid(n / 4), 256, 0, ST>>>((__nv_bfloat16*)param, (const __nv_bfloat16*)grad, master, m, v, n / 4, state, decoupled, inv_clip);
    return CHECK_LAUNCH();
  }
  if (pd == OA_BF16 && gd == OA_BF16)
    adam_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, ST>>>((__nv_bfloat16*)param, (const __nv_bfloat16*)grad, master, m, v, n, state, decoupled, inv_clip);
  else if (pd == OA_BF16 && gd == OA_F32)
    adam_kernel<__nv_bfloat16, float><<<g, 256, 0, ST>>>((__nv_bfloat16*)param, (const float*)grad, master, m, v, n, state, decoupled, inv_clip);
  else if (pd == OA_F32 && gd == OA_F32)
    adam_kernel<float, float><<<g, 256, 0, ST>>>((float*)param, (const float*)grad, master, m, v, n, state, decoupled, inv_clip);
  else if (pd == OA_F32 && gd == OA_BF16)
    adam_kernel<float, __nv_bfloat16><<<g, 256, 0, ST>>>((float*)param, (const __nv_bfloat16*)grad, master, m, v, n, state, decoupled, inv_clip);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}

extern "C" int oa_sgd(int pd, int gd, void* param, const void* grad, float* master, float* mom, long long n, float lr,
                      float momentum, float weight_decay, void* stream) {
  if (n <= 0) return OA_OK;
  int g = ogrid(n);
  if (pd == OA_BF16 && gd == OA_BF16)
    sgd_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, ST>>>((__nv_bfloat16*)param, (const __nv_bfloat16*)grad, master, mom, n, lr, momentum, weight_decay);
  else if (pd == OA_BF16 && gd == OA_F32)
    sgd_kernel<__nv_bfloat16, float><<<g, 256, 0, ST>>>((__nv_bfloat16*)param, (const float*)grad, master, mom, n, lr, momentum, weight_decay);
  else if (pd == OA_F32 && gd == OA_F32)
    sgd_kernel<float, float><<<g, 256, 0, ST>>>((float*)param, (const float*)grad, master, mom, n, lr, momentum, weight_decay);
  else if (pd == OA_F32 && gd == OA_BF16)
    sgd_kernel<float, __nv_bfloat16><<<g, 256, 0, ST>>>((float*)param, (const __nv_bfloat16*)grad, master, mom, n, lr, momentum, weight_decay);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}

// partial: float[1184] scratch.
extern "C" int oa_sumsq(int dtype, const void* x, long long n, float* partial, float* out, int accumulate, void* stream) {
  int g = ogrid(n);
  if (dtype == OA_F32) sumsq_partial_kernel<float><<<g, 256, 0, ST>>>((const float*)x, n, partial);
  else if (dtype == OA_BF16) sumsq_partial_kernel<__nv_bfloat16><<<g, 256, 0, ST>>>((const __nv_bfloat16*)x, n, partial);
  else return OA_ERR_UNSUPPORTED;
  sumsq_final_kernel<<<1, 256, 0, ST>>>(partial, g, out, accumulate);
  return CHECK_LAUNCH();
}
extern "C" int oa_clip_coef(const float* sumsq, float max_norm, float* coef, void* stream) {
  clip_coef_kernel<<<1, 1, 0, ST>>>(sumsq, max_norm, coef);
  return CHECK_LAUNCH();
}
extern "C" int oa_scale_inplace(int dtype, void* x, long long n, const float* coef, void* stream) {
  if (n <= 0) return OA_OK;
  if (dtype == OA_F32) scale_inplace_kernel<float><<<ogrid(n), 256, 0, ST>>>((float*)x, n, coef);
  else if (dtype == OA_BF16) scale_inplace_kernel<__nv_bfloat16><<<ogrid(n), 256, 0, ST>>>((__nv_bfloat16*)x, n, coef);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}
