// ChannelNorm: LayerNorm over the channel axis of a [B, C, T] tensor without transposing it (fp32 and bf16 storage, fp32
// math), with an optional fused ReLU.  Contract: ChannelNorm / ChannelNormBwd / ChannelNormRelu / ChannelNormReluBwd of the
// reference (Source/Public/Oa/Ml/FnMatrix.h:544-568).  Threads run along T, so every load of a channel row is coalesced;
// the statistics pass and the output pass read x twice (the second read is served by L2 for the sizes of a 1-D conv stack).
// Parameter gradients are reduced by one CTA per channel in a fixed order: results are reproducible.
#include "common.cuh"
#include "api.h"

namespace oa {

template <typename T> __device__ __forceinline__ float cn_load(const T* p, long long i);
template <> __device__ __forceinline__ float cn_load<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float cn_load<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T> __device__ __forceinline__ void cn_store(T* p, long long i, float v);
template <> __device__ __forceinline__ void cn_store<float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void cn_store<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

template <typename T>
__global__ void channel_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y,
                                        float* __restrict__ mean_out, float* __restrict__ rstd_out, int B, int C, int L, float eps, int relu) {
  const long long total = (long long)B * L;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / L, t = i - b * L;
    const long long base = b * C * L + t;
    float s = 0.f, ss = 0.f;
    for (int c = 0; c < C; ++c) {
      const float v = cn_load(x, base + (long long)c * L);
      s += v;
      ss = fmaf(v, v, ss);
    }
    const float mean = s / (float)C;
    const float rstd = rsqrtf(fmaxf(ss / (float)C - mean * mean, 0.f) + eps);
    mean_out[i] = mean;
    rstd_out[i] = rstd;
    for (int c = 0; c < C; ++c) {
      float v = (cn_load(x, base + (long long)c * L) - mean) * rstd * cn_load(w, c) + (bias ? cn_load(bias, c) : 0.f);
      if (relu) v = fmaxf(v, 0.f);
      cn_store(y, base + (long long)c * L, v);
    }
  }
}

// dx = rstd * (gw - mean_c(gw) - xhat * mean_c(gw * xhat)), gw = g * w (g masked by y > 0 for the ReLU form)
template <typename T>
__global__ void channel_norm_bwd_dx_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ g, const T* __restrict__ y_relu,
                                           const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx, int B, int C,
                                           int L) {
  const long long total = (long long)B * L;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / L, t = i - b * L;
    const long long base = b * C * L + t;
    const float mean = mean_in[i], rstd = rstd_in[i];
    float s1 = 0.f, s2 = 0.f;
    for (int c = 0; c < C; ++c) {
      const long long k = base + (long long)c * L;
      float gv = cn_load(g, k);
      if (y_relu && !(cn_load(y_relu, k) > 0.f)) gv = 0.f;
      const float gw = gv * cn_load(w, c);
      s1 += gw;
      s2 = fmaf(gw, (cn_load(x, k) - mean) * rstd, s2);
    }
    s1 /= (float)C;
    s2 /= (float)C;
    for (int c = 0; c < C; ++c) {
      const long long k = base + (long long)c * L;
      float gv = cn_load(g, k);
      if (y_relu && !(cn_load(y_relu, k) > 0.f)) gv = 0.f;
      const float xhat = (cn_load(x, k) - mean) * rstd;
      cn_store(dx, k, rstd * (gv * cn_load(w, c) - s1 - xhat * s2));
    }
  }
}

// one CTA per channel: dw[c] = sum_{b,t} g * xhat, db[c] = sum g (fixed-order tree)
template <typename T>
__global__ void __launch_bounds__(256) channel_norm_bwd_param_kernel(const T* __restrict__ x, const T* __restrict__ g, const T* __restrict__ y_relu,
                                                                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                                                     float* __restrict__ dw, float* __restrict__ db, int B, int C, int L) {
  __shared__ float sw[256], sb[256];
  const int c = blockIdx.x;
  float aw = 0.f, ab = 0.f;
  const long long total = (long long)B * L;
  for (long long i = threadIdx.x; i < total; i += 256) {
    const long long b = i / L, t = i - b * L;
    const long long k = (b * C + c) * L + t;
    float gv = cn_load(g, k);
    if (y_relu && !(cn_load(y_relu, k) > 0.f)) gv = 0.f;
    aw = fmaf(gv, (cn_load(x, k) - mean_in[i]) * rstd_in[i], aw);
    ab += gv;
  }
  sw[threadIdx.x] = aw;
  sb[threadIdx.x] = ab;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) { sw[threadIdx.x] += sw[threadIdx.x + o]; sb[threadIdx.x] += sb[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { dw[c] = sw[0]; db[c] = sb[0]; }
}

static inline int cn_grid(long long n) {
  long long g = (n + 127) / 128;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace oa

using namespace oa;

extern "C" {

int oa_channel_norm_fwd(int dtype, const void* x, const void* w, const void* bias, void* y, void* mean, void* rstd, int B, int C, int L, float eps,
                        int relu, void* stream) {
  if (B <= 0 || C <= 0 || L <= 0) return OA_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == OA_F32)
    channel_norm_fwd_kernel<float><<<cn_grid((long long)B * L), 128, 0, st>>>((const float*)x, (const float*)w, (const float*)bias, (float*)y,
                                                                               (float*)mean, (float*)rstd, B, C, L, eps, relu);
  else if (dtype == OA_BF16)
    channel_norm_fwd_kernel<__nv_bfloat16><<<cn_grid((long long)B * L), 128, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                                                       (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, (float*)mean,
                                                                                       (float*)rstd, B, C, L, eps, relu);
  else return OA_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

int oa_channel_norm_bwd(int dtype, const void* x, const void* w, const void* g, const void* y_relu, const void* mean, const void* rstd, void* dx,
                        void* dw_f32, void* db_f32, int B, int C, int L, void* stream) {
  if (B <= 0 || C <= 0 || L <= 0) return OA_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == OA_F32) {
    channel_norm_bwd_dx_kernel<float><<<cn_grid((long long)B * L), 128, 0, st>>>((const float*)x, (const float*)w, (const float*)g,
                                                                                  (const float*)y_relu, (const float*)mean, (const float*)rstd,
                                                                                  (float*)dx, B, C, L);
    channel_norm_bwd_param_kernel<float><<<C, 256, 0, st>>>((const float*)x, (const float*)g, (const float*)y_relu, (const float*)mean,
                                                             (const float*)rstd, (float*)dw_f32, (float*)db_f32, B, C, L);
  } else if (dtype == OA_BF16) {
    channel_norm_bwd_dx_kernel<__nv_bfloat16><<<cn_grid((long long)B * L), 128, 0, st>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)g, (const __nv_bfloat16*)y_relu, (const float*)mean,
        (const float*)rstd, (__nv_bfloat16*)dx, B, C, L);
    channel_norm_bwd_param_kernel<__nv_bfloat16><<<C, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)g, (const __nv_bfloat16*)y_relu,
                                                                     (const float*)mean, (const float*)rstd, (float*)dw_f32, (float*)db_f32, B, C, L);
  } else return OA_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

}  // extern "C"
