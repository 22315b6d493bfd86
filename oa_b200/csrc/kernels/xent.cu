// Fused softmax cross-entropy: per-row fp32 loss (lse - logit[target]) and, in the same kernel,
// the logits gradient (softmax - onehot) * grad_scale, optionally written over the logits.
// An out-of-range target gives a NaN row loss instead of an out-of-bounds read, and a target
// equal to `ignore_index` gives loss 0 and a zero gradient row (masked cross-entropy).
// Reference semantics: Source/Private/Oa/Ml/Shader/Compute/Nn/CrossEntropy/CrossEntropy.slang:58-75,
// CrossEntropyBwd.slang:69-78 and the fused CrossEntropyLossGradBwd registry entry.
#include "common.cuh"
#include "api.h"

namespace oa {

template <typename T> struct XIO;
template <> struct XIO<float> {
  static constexpr int VEC = 4;
  __device__ static void load(const float* p, float* v) {
    float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  __device__ static void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
  __device__ static float ld1(const float* p) { return *p; }
};
template <> struct XIO<__nv_bfloat16> {
  static constexpr int VEC = 8;
  __device__ static void load(const __nv_bfloat16* p, float* v) {
    uint4 x = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(x.x), b = unpack_bf16x2(x.y), c = unpack_bf16x2(x.z), d = unpack_bf16x2(x.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  __device__ static void store(__nv_bfloat16* p, const float* v) {
    *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                              pack_bf16x2(v[6], v[7]));
  }
  __device__ static float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
};

constexpr int XENT_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(XENT_THREADS)
xent_kernel(const T* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ row_loss, T* dlogits,
            int vocab, int ld, float grad_scale, int ignore_index, int vec_ok) {
  constexpr int V = XIO<T>::VEC;
  __shared__ float red_m[XENT_THREADS / 32], red_s[XENT_THREADS / 32];
  const long long row = blockIdx.x;
  const T* p = logits + row * ld;
  const int tgt = targets[row];
  const int nvec = vec_ok ? vocab / V : 0;        // rows that do not start on a 16-byte boundary take the scalar loops
  const bool ignored = (tgt == ignore_index);
  const bool oor = !ignored && (tgt < 0 || tgt >= vocab);
  // read before any thread can overwrite the logits with the gradient (dlogits may alias logits)
  const float tgt_logit = (threadIdx.x == 0 && !ignored && !oor) ? XIO<T>::ld1(p + tgt) : 0.f;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += XENT_THREADS) {
    float v[V];
    XIO<T>::load(p + i * V, v);
    float mx = v[0];
#pragma unroll
    for (int j = 1; j < V; ++j) mx = fmaxf(mx, v[j]);
    if (mx > m) { s *= __expf(m - mx); m = mx; }
#pragma unroll
    for (int j = 0; j < V; ++j) s += __expf(v[j] - m);
  }
  for (int c = nvec * V + threadIdx.x; c < vocab; c += XENT_THREADS) {
    float v = XIO<T>::ld1(p + c);
    if (v > m) { s *= __expf(m - v); m = v; }
    s += __expf(v - m);
  }
  // block combine of (m, s)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) { red_m[threadIdx.x >> 5] = m; red_s[threadIdx.x >> 5] = s; }
  __syncthreads();
  m = red_m[0]; s = red_s[0];
#pragma unroll
  for (int w = 1; w < XENT_THREADS / 32; ++w) {
    float om = red_m[w], os = red_s[w];
    float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  const float lse = m + logf(s);
  if (threadIdx.x == 0) {
    float l = ignored ? 0.f : (oor ? __int_as_float(0x7fc00000) : lse - tgt_logit);
    row_loss[row] = l;
  }
  if (!dlogits) return;
  T* d = dlogits + row * ld;
  const float gs = ignored ? 0.f : grad_scale;
  for (int i = threadIdx.x; i < nvec; i += XENT_THREADS) {
    float v[V];
    XIO<T>::load(p + i * V, v);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float pr = __expf(v[j] - lse);
      v[j] = (pr - ((i * V + j) == tgt ? 1.f : 0.f)) * gs;
    }
    XIO<T>::store(d + i * V, v);
  }
  for (int c = nvec * V + threadIdx.x; c < vocab; c += XENT_THREADS) {
    float pr = __expf(XIO<T>::ld1(p + c) - lse);
    float g = (pr - (c == tgt ? 1.f : 0.f)) * gs;
    if constexpr (sizeof(T) == 4) d[c] = g; else d[c] = __float2bfloat16_rn(g);
  }
}

// out[0] = scale * sum(x), one CTA, fixed reduction order.
__global__ void mean_f32_kernel(const float* __restrict__ x, float* __restrict__ out, long long n, float scale) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    out[0] = t * scale;
  }
}

}  // namespace oa

using namespace oa;

extern "C" int oa_xent_fwd_bwd(int dtype, const void* logits, const int* targets, float* row_loss, void* dlogits,
                               long long rows, int vocab, int ld, float grad_scale, int ignore_index, void* stream) {
  if (rows <= 0) return OA_OK;
  const int es = dtype == OA_F32 ? 4 : 2;
  const int vec_ok = ((long long)ld * es) % 16 == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0 &&
                     (!dlogits || (reinterpret_cast<uintptr_t>(dlogits) & 15) == 0);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == OA_F32)
    xent_kernel<float><<<(unsigned)rows, XENT_THREADS, 0, st>>>((const float*)logits, targets, row_loss, (float*)dlogits, vocab, ld, grad_scale, ignore_index, vec_ok);
  else if (dtype == OA_BF16)
    xent_kernel<__nv_bfloat16><<<(unsigned)rows, XENT_THREADS, 0, st>>>((const __nv_bfloat16*)logits, targets, row_loss, (__nv_bfloat16*)dlogits, vocab, ld, grad_scale, ignore_index, vec_ok);
  else return OA_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

// ---- vocabulary-parallel cross-entropy (tensor parallel head): every rank holds [rows, vocab / W] logits.
// stats: (max, sum exp(l - max), target logit if the target falls into this shard else 0) per row;
// finish: global lse from all ranks' stats, row loss, and dlogits = (exp(l - lse) - onehot) * scale written in place.
namespace oa {

template <typename T>
__global__ void __launch_bounds__(XENT_THREADS)
vp_xent_stats_kernel(const T* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ stats, int vocab, int v0) {
  constexpr int V = XIO<T>::VEC;
  __shared__ float red_m[XENT_THREADS / 32], red_s[XENT_THREADS / 32];
  const long long row = blockIdx.x;
  const T* p = logits + row * vocab;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < vocab / V; i += XENT_THREADS) {
    float v[V];
    XIO<T>::load(p + i * V, v);
    float mx = v[0];
#pragma unroll
    for (int j = 1; j < V; ++j) mx = fmaxf(mx, v[j]);
    if (mx > m) { s *= __expf(m - mx); m = mx; }
#pragma unroll
    for (int j = 0; j < V; ++j) s += __expf(v[j] - m);
  }
  // combine (m, s) pairs: warp, then block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
    m = mm;
  }
  if ((threadIdx.x & 31) == 0) { red_m[threadIdx.x >> 5] = m; red_s[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = red_m[0], S = red_s[0];
    for (int w = 1; w < XENT_THREADS / 32; ++w) {
      const float mm = fmaxf(M, red_m[w]);
      S = (M == -INFINITY ? 0.f : S * __expf(M - mm)) + (red_m[w] == -INFINITY ? 0.f : red_s[w] * __expf(red_m[w] - mm));
      M = mm;
    }
    const int t = targets[row] - v0;
    stats[row * 3 + 0] = M;
    stats[row * 3 + 1] = S;
    stats[row * 3 + 2] = (t >= 0 && t < vocab) ? XIO<T>::ld1(p + t) : 0.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(XENT_THREADS)
vp_xent_finish_kernel(T* __restrict__ logits, const int* __restrict__ targets, const float* all_stats, float* __restrict__ row_loss,
                      long long rows, int vocab, int v0, int world, float scale, int want_grad) {
  constexpr int V = XIO<T>::VEC;
  const long long row = blockIdx.x;
  float M = -INFINITY;
  // peers wrote these: read through L2 (L1 may hold the previous step's values)
  for (int r = 0; r < world; ++r) M = fmaxf(M, __ldcg(all_stats + ((long long)r * rows + row) * 3));
  float S = 0.f, tl = 0.f;
  for (int r = 0; r < world; ++r) {
    const float* st = all_stats + ((long long)r * rows + row) * 3;
    S += __ldcg(st + 1) * __expf(__ldcg(st) - M);
    tl += __ldcg(st + 2);
  }
  const float lse = M + __logf(S);
  if (threadIdx.x == 0) row_loss[row] = lse - tl;
  if (!want_grad) return;
  T* p = logits + row * vocab;
  const int t = targets[row] - v0;
  for (int i = threadIdx.x; i < vocab / V; i += XENT_THREADS) {
    float v[V];
    XIO<T>::load(p + i * V, v);
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = (__expf(v[j] - lse) - ((i * V + j) == t ? 1.f : 0.f)) * scale;
    XIO<T>::store(p + i * V, v);
  }
}

}  // namespace oa

extern "C" int oa_vp_xent_stats(int dtype, const void* logits, const int* targets, float* stats, long long rows, int vocab, int v0,
                                void* stream) {
  if (rows <= 0) return OA_OK;
  if (vocab % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return OA_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == OA_F32) oa::vp_xent_stats_kernel<float><<<(unsigned)rows, oa::XENT_THREADS, 0, st>>>((const float*)logits, targets, stats, vocab, v0);
  else if (dtype == OA_BF16)
    oa::vp_xent_stats_kernel<__nv_bfloat16><<<(unsigned)rows, oa::XENT_THREADS, 0, st>>>((const __nv_bfloat16*)logits, targets, stats, vocab, v0);
  else return OA_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_vp_xent_finish(int dtype, void* logits, const int* targets, const float* all_stats, float* row_loss, long long rows,
                                 int vocab, int v0, int world, float scale, int want_grad, void* stream) {
  if (rows <= 0) return OA_OK;
  if (vocab % 8 || (reinterpret_cast<uintptr_t>(logits) & 15)) return OA_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == OA_F32)
    oa::vp_xent_finish_kernel<float><<<(unsigned)rows, oa::XENT_THREADS, 0, st>>>((float*)logits, targets, all_stats, row_loss, rows, vocab, v0, world, scale, want_grad);
  else if (dtype == OA_BF16)
    oa::vp_xent_finish_kernel<__nv_bfloat16><<<(unsigned)rows, oa::XENT_THREADS, 0, st>>>((__nv_bfloat16*)logits, targets, all_stats, row_loss, rows, vocab, v0, world, scale, want_grad);
  else return OA_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_mean_f32(const float* x, float* out, long long n, float scale, void* stream) {
  mean_f32_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(x, out, n, scale);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
