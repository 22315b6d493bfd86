// Sparse dropless mixture-of-experts routing kernels: fused router (softmax + top-k + renormalised route weights),
// multi-CTA deterministic expert plan, row gather / combine with their single-writer backward passes.
//
// Reference contracts: TopK descending with ties to the lower index (Core/Shader/Compute/Flat/TopK.slang:39-77);
// route weights w[t,k] = p[t,e_k] / sum_k p[t,e_k] over the UNBIASED softmax probabilities, selection may add a
// routing bias (Ml/Shader/Compute/Nn/Moe/MoeRouteWeights.slang:24-40, Nn/Moe/Moe.cpp:205-225); packing is stable
// expert-major with the token-major route order preserved inside each expert (MoeExpertPlan.slang:1-4); combine
// out[t,:] = sum_k gate[t,k] * packed[inv[t,k],:] (MoeCombine.slang:1-22).
// The reference's plan kernel is one work-group looping over all routes; here it is three small multi-CTA kernels
// (per-block histograms, scan, stable placement) that scale to hundreds of thousands of routes, and every expert
// segment is padded to a multiple of 128 rows so that grouped tensor-core GEMM tiles never straddle two experts.
#include "common.cuh"
#include "api.h"

namespace oa {

template <typename T> __device__ __forceinline__ float mld(const T* p);
template <> __device__ __forceinline__ float mld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float mld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void mst(T* p, float v);
template <> __device__ __forceinline__ void mst<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void mst<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int MOE_MAX_E = 256;
constexpr int MOE_MAX_K = 8;
constexpr int MOE_SEG_ALIGN = 128;

// One warp per token: probs = softmax(logits), indices = top-k of (logits + sel_bias), weights = renormalised probs.
template <typename T>
__global__ void moe_router_kernel(const T* __restrict__ logits, const float* __restrict__ sel_bias, float* __restrict__ probs,
                                  int* __restrict__ topk_idx, float* __restrict__ topk_w, long long tokens, int E, int Kk) {
  long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  constexpr int PER = MOE_MAX_E / 32;
  float v[PER], sel[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    int e = lane + 32 * i;
    v[i] = e < E ? mld<T>(logits + t * E + e) : -INFINITY;
    sel[i] = e < E ? v[i] + (sel_bias ? sel_bias[e] : 0.f) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) { v[i] = lane + 32 * i < E ? __expf(v[i] - mx) : 0.f; sum += v[i]; }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] *= inv;
    if (lane + 32 * i < E) probs[t * E + lane + 32 * i] = v[i];
  }
  float wsum = 0.f;
  float myw = 0.f;
  int myidx = 0;
  for (int k = 0; k < Kk; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      int e = lane + 32 * i;
      if (sel[i] > best || (sel[i] == best && e < bi)) { best = sel[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    // the owner lane removes the winner and reports its probability
    float pw = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if (lane + 32 * i == bi) { pw = v[i]; sel[i] = -INFINITY; }
    pw = warp_sum(pw);
    wsum += pw;
    if (lane == k) { myw = pw; myidx = bi; }
  }
  if (lane < Kk) {
    topk_idx[t * Kk + lane] = myidx;
    topk_w[t * Kk + lane] = myw / wsum;
  }
}

// dlogits from (dW over the selected routes, dProbs added by the balancing loss).
//   w_k = p_k / S  =>  dp_sel_k = (dw_k - sum_j dw_j w_j) / S ;  dlogits = p * (dp - sum_e dp_e p_e)
template <typename T>
__global__ void moe_router_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ topk_idx,
                                      const float* __restrict__ topk_w, const float* __restrict__ dw,
                                      const float* __restrict__ dprobs_col, float dprobs_scale, T* __restrict__ dlogits,
                                      long long tokens, int E, int Kk) {
  long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  constexpr int PER = MOE_MAX_E / 32;
  float S = 0.f, dot = 0.f;
  for (int k = 0; k < Kk; ++k) {
    int e = topk_idx[t * Kk + k];
    S += probs[t * E + e];
    dot += dw[t * Kk + k] * topk_w[t * Kk + k];
  }
  float p[PER], dp[PER];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    int e = lane + 32 * i;
    p[i] = e < E ? probs[t * E + e] : 0.f;
    dp[i] = (e < E && dprobs_col) ? dprobs_col[e] * dprobs_scale : 0.f;
    for (int k = 0; k < Kk; ++k)
      if (e == topk_idx[t * Kk + k]) dp[i] += (dw[t * Kk + k] - dot) / S;
    acc += dp[i] * p[i];
  }
  acc = warp_sum(acc);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    int e = lane + 32 * i;
    if (e < E) mst<T>(dlogits + t * E + e, p[i] * (dp[i] - acc));
  }
}

// ---- plan ------------------------------------------------------------------------------------------------
constexpr int PLAN_THREADS = 1024;

// block_hist[b][e] = number of routes of expert e among routes [b*1024, b*1024+1024)
__global__ void moe_plan_count_kernel(const int* __restrict__ topk_idx, long long routes, int E, int* __restrict__ block_hist) {
  __shared__ int hist[MOE_MAX_E];
  for (int i = threadIdx.x; i < E; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  long long r = (long long)blockIdx.x * PLAN_THREADS + threadIdx.x;
  if (r < routes) {
    int e = topk_idx[r];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) block_hist[(long long)blockIdx.x * E + i] = hist[i];
}

// One block: counts[e], padded offsets[e+1], block_base[b][e] = offsets[e] + routes of e in earlier blocks.
__global__ void moe_plan_scan_kernel(const int* __restrict__ block_hist, int nblocks, int E, int* __restrict__ counts,
                                     int* __restrict__ offsets, int* __restrict__ block_base) {
  __shared__ int total[MOE_MAX_E];
  __shared__ int start[MOE_MAX_E + 1];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int b = 0; b < nblocks; ++b) {
      int c = block_hist[(long long)b * E + e];
      block_base[(long long)b * E + e] = run;
      run += c;
    }
    total[e] = run;
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = off;
      offsets[e] = off;
      off += (total[e] + MOE_SEG_ALIGN - 1) / MOE_SEG_ALIGN * MOE_SEG_ALIGN;
    }
    start[E] = off;
    offsets[E] = off;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int b = 0; b < nblocks; ++b) block_base[(long long)b * E + e] += start[e];
}

// Stable placement: position = block_base[b][e] + (routes of e in earlier warps of this block) + rank inside the warp.
__global__ void moe_plan_place_kernel(const int* __restrict__ topk_idx, long long routes, int E, int Kk,
                                      const int* __restrict__ block_base, int* __restrict__ packed_token,
                                      int* __restrict__ inverse) {
  __shared__ int warp_hist[PLAN_THREADS / 32][MOE_MAX_E];   // 32 KB for E = 256
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = lane; i < E; i += 32) warp_hist[warp][i] = 0;
  __syncwarp();
  long long r = (long long)blockIdx.x * PLAN_THREADS + threadIdx.x;
  int e = (r < routes) ? topk_idx[r] : -1;
  bool valid = e >= 0 && e < E;
  unsigned peers = __match_any_sync(0xffffffffu, valid ? e : -1 - lane);
  int rank = __popc(peers & ((1u << lane) - 1));
  if (valid && rank == 0) warp_hist[warp][e] = __popc(peers);
  __syncthreads();
  // exclusive scan over the warps of this block, per expert
  for (int x = threadIdx.x; x < E; x += blockDim.x) {
    int run = 0;
    for (int w = 0; w < PLAN_THREADS / 32; ++w) {
      int c = warp_hist[w][x];
      warp_hist[w][x] = run;
      run += c;
    }
  }
  __syncthreads();
  if (valid) {
    int pos = block_base[(long long)blockIdx.x * E + e] + warp_hist[warp][e] + rank;
    packed_token[pos] = (int)(r / Kk);
    inverse[r] = pos;
  } else if (r < routes) {
    inverse[r] = -1;
  }
}

// packed[r,:] = x[packed_token[r],:]  (zero rows for padding, packed_token[r] < 0)
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ packed_token, T* __restrict__ packed,
                                  const int* __restrict__ offsets, int E, int dim, long long max_rows) {
  const long long rows = max_rows;   // rows past the last segment are padding too (packed_token = -1): keep them zero
  (void)offsets; (void)E;
  const int vec = dim / 8;
  long long total = rows * vec;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long r = i / vec;
    int c = (int)(i % vec) * 8;
    int t = packed_token[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t >= 0) v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + (long long)t * dim + c);
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(packed) + r * dim + c) = v;
  }
}

// out[t,:] = (base ? base[t,:] : 0) + sum_k gate[t,k] * packed[inverse[t,k],:]      (bf16, 8 columns per thread)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ packed, const float* __restrict__ gate,
                                   const int* __restrict__ inverse, const __nv_bfloat16* __restrict__ base,
                                   __nv_bfloat16* __restrict__ out, long long tokens, int Kk, int dim) {
  const int vec = dim / 8;
  long long total = tokens * vec;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long t = i / vec;
    int c = (int)(i % vec) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (base) {
      uint4 b = *reinterpret_cast<const uint4*>(base + t * dim + c);
      float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
      acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
    }
    for (int k = 0; k < Kk; ++k) {
      int r = inverse[t * Kk + k];
      if (r < 0) continue;
      float g = gate[t * Kk + k];
      uint4 b = *reinterpret_cast<const uint4*>(packed + (long long)r * dim + c);
      float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
      acc[0] += g * f0.x; acc[1] += g * f0.y; acc[2] += g * f1.x; acc[3] += g * f1.y;
      acc[4] += g * f2.x; acc[5] += g * f2.y; acc[6] += g * f3.x; acc[7] += g * f3.y;
    }
    *reinterpret_cast<uint4*>(out + t * dim + c) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                              pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// Backward of combine: dpacked[r,:] = gate[route(r)] * dout[token(r),:] (zero for padding rows) and
// dgate[t,k] = <dout[t,:], packed[inverse[t,k],:]>.  One warp per packed row; each route has one writer.
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ packed, const float* __restrict__ gate,
                                       const int* __restrict__ inverse, const int* __restrict__ packed_token,
                                       const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dpacked,
                                       float* __restrict__ dgate, const int* __restrict__ offsets, int E, int Kk, int dim,
                                       long long max_rows) {
  const long long rows = max_rows;
  (void)offsets; (void)E;
  long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  int t = packed_token[r];
  __nv_bfloat16* dp = dpacked + r * dim;
  if (t < 0) {
    for (int c = lane * 8; c < dim; c += 256) *reinterpret_cast<uint4*>(dp + c) = make_uint4(0, 0, 0, 0);
    return;
  }
  int kk = 0;
  for (int k = 0; k < Kk; ++k)
    if (inverse[(long long)t * Kk + k] == (int)r) kk = k;
  const float g = gate[(long long)t * Kk + kk];
  float dot = 0.f;
  for (int c = lane * 8; c < dim; c += 256) {
    uint4 d = *reinterpret_cast<const uint4*>(dout + (long long)t * dim + c);
    uint4 y = *reinterpret_cast<const uint4*>(packed + r * dim + c);
    float2 d0 = unpack_bf16x2(d.x), d1 = unpack_bf16x2(d.y), d2 = unpack_bf16x2(d.z), d3 = unpack_bf16x2(d.w);
    float2 y0 = unpack_bf16x2(y.x), y1 = unpack_bf16x2(y.y), y2 = unpack_bf16x2(y.z), y3 = unpack_bf16x2(y.w);
    dot += d0.x * y0.x + d0.y * y0.y + d1.x * y1.x + d1.y * y1.y + d2.x * y2.x + d2.y * y2.y + d3.x * y3.x + d3.y * y3.y;
    *reinterpret_cast<uint4*>(dp + c) = make_uint4(pack_bf16x2(g * d0.x, g * d0.y), pack_bf16x2(g * d1.x, g * d1.y),
                                                   pack_bf16x2(g * d2.x, g * d2.y), pack_bf16x2(g * d3.x, g * d3.y));
  }
  dot = warp_sum(dot);
  if (lane == 0) dgate[(long long)t * Kk + kk] = dot;
}

// Backward of gather: dx[t,:] = (base ? base[t,:] : 0) + sum_k dpacked[inverse[t,k],:]  (single writer per token)
__global__ void moe_gather_bwd_kernel(const __nv_bfloat16* __restrict__ dpacked, const int* __restrict__ inverse,
                                      const __nv_bfloat16* __restrict__ base, __nv_bfloat16* __restrict__ dx, long long tokens,
                                      int Kk, int dim) {
  const int vec = dim / 8;
  long long total = tokens * vec;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long t = i / vec;
    int c = (int)(i % vec) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (base) {
      uint4 b = *reinterpret_cast<const uint4*>(base + t * dim + c);
      float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
      acc[0] = f0.x; acc[1] = f0.y; acc[2] = f1.x; acc[3] = f1.y; acc[4] = f2.x; acc[5] = f2.y; acc[6] = f3.x; acc[7] = f3.y;
    }
    for (int k = 0; k < Kk; ++k) {
      int r = inverse[t * Kk + k];
      if (r < 0) continue;
      uint4 b = *reinterpret_cast<const uint4*>(dpacked + (long long)r * dim + c);
      float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
      acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y; acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
    }
    *reinterpret_cast<uint4*>(dx + t * dim + c) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                             pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

__global__ void fill_int_kernel(int* p, long long n, int v) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = v;
}

}  // namespace oa

using namespace oa;
#define ST ((cudaStream_t)stream)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH)

static inline int mgrid(long long work) {
  long long b = (work + 255) / 256;
  if (b > 148 * 8) b = 148 * 8;
  return (int)(b < 1 ? 1 : b);
}

extern "C" int oa_moe_router(int dtype, const void* logits, const float* sel_bias, float* probs, int* topk_idx, float* topk_w,
                             long long tokens, int E, int K, void* stream) {
  if (E < 1 || E > MOE_MAX_E || K < 1 || K > MOE_MAX_K || K > E) return OA_ERR_UNSUPPORTED;
  if (tokens <= 0) return OA_OK;
  unsigned blocks = (unsigned)((tokens + 7) / 8);
  if (dtype == OA_F32) moe_router_kernel<float><<<blocks, 256, 0, ST>>>((const float*)logits, sel_bias, probs, topk_idx, topk_w, tokens, E, K);
  else if (dtype == OA_BF16) moe_router_kernel<__nv_bfloat16><<<blocks, 256, 0, ST>>>((const __nv_bfloat16*)logits, sel_bias, probs, topk_idx, topk_w, tokens, E, K);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}
extern "C" int oa_moe_router_bwd(int dtype, const float* probs, const int* topk_idx, const float* topk_w, const float* dw,
                                 const float* dprobs_col, float dprobs_scale, void* dlogits, long long tokens, int E, int K,
                                 void* stream) {
  if (E < 1 || E > MOE_MAX_E || K < 1 || K > MOE_MAX_K) return OA_ERR_UNSUPPORTED;
  if (tokens <= 0) return OA_OK;
  unsigned blocks = (unsigned)((tokens + 7) / 8);
  if (dtype == OA_F32) moe_router_bwd_kernel<float><<<blocks, 256, 0, ST>>>(probs, topk_idx, topk_w, dw, dprobs_col, dprobs_scale, (float*)dlogits, tokens, E, K);
  else if (dtype == OA_BF16) moe_router_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, ST>>>(probs, topk_idx, topk_w, dw, dprobs_col, dprobs_scale, (__nv_bfloat16*)dlogits, tokens, E, K);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}
// scratch: int[2 * nblocks * E] with nblocks = ceil(routes / 1024).  Outputs: counts[E], offsets[E+1] (padded to 128),
// packed_token[max_rows] (-1 for padding), inverse[routes].
extern "C" size_t oa_moe_plan_scratch_bytes(long long routes, int E) {
  long long nb = (routes + PLAN_THREADS - 1) / PLAN_THREADS;
  return (size_t)(2 * nb * E) * sizeof(int);
}
extern "C" int oa_moe_plan(const int* topk_idx, long long tokens, int K, int E, int* counts, int* offsets, int* packed_token,
                           int* inverse, long long max_rows, int* scratch, void* stream) {
  if (E < 1 || E > MOE_MAX_E || K < 1) return OA_ERR_UNSUPPORTED;
  long long routes = tokens * K;
  if (routes <= 0) return OA_OK;
  if (max_rows < routes + (long long)E * (MOE_SEG_ALIGN - 1)) return OA_ERR_ARG;
  int nb = (int)((routes + PLAN_THREADS - 1) / PLAN_THREADS);
  int* block_hist = scratch;
  int* block_base = scratch + (long long)nb * E;
  fill_int_kernel<<<mgrid(max_rows), 256, 0, ST>>>(packed_token, max_rows, -1);
  moe_plan_count_kernel<<<nb, PLAN_THREADS, 0, ST>>>(topk_idx, routes, E, block_hist);
  moe_plan_scan_kernel<<<1, 256, 0, ST>>>(block_hist, nb, E, counts, offsets, block_base);
  moe_plan_place_kernel<<<nb, PLAN_THREADS, 0, ST>>>(topk_idx, routes, E, K, block_base, packed_token, inverse);
  return CHECK_LAUNCH();
}
extern "C" int oa_moe_gather(const void* x, const int* packed_token, void* packed, const int* offsets, int E, int dim,
                             long long max_rows, void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  moe_gather_kernel<__nv_bfloat16><<<mgrid(max_rows * (dim / 8)), 256, 0, ST>>>((const __nv_bfloat16*)x, packed_token, (__nv_bfloat16*)packed, offsets, E, dim, max_rows);
  return CHECK_LAUNCH();
}
extern "C" int oa_moe_combine(const void* packed, const float* gate, const int* inverse, const void* base, void* out,
                              long long tokens, int K, int dim, void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  moe_combine_kernel<<<mgrid(tokens * (dim / 8)), 256, 0, ST>>>((const __nv_bfloat16*)packed, gate, inverse, (const __nv_bfloat16*)base, (__nv_bfloat16*)out, tokens, K, dim);
  return CHECK_LAUNCH();
}
extern "C" int oa_moe_combine_bwd(const void* packed, const float* gate, const int* inverse, const int* packed_token,
                                  const void* dout, void* dpacked, float* dgate, const int* offsets, int E, int K, int dim,
                                  long long max_rows, void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  unsigned blocks = (unsigned)((max_rows + 7) / 8);
  moe_combine_bwd_kernel<<<blocks, 256, 0, ST>>>((const __nv_bfloat16*)packed, gate, inverse, packed_token, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dpacked, dgate, offsets, E, K, dim, max_rows);
  return CHECK_LAUNCH();
}
extern "C" int oa_moe_gather_bwd(const void* dpacked, const int* inverse, const void* base, void* dx, long long tokens, int K,
                                 int dim, void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  moe_gather_bwd_kernel<<<mgrid(tokens * (dim / 8)), 256, 0, ST>>>((const __nv_bfloat16*)dpacked, inverse, (const __nv_bfloat16*)base, (__nv_bfloat16*)dx, tokens, K, dim);
  return CHECK_LAUNCH();
}
