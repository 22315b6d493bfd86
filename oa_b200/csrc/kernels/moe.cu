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

// =====================================================================================================
// Expert parallelism: the all-to-all dispatch / combine as peer-memory kernels (one process per GPU).
// Rank s owns experts [s*E_loc, (s+1)*E_loc).  Every rank knows counts_all[src][e] (exchanged with oa_peer_push), so
// every sender can compute the row that each of its routes occupies in the owner's expert-major buffer:
//   row = seg_off[e] + sum_{s' < s} counts_all[s'][e] + (rank of the route among this sender's routes to e)
// with seg_off the owner's 128-padded segment starts.  Dispatch = gather fused with the remote store (rows are
// written straight into the owner's buffer over NVLink), combine = weighted pull of the result rows from the owners.
namespace oa {

struct PeerPtrs { void* ptr[8]; };

// Per-route destination: route_rank[r], route_row[r]; owner-side plan: loc_offsets[E_loc+1], loc_counts[E_loc],
// loc_valid[max_rows] (1 = real row, 0 = padding).
__global__ void ep_layout_kernel(const int* __restrict__ counts_all, const int* __restrict__ topk_idx, const int* __restrict__ inverse,
                                 const int* __restrict__ offsets_local, int* __restrict__ route_rank, int* __restrict__ route_row,
                                 int* __restrict__ loc_offsets, int* __restrict__ loc_counts, int* __restrict__ counts_global,
                                 int* __restrict__ need, long long routes, int E, int world, int rank) {
  __shared__ int seg_off[MOE_MAX_E];     // owner-local padded segment start of every global expert
  __shared__ int src_off[MOE_MAX_E];     // rows of earlier sources inside the segment
  const int E_loc = E / world;
  if (threadIdx.x == 0) {
    int most = 0;
    for (int d = 0; d < world; ++d) {
      int off = 0;
      for (int le = 0; le < E_loc; ++le) {
        int e = d * E_loc + le, tot = 0, before = 0;
        for (int s = 0; s < world; ++s) {
          int c = counts_all[s * E + e];
          if (s < rank) before += c;
          tot += c;
        }
        seg_off[e] = off;
        src_off[e] = before;
        if (blockIdx.x == 0) {
          counts_global[e] = tot;
          if (d == rank) { loc_offsets[le] = off; loc_counts[le] = tot; }
        }
        off += (tot + MOE_SEG_ALIGN - 1) / MOE_SEG_ALIGN * MOE_SEG_ALIGN;
      }
      if (blockIdx.x == 0 && d == rank) { loc_offsets[E_loc] = off; if (need) need[0] = off; }
      most = max(most, off);
    }
    // rows (padded per expert) that the busiest owner receives: the same number on every rank, computed from the same table,
    // so that all ranks size their peer-mapped buffers alike before any row moves
    if (blockIdx.x == 0 && need) need[1] = most;
  }
  __syncthreads();
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < routes; r += stride) {
    int e = topk_idx[r];
    int within = inverse[r] - offsets_local[e];
    route_rank[r] = e / E_loc;
    route_row[r] = seg_off[e] + src_off[e] + within;
  }
}

// dst_peer[route_rank[r]][route_row[r], :] = scale_r * x[token(r), :]   (scale = gate[r] when given)
__global__ void ep_push_rows_kernel(const __nv_bfloat16* __restrict__ x, PeerPtrs dst, const int* __restrict__ route_rank,
                                    const int* __restrict__ route_row, const float* __restrict__ gate, long long routes, int Kk,
                                    int dim, int cap_rows, int* status) {
  const int vec = dim / 8;
  long long total = routes * vec;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long r = i / vec;
    int c = (int)(i % vec) * 8;
    uint4 v = *reinterpret_cast<const uint4*>(x + (r / Kk) * dim + c);
    if (gate) {
      const float g = gate[r];
      float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
      v = make_uint4(pack_bf16x2(g * f0.x, g * f0.y), pack_bf16x2(g * f1.x, g * f1.y), pack_bf16x2(g * f2.x, g * f2.y),
                     pack_bf16x2(g * f3.x, g * f3.y));
    }
    const int row = route_row[r];
    if (row < 0 || row >= cap_rows) {          // more rows than the owner's buffer holds: drop and report
      if (c == 0) report_error(status, OA_KERR_BAD_ARG);
      continue;
    }
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(dst.ptr[route_rank[r]]) + (long long)row * dim + c;
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(d), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
}

// out[t,:] = base[t,:] + sum_k gate[t,k] * src_peer[rank(t,k)][row(t,k), :]; when dgate != null also
// dgate[t,k] = <dout[t,:], src_peer[..][row,:]> (backward of combine) and nothing is written to out.
__global__ void ep_pull_rows_kernel(PeerPtrs src, const int* __restrict__ route_rank, const int* __restrict__ route_row,
                                    const float* __restrict__ gate, const __nv_bfloat16* __restrict__ base,
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
      const long long r = t * Kk + k;
      const float g = gate ? gate[r] : 1.f;
      const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.ptr[route_rank[r]]) + (long long)route_row[r] * dim + c;
      uint4 b;
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(s) : "memory");
      float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
      acc[0] += g * f0.x; acc[1] += g * f0.y; acc[2] += g * f1.x; acc[3] += g * f1.y;
      acc[4] += g * f2.x; acc[5] += g * f2.y; acc[6] += g * f3.x; acc[7] += g * f3.y;
    }
    *reinterpret_cast<uint4*>(out + t * dim + c) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                              pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

// dgate[r] = <dout[token(r), :], src_peer[rank(r)][row(r), :]>, one warp per route.
__global__ void ep_pull_dot_kernel(PeerPtrs src, const int* __restrict__ route_rank, const int* __restrict__ route_row,
                                   const __nv_bfloat16* __restrict__ dout, float* __restrict__ dgate, long long routes, int Kk, int dim) {
  long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= routes) return;
  const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.ptr[route_rank[r]]) + (long long)route_row[r] * dim;
  const __nv_bfloat16* d = dout + (r / Kk) * dim;
  float dot = 0.f;
  for (int c = lane * 8; c < dim; c += 256) {
    uint4 y;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(y.x), "=r"(y.y), "=r"(y.z), "=r"(y.w) : "l"(s + c) : "memory");
    uint4 g = *reinterpret_cast<const uint4*>(d + c);
    float2 d0 = unpack_bf16x2(g.x), d1 = unpack_bf16x2(g.y), d2 = unpack_bf16x2(g.z), d3 = unpack_bf16x2(g.w);
    float2 y0 = unpack_bf16x2(y.x), y1 = unpack_bf16x2(y.y), y2 = unpack_bf16x2(y.z), y3 = unpack_bf16x2(y.w);
    dot += d0.x * y0.x + d0.y * y0.y + d1.x * y1.x + d1.y * y1.y + d2.x * y2.x + d2.y * y2.y + d3.x * y3.x + d3.y * y3.y;
  }
  dot = warp_sum(dot);
  if (lane == 0) dgate[r] = dot;
}

// Zeroes the padding rows of an owner-side buffer: rows [loc_offsets[le] + loc_counts[le], loc_offsets[le+1]).
__global__ void ep_zero_pad_kernel(__nv_bfloat16* buf, const int* __restrict__ loc_offsets, const int* __restrict__ loc_counts,
                                   int E_loc, int dim) {
  const int le = blockIdx.y;
  const int r0 = loc_offsets[le] + loc_counts[le], r1 = loc_offsets[le + 1];
  const int vec = dim / 8;
  long long total = (long long)(r1 - r0) * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    *reinterpret_cast<uint4*>(buf + (long long)(r0 + i / vec) * dim + (i % vec) * 8) = make_uint4(0, 0, 0, 0);
}

}  // namespace oa

static PeerPtrs make_peers(const void* const* ptrs, int world) {
  PeerPtrs t;
  for (int i = 0; i < 8; ++i) t.ptr[i] = i < world ? const_cast<void*>(ptrs[i]) : nullptr;
  return t;
}

extern "C" int oa_ep_layout(const int* counts_all, const int* topk_idx, const int* inverse, const int* offsets_local,
                            int* route_rank, int* route_row, int* loc_offsets, int* loc_counts, int* counts_global, int* need,
                            long long routes, int E, int world, int rank, void* stream) {
  if (E > MOE_MAX_E || world < 1 || world > 8 || E % world) return OA_ERR_ARG;
  ep_layout_kernel<<<mgrid(routes), 256, 0, ST>>>(counts_all, topk_idx, inverse, offsets_local, route_rank, route_row, loc_offsets,
                                                  loc_counts, counts_global, need, routes, E, world, rank);
  return CHECK_LAUNCH();
}
extern "C" int oa_ep_push_rows(const void* x, const void* const* dst_peers, const int* route_rank, const int* route_row,
                               const float* gate, long long routes, int K, int dim, int world, int cap_rows, int* status,
                               void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  ep_push_rows_kernel<<<mgrid(routes * (dim / 8)), 256, 0, ST>>>((const __nv_bfloat16*)x, make_peers(dst_peers, world), route_rank,
                                                                route_row, gate, routes, K, dim, cap_rows, status);
  return CHECK_LAUNCH();
}
extern "C" int oa_ep_pull_rows(const void* const* src_peers, const int* route_rank, const int* route_row, const float* gate,
                               const void* base, void* out, long long tokens, int K, int dim, int world, void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  ep_pull_rows_kernel<<<mgrid(tokens * (dim / 8)), 256, 0, ST>>>(make_peers(src_peers, world), route_rank, route_row, gate,
                                                                (const __nv_bfloat16*)base, (__nv_bfloat16*)out, tokens, K, dim);
  return CHECK_LAUNCH();
}
extern "C" int oa_ep_pull_dot(const void* const* src_peers, const int* route_rank, const int* route_row, const void* dout,
                              float* dgate, long long routes, int K, int dim, int world, void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  unsigned blocks = (unsigned)((routes + 7) / 8);
  ep_pull_dot_kernel<<<blocks, 256, 0, ST>>>(make_peers(src_peers, world), route_rank, route_row, (const __nv_bfloat16*)dout, dgate,
                                             routes, K, dim);
  return CHECK_LAUNCH();
}
extern "C" int oa_ep_zero_pad(void* buf, const int* loc_offsets, const int* loc_counts, int E_loc, int dim, void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  dim3 grid(8, E_loc);
  ep_zero_pad_kernel<<<grid, 256, 0, ST>>>((__nv_bfloat16*)buf, loc_offsets, loc_counts, E_loc, dim);
  return CHECK_LAUNCH();
}
