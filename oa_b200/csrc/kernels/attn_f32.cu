// Exact-fp32 attention (forward and backward) for the engine's FP32 precision mode and for gradient
// checks.  Same contract as the bf16 tensor-core kernels in flash_attn.cu: q, k, v are [B*S, row_stride]
// views with head h at column h*head_dim, o is [B*S, H*head_dim], lse is [B, H, S] (natural log).
//
// Every output element has a single writer, like the reference's FlashCausal / FlashCausalBwdQ /
// FlashCausalBwdKV (Source/Private/Oa/Ml/Shader/Compute/Nn/Attention/*.slang), but the other side of the
// product is streamed through shared memory 32 rows at a time with an online softmax, so there is no
// sequence-length cap and global memory is read in whole rows.
//
// Work split (all three kernels): a CTA of 128 threads owns 128 / TPR rows of one (batch, head); a row is
// shared by TPR threads (1, 2 or 4) that each keep 32 of the head dimensions in registers and combine their
// partial dot products with shuffles.  Forward and dQ rows are queries (keys / values stream through shared
// memory), dK / dV rows are keys (queries and output gradients stream through shared memory together with
// their log-sum-exp and delta = rowsum(dO * O)).
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr int AF_THREADS = 128;
constexpr int AF_TILE = 32;     // streamed rows per step
constexpr int AF_SEG = 36;      // floats per 32-dimension segment in shared memory (padded: segments land in different banks)

// Loads rows [r0, r0 + 32) of a [rows, stride] matrix (columns [col0, col0 + hd)) into sm[32][TPR][AF_SEG]; rows >= limit
// and dimensions >= hd become 0.
template <int TPR>
__device__ __forceinline__ void af_load_tile(float* sm, const float* __restrict__ g, long long stride, long long row_base, int r0,
                                             int limit, int col0, int hd) {
  for (int idx = threadIdx.x; idx < AF_TILE * TPR * 32; idx += AF_THREADS) {
    const int r = idx / (TPR * 32), c = idx % (TPR * 32);
    float x = 0.f;
    if (r0 + r < limit && c < hd) x = g[(row_base + r0 + r) * stride + col0 + c];
    sm[(r * TPR + (c >> 5)) * AF_SEG + (c & 31)] = x;
  }
}

template <int TPR>
__device__ __forceinline__ float af_reduce(float x) {
  if (TPR >= 2) x += __shfl_xor_sync(0xffffffffu, x, 1);
  if (TPR >= 4) x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

__device__ __forceinline__ float af_dot32(const float* a, const float* __restrict__ sm_row) {
  float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
  for (int t = 0; t < 32; t += 4) {
    const float4 x = *reinterpret_cast<const float4*>(sm_row + t);
    d0 = fmaf(a[t], x.x, d0); d1 = fmaf(a[t + 1], x.y, d1); d2 = fmaf(a[t + 2], x.z, d2); d3 = fmaf(a[t + 3], x.w, d3);
  }
  return (d0 + d1) + (d2 + d3);
}

__device__ __forceinline__ void af_axpy32(float* acc, float a, const float* __restrict__ sm_row) {
#pragma unroll
  for (int t = 0; t < 32; t += 4) {
    const float4 x = *reinterpret_cast<const float4*>(sm_row + t);
    acc[t] = fmaf(a, x.x, acc[t]); acc[t + 1] = fmaf(a, x.y, acc[t + 1]);
    acc[t + 2] = fmaf(a, x.z, acc[t + 2]); acc[t + 3] = fmaf(a, x.w, acc[t + 3]);
  }
}

template <int TPR>
__global__ void __launch_bounds__(AF_THREADS)
attn_f32_fwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                    float* __restrict__ o, float* __restrict__ lse, int heads, int seq, int hd, long long rs, long long os,
                    float scale, int causal) {
  constexpr int ROWS = AF_THREADS / TPR;
  __shared__ __align__(16) float sK[AF_TILE * TPR * AF_SEG];
  __shared__ __align__(16) float sV[AF_TILE * TPR * AF_SEG];
  const int h = blockIdx.y, b = blockIdx.z;
  const int i0 = blockIdx.x * ROWS;
  const int i = i0 + threadIdx.x / TPR, seg = threadIdx.x % TPR;
  const long long row0 = (long long)b * seq;
  const bool row_ok = i < seq;
  float qr[32], acc[32];
#pragma unroll
  for (int t = 0; t < 32; ++t) {
    const int d = seg * 32 + t;
    qr[t] = (row_ok && d < hd) ? q[(row0 + i) * rs + h * hd + d] * scale : 0.f;
    acc[t] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int kend = causal ? min(seq, i0 + ROWS) : seq;       // keys this CTA needs
  for (int j0 = 0; j0 < kend; j0 += AF_TILE) {
    __syncthreads();
    af_load_tile<TPR>(sK, k, rs, row0, j0, seq, h * hd, hd);
    af_load_tile<TPR>(sV, v, rs, row0, j0, seq, h * hd, hd);
    __syncthreads();
    float s[AF_TILE];
    float mt = -INFINITY;
#pragma unroll
    for (int j = 0; j < AF_TILE; ++j) {
      float d = af_reduce<TPR>(af_dot32(qr, sK + (j * TPR + seg) * AF_SEG));
      const int kj = j0 + j;
      const bool alive = kj < seq && (!causal || kj <= i);
      s[j] = alive ? d : -INFINITY;
      mt = fmaxf(mt, s[j]);
    }
    const float mn = fmaxf(m, mt);
    const float mu = (mn == -INFINITY) ? 0.f : mn;
    const float alpha = __expf(m - mu);
    float ls = 0.f;
#pragma unroll
    for (int t = 0; t < 32; ++t) acc[t] *= alpha;
#pragma unroll
    for (int j = 0; j < AF_TILE; ++j) {
      const float p = __expf(s[j] - mu);
      ls += p;
      af_axpy32(acc, p, sV + (j * TPR + seg) * AF_SEG);
    }
    l = l * alpha + ls;
    m = mn;
  }
  if (!row_ok) return;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int t = 0; t < 32; ++t) {
    const int d = seg * 32 + t;
    if (d < hd) o[(row0 + i) * os + h * hd + d] = acc[t] * inv;
  }
  if (seg == 0 && lse) lse[((long long)b * heads + h) * seq + i] = m + logf(l);
}

// dQ: rows are queries; K and V stream through shared memory.
template <int TPR>
__global__ void __launch_bounds__(AF_THREADS)
attn_f32_bwd_q_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                      const float* __restrict__ o, const float* __restrict__ dout, const float* __restrict__ lse,
                      float* __restrict__ dq, int heads, int seq, int hd, long long rs, long long os, long long ds_, float scale,
                      int causal) {
  constexpr int ROWS = AF_THREADS / TPR;
  __shared__ __align__(16) float sK[AF_TILE * TPR * AF_SEG];
  __shared__ __align__(16) float sV[AF_TILE * TPR * AF_SEG];
  const int h = blockIdx.y, b = blockIdx.z;
  const int i0 = blockIdx.x * ROWS;
  const int i = i0 + threadIdx.x / TPR, seg = threadIdx.x % TPR;
  const long long row0 = (long long)b * seq;
  const bool row_ok = i < seq;
  float qr[32], dor[32], acc[32];
  float delta = 0.f;
#pragma unroll
  for (int t = 0; t < 32; ++t) {
    const int d = seg * 32 + t;
    const bool ok = row_ok && d < hd;
    qr[t] = ok ? q[(row0 + i) * rs + h * hd + d] * scale : 0.f;
    dor[t] = ok ? dout[(row0 + i) * os + h * hd + d] : 0.f;
    if (ok) delta = fmaf(dor[t], o[(row0 + i) * os + h * hd + d], delta);
    acc[t] = 0.f;
  }
  delta = af_reduce<TPR>(delta);
  const float L = row_ok ? lse[((long long)b * heads + h) * seq + i] : 0.f;
  const int kend = causal ? min(seq, i0 + ROWS) : seq;
  for (int j0 = 0; j0 < kend; j0 += AF_TILE) {
    __syncthreads();
    af_load_tile<TPR>(sK, k, rs, row0, j0, seq, h * hd, hd);
    af_load_tile<TPR>(sV, v, rs, row0, j0, seq, h * hd, hd);
    __syncthreads();
#pragma unroll 4
    for (int j = 0; j < AF_TILE; ++j) {
      const float* kr = sK + (j * TPR + seg) * AF_SEG;
      const float d = af_reduce<TPR>(af_dot32(qr, kr));
      const float dp = af_reduce<TPR>(af_dot32(dor, sV + (j * TPR + seg) * AF_SEG));
      const int kj = j0 + j;
      const bool alive = row_ok && kj < seq && (!causal || kj <= i);
      const float ds = alive ? __expf(d - L) * (dp - delta) * scale : 0.f;
      af_axpy32(acc, ds, kr);
    }
  }
  if (!row_ok) return;
#pragma unroll
  for (int t = 0; t < 32; ++t) {
    const int d = seg * 32 + t;
    if (d < hd) dq[(row0 + i) * ds_ + h * hd + d] = acc[t];
  }
}

// dK, dV: rows are keys; Q and dO stream through shared memory with the queries' log-sum-exp and delta.
template <int TPR>
__global__ void __launch_bounds__(AF_THREADS)
attn_f32_bwd_kv_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                       const float* __restrict__ o, const float* __restrict__ dout, const float* __restrict__ lse,
                       float* __restrict__ dk, float* __restrict__ dv, int heads, int seq, int hd, long long rs, long long os,
                       long long ds_, float scale, int causal) {
  constexpr int ROWS = AF_THREADS / TPR;
  __shared__ __align__(16) float sQ[AF_TILE * TPR * AF_SEG];
  __shared__ __align__(16) float sDO[AF_TILE * TPR * AF_SEG];
  __shared__ float sL[AF_TILE], sDelta[AF_TILE];
  const int h = blockIdx.y, b = blockIdx.z;
  const int j0 = blockIdx.x * ROWS;
  const int j = j0 + threadIdx.x / TPR, seg = threadIdx.x % TPR;
  const long long row0 = (long long)b * seq;
  const bool row_ok = j < seq;
  float kr[32], vr[32], acck[32], accv[32];
#pragma unroll
  for (int t = 0; t < 32; ++t) {
    const int d = seg * 32 + t;
    const bool ok = row_ok && d < hd;
    kr[t] = ok ? k[(row0 + j) * rs + h * hd + d] * scale : 0.f;
    vr[t] = ok ? v[(row0 + j) * rs + h * hd + d] : 0.f;
    acck[t] = 0.f; accv[t] = 0.f;
  }
  const int istart = causal ? (j0 / AF_TILE) * AF_TILE : 0;    // first query tile any key of this CTA can see
  for (int i0 = istart; i0 < seq; i0 += AF_TILE) {
    __syncthreads();
    af_load_tile<TPR>(sQ, q, rs, row0, i0, seq, h * hd, hd);
    af_load_tile<TPR>(sDO, dout, os, row0, i0, seq, h * hd, hd);
    {
      // delta of the 32 queries: 4 threads per query, shuffle-combined
      const int r = threadIdx.x >> 2, part = threadIdx.x & 3;
      float dl = 0.f;
      if (i0 + r < seq)
        for (int d = part; d < hd; d += 4) dl = fmaf(dout[(row0 + i0 + r) * os + h * hd + d], o[(row0 + i0 + r) * os + h * hd + d], dl);
      dl += __shfl_xor_sync(0xffffffffu, dl, 1);
      dl += __shfl_xor_sync(0xffffffffu, dl, 2);
      if (part == 0) {
        sDelta[r] = dl;
        sL[r] = (i0 + r < seq) ? lse[((long long)b * heads + h) * seq + i0 + r] : INFINITY;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int ii = 0; ii < AF_TILE; ++ii) {
      const float* qrow = sQ + (ii * TPR + seg) * AF_SEG;
      const float* dorow = sDO + (ii * TPR + seg) * AF_SEG;
      const float d = af_reduce<TPR>(af_dot32(kr, qrow));
      const float dp = af_reduce<TPR>(af_dot32(vr, dorow));
      const int qi = i0 + ii;
      const bool alive = row_ok && qi < seq && (!causal || j <= qi);
      const float p = alive ? __expf(d - sL[ii]) : 0.f;
      const float ds = p * (dp - sDelta[ii]);     // the key registers carry the scale: dK = scale * dS^T Q restored below
      af_axpy32(accv, p, dorow);
      af_axpy32(acck, ds, qrow);
    }
  }
  if (!row_ok) return;
#pragma unroll
  for (int t = 0; t < 32; ++t) {
    const int d = seg * 32 + t;
    if (d < hd) {
      dk[(row0 + j) * ds_ + h * hd + d] = acck[t] * scale;
      dv[(row0 + j) * ds_ + h * hd + d] = accv[t];
    }
  }
}

}  // namespace oa

using namespace oa;

static inline int af_tpr(int hd) { return hd <= 32 ? 1 : (hd <= 64 ? 2 : 4); }

extern "C" int oa_attn_f32(const float* q, const float* k, const float* v, float* o, float* lse, int batch, int heads,
                           int seq, int head_dim, long long row_stride, long long o_row_stride, float scale, int causal,
                           void* stream) {
  if (head_dim < 1 || head_dim > 128) return OA_ERR_UNSUPPORTED;
  if (batch <= 0 || heads <= 0 || seq <= 0) return OA_OK;
  if (heads > 65535 || batch > 65535) return OA_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int tpr = af_tpr(head_dim), rows = AF_THREADS / tpr;
  dim3 grid((seq + rows - 1) / rows, heads, batch);
  if (tpr == 1) attn_f32_fwd_kernel<1><<<grid, AF_THREADS, 0, st>>>(q, k, v, o, lse, heads, seq, head_dim, row_stride, o_row_stride, scale, causal);
  else if (tpr == 2) attn_f32_fwd_kernel<2><<<grid, AF_THREADS, 0, st>>>(q, k, v, o, lse, heads, seq, head_dim, row_stride, o_row_stride, scale, causal);
  else attn_f32_fwd_kernel<4><<<grid, AF_THREADS, 0, st>>>(q, k, v, o, lse, heads, seq, head_dim, row_stride, o_row_stride, scale, causal);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_attn_f32_bwd(const float* q, const float* k, const float* v, const float* o, const float* dout,
                               const float* lse, float* dq, float* dk, float* dv, int batch, int heads, int seq,
                               int head_dim, long long row_stride, long long o_row_stride, long long d_row_stride,
                               float scale, int causal, void* stream) {
  if (head_dim < 1 || head_dim > 128) return OA_ERR_UNSUPPORTED;
  if (batch <= 0 || heads <= 0 || seq <= 0) return OA_OK;
  if (heads > 65535 || batch > 65535) return OA_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int tpr = af_tpr(head_dim), rows = AF_THREADS / tpr;
  dim3 grid((seq + rows - 1) / rows, heads, batch);
#define AF_BWD(T)                                                                                                                \
  attn_f32_bwd_q_kernel<T><<<grid, AF_THREADS, 0, st>>>(q, k, v, o, dout, lse, dq, heads, seq, head_dim, row_stride, o_row_stride, \
                                                        d_row_stride, scale, causal);                                            \
  attn_f32_bwd_kv_kernel<T><<<grid, AF_THREADS, 0, st>>>(q, k, v, o, dout, lse, dk, dv, heads, seq, head_dim, row_stride,          \
                                                         o_row_stride, d_row_stride, scale, causal);
  if (tpr == 1) { AF_BWD(1) } else if (tpr == 2) { AF_BWD(2) } else { AF_BWD(4) }
#undef AF_BWD
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
