// Exact-fp32 attention (forward and backward) for the engine's FP32 precision mode and for gradient
// checks.  Same contract as the bf16 tensor-core kernels in flash_attn.cu: q, k, v are [B*S, row_stride]
// views with head h at column h*head_dim, o is [B*S, H*head_dim], lse is [B, H, S] (natural log).
// One warp per query row (forward, dQ) or per key row (dK, dV): each output element has a single
// writer, like the reference's FlashCausal / FlashCausalBwdQ / FlashCausalBwdKV
// (Source/Private/Oa/Ml/Shader/Compute/Nn/Attention/*.slang), but keys are streamed 32 at a time with
// an online softmax, so there is no sequence-length cap.
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr int AF_MAXD = 4;  // head_dim <= 128 -> up to 4 values per lane

__global__ void attn_f32_fwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                    float* __restrict__ o, float* __restrict__ lse, int batch, int heads, int seq, int hd,
                                    long long rs, long long os, float scale, int causal) {
  long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= (long long)batch * heads * seq) return;
  const int i = (int)(w % seq);
  const int h = (int)((w / seq) % heads);
  const int b = (int)(w / ((long long)seq * heads));
  const long long row0 = (long long)b * seq;
  const float* qp = q + (row0 + i) * rs + h * hd;
  const int nd = (hd + 31) / 32;
  float acc[AF_MAXD] = {0.f, 0.f, 0.f, 0.f};
  float m = -INFINITY, l = 0.f;
  const int kend = causal ? i + 1 : seq;
  for (int j0 = 0; j0 < kend; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j < kend) {
      const float* kp = k + (row0 + j) * rs + h * hd;
      float d = 0.f;
      for (int t = 0; t < hd; ++t) d = fmaf(qp[t], kp[t], d);
      s = d * scale;
    }
    float mb = warp_max(s);
    float mn = fmaxf(m, mb);
    float alpha = __expf(m - mn);
    float p = (j < kend) ? __expf(s - mn) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int t = 0; t < AF_MAXD; ++t) acc[t] *= alpha;
    const int cnt = min(32, kend - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      float pj = __shfl_sync(0xffffffffu, p, jj);
      const float* vp = v + (row0 + j0 + jj) * rs + h * hd;
#pragma unroll
      for (int t = 0; t < AF_MAXD; ++t)
        if (t < nd && lane + 32 * t < hd) acc[t] = fmaf(pj, vp[lane + 32 * t], acc[t]);
    }
    m = mn;
  }
  float inv = 1.f / l;
#pragma unroll
  for (int t = 0; t < AF_MAXD; ++t)
    if (t < nd && lane + 32 * t < hd) o[(row0 + i) * os + h * hd + lane + 32 * t] = acc[t] * inv;
  if (lane == 0 && lse) lse[((long long)b * heads + h) * seq + i] = m + logf(l);
}

// dQ: one warp per query row.
__global__ void attn_f32_bwd_q_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                      const float* __restrict__ o, const float* __restrict__ dout,
                                      const float* __restrict__ lse, float* __restrict__ dq, int batch, int heads, int seq,
                                      int hd, long long rs, long long os, long long ds_, float scale, int causal) {
  long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= (long long)batch * heads * seq) return;
  const int i = (int)(w % seq);
  const int h = (int)((w / seq) % heads);
  const int b = (int)(w / ((long long)seq * heads));
  const long long row0 = (long long)b * seq;
  const float* qp = q + (row0 + i) * rs + h * hd;
  const float* dop = dout + (row0 + i) * os + h * hd;
  const float* op = o + (row0 + i) * os + h * hd;
  const int nd = (hd + 31) / 32;
  float delta = 0.f;
  for (int t = lane; t < hd; t += 32) delta += dop[t] * op[t];
  delta = warp_sum(delta);
  const float L = lse[((long long)b * heads + h) * seq + i];
  float acc[AF_MAXD] = {0.f, 0.f, 0.f, 0.f};
  const int kend = causal ? i + 1 : seq;
  for (int j0 = 0; j0 < kend; j0 += 32) {
    const int j = j0 + lane;
    float dsv = 0.f;
    if (j < kend) {
      const float* kp = k + (row0 + j) * rs + h * hd;
      const float* vp = v + (row0 + j) * rs + h * hd;
      float d = 0.f, dp = 0.f;
      for (int t = 0; t < hd; ++t) { d = fmaf(qp[t], kp[t], d); dp = fmaf(dop[t], vp[t], dp); }
      float p = __expf(d * scale - L);
      dsv = p * (dp - delta) * scale;
    }
    const int cnt = min(32, kend - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      float dj = __shfl_sync(0xffffffffu, dsv, jj);
      const float* kp = k + (row0 + j0 + jj) * rs + h * hd;
#pragma unroll
      for (int t = 0; t < AF_MAXD; ++t)
        if (t < nd && lane + 32 * t < hd) acc[t] = fmaf(dj, kp[lane + 32 * t], acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < AF_MAXD; ++t)
    if (t < nd && lane + 32 * t < hd) dq[(row0 + i) * ds_ + h * hd + lane + 32 * t] = acc[t];
}

// dK, dV: one warp per key row; lanes take 32 queries at a time.
__global__ void attn_f32_bwd_kv_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                       const float* __restrict__ o, const float* __restrict__ dout,
                                       const float* __restrict__ lse, float* __restrict__ dk, float* __restrict__ dv,
                                       int batch, int heads, int seq, int hd, long long rs, long long os, long long ds_,
                                       float scale, int causal) {
  long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= (long long)batch * heads * seq) return;
  const int j = (int)(w % seq);
  const int h = (int)((w / seq) % heads);
  const int b = (int)(w / ((long long)seq * heads));
  const long long row0 = (long long)b * seq;
  const float* kp = k + (row0 + j) * rs + h * hd;
  const float* vp = v + (row0 + j) * rs + h * hd;
  const int nd = (hd + 31) / 32;
  float acck[AF_MAXD] = {0.f, 0.f, 0.f, 0.f}, accv[AF_MAXD] = {0.f, 0.f, 0.f, 0.f};
  const int istart = causal ? j : 0;
  for (int i0 = istart; i0 < seq; i0 += 32) {
    const int i = i0 + lane;
    float pv = 0.f, dsv = 0.f;
    if (i < seq) {
      const float* qp = q + (row0 + i) * rs + h * hd;
      const float* dop = dout + (row0 + i) * os + h * hd;
      const float* op = o + (row0 + i) * os + h * hd;
      float d = 0.f, dp = 0.f, delta = 0.f;
      for (int t = 0; t < hd; ++t) {
        d = fmaf(qp[t], kp[t], d);
        dp = fmaf(dop[t], vp[t], dp);
        delta = fmaf(dop[t], op[t], delta);
      }
      pv = __expf(d * scale - lse[((long long)b * heads + h) * seq + i]);
      dsv = pv * (dp - delta) * scale;
    }
    const int cnt = min(32, seq - i0);
    for (int ii = 0; ii < cnt; ++ii) {
      float pi = __shfl_sync(0xffffffffu, pv, ii);
      float di = __shfl_sync(0xffffffffu, dsv, ii);
      const float* qp = q + (row0 + i0 + ii) * rs + h * hd;
      const float* dop = dout + (row0 + i0 + ii) * os + h * hd;
#pragma unroll
      for (int t = 0; t < AF_MAXD; ++t)
        if (t < nd && lane + 32 * t < hd) {
          accv[t] = fmaf(pi, dop[lane + 32 * t], accv[t]);
          acck[t] = fmaf(di, qp[lane + 32 * t], acck[t]);
        }
    }
  }
#pragma unroll
  for (int t = 0; t < AF_MAXD; ++t)
    if (t < nd && lane + 32 * t < hd) {
      dk[(row0 + j) * ds_ + h * hd + lane + 32 * t] = acck[t];
      dv[(row0 + j) * ds_ + h * hd + lane + 32 * t] = accv[t];
    }
}

}  // namespace oa

using namespace oa;

extern "C" int oa_attn_f32(const float* q, const float* k, const float* v, float* o, float* lse, int batch, int heads,
                           int seq, int head_dim, long long row_stride, long long o_row_stride, float scale, int causal,
                           void* stream) {
  if (head_dim < 1 || head_dim > 128) return OA_ERR_UNSUPPORTED;
  long long warps = (long long)batch * heads * seq;
  if (warps <= 0) return OA_OK;
  unsigned blocks = (unsigned)((warps + 3) / 4);
  attn_f32_fwd_kernel<<<blocks, 128, 0, (cudaStream_t)stream>>>(q, k, v, o, lse, batch, heads, seq, head_dim, row_stride,
                                                                o_row_stride, scale, causal);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_attn_f32_bwd(const float* q, const float* k, const float* v, const float* o, const float* dout,
                               const float* lse, float* dq, float* dk, float* dv, int batch, int heads, int seq,
                               int head_dim, long long row_stride, long long o_row_stride, long long d_row_stride,
                               float scale, int causal, void* stream) {
  if (head_dim < 1 || head_dim > 128) return OA_ERR_UNSUPPORTED;
  long long warps = (long long)batch * heads * seq;
  if (warps <= 0) return OA_OK;
  unsigned blocks = (unsigned)((warps + 3) / 4);
  cudaStream_t st = (cudaStream_t)stream;
  attn_f32_bwd_q_kernel<<<blocks, 128, 0, st>>>(q, k, v, o, dout, lse, dq, batch, heads, seq, head_dim, row_stride,
                                                o_row_stride, d_row_stride, scale, causal);
  attn_f32_bwd_kv_kernel<<<blocks, 128, 0, st>>>(q, k, v, o, dout, lse, dk, dv, batch, heads, seq, head_dim, row_stride,
                                                 o_row_stride, d_row_stride, scale, causal);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
