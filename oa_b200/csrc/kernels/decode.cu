// KV-cache serving kernels.  The reference has no KV cache: its generation loop re-runs the whole window for every new
// token (Tutorial/Cpp/Ml/Nlp/TutorialNlpCommon.h:145-177), so these are new.
//   oa_kv_append   copies the (already rotated) key and value rows of new tokens into the per-layer cache
//                  [batch, heads, max_seq, head_dim];
//   oa_decode_attn one query token per sequence against the cache: one CTA per (sequence, head), four warps stride over
//                  the cached positions with a running softmax (lane = position for q.k, lane = head-dim slice for p.v),
//                  the four partial states are merged through shared memory.  Bandwidth bound: it reads the cache once.
#include "common.cuh"
#include "api.h"

namespace oa {

__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k_src, const __nv_bfloat16* __restrict__ v_src, long long src_stride,
                                 __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, int batch, int s_new, int heads, int hd,
                                 int pos0, int max_seq, const int* __restrict__ pos_dev) {
  // one thread per 8 elements of one (token, head) row; pos_dev (optional) adds a device-resident offset so that a decode
  // step captured in a CUDA graph advances without host-side parameters
  if (pos_dev) pos0 += *pos_dev;
  const int vec = hd >> 3;
  const long long total = (long long)batch * s_new * heads * vec;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec);
    long long r = i / vec;
    const int h = (int)(r % heads); r /= heads;
    const int s = (int)(r % s_new);
    const int b = (int)(r / s_new);
    const long long src = ((long long)b * s_new + s) * src_stride + h * hd + v * 8;
    if (pos0 + s >= max_seq) continue;           // a full cache drops the token (the host checks capacity before replaying)
    const long long dst = (((long long)b * heads + h) * max_seq + pos0 + s) * hd + v * 8;
    *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(k_src + src);
    *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(v_src + src);
  }
}

template <int HD>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ kc,
                   const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out, long long out_stride, int heads, int len,
                   int max_seq, float scale_log2, const int* __restrict__ pos_dev) {
  if (pos_dev) len = min(len + *pos_dev, max_seq);
  constexpr int PER = HD / 32;                  // head-dim elements per lane in the p.v phase
  __shared__ float s_q[HD];
  __shared__ float s_m[4], s_l[4];
  __shared__ float s_acc[4][HD];
  const int b = blockIdx.x / heads, h = blockIdx.x % heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int d = threadIdx.x; d < HD; d += 128) s_q[d] = __bfloat162float(q[(long long)b * q_stride + h * HD + d]);
  __syncthreads();
  const __nv_bfloat16* kb = kc + ((long long)b * heads + h) * max_seq * HD;
  const __nv_bfloat16* vb = vc + ((long long)b * heads + h) * max_seq * HD;
  float m = -INFINITY, l = 0.f, acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  for (int s0 = warp * 32; s0 < len; s0 += 128) {
    const int s = s0 + lane;
    float sc = -INFINITY;
    if (s < len) {
      const uint4* kr = reinterpret_cast<const uint4*>(kb + (long long)s * HD);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) {
        const uint4 kv = kr[j];
        const float2 a = unpack_bf16x2(kv.x), c = unpack_bf16x2(kv.y), e = unpack_bf16x2(kv.z), g = unpack_bf16x2(kv.w);
        const float* qq = s_q + j * 8;
        dot += a.x * qq[0] + a.y * qq[1] + c.x * qq[2] + c.y * qq[3] + e.x * qq[4] + e.y * qq[5] + g.x * qq[6] + g.y * qq[7];
      }
      sc = dot * scale_log2;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float p = s < len ? fast_exp2(sc - m_new) : 0.f;
    const float corr = m == -INFINITY ? 0.f : fast_exp2(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] *= corr;
    const int n = min(32, len - s0);
    // p.v: eight value rows are loaded before the first multiply-add so that their latencies overlap
#pragma unroll 1
    for (int j0 = 0; j0 < n; j0 += 8) {
      uint2 vv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = min(j0 + u, n - 1);
        const __nv_bfloat16* vr = vb + (long long)(s0 + j) * HD + lane * PER;
        if (PER == 4) vv[u] = *reinterpret_cast<const uint2*>(vr);
        else vv[u] = make_uint2(*reinterpret_cast<const uint32_t*>(vr), 0u);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float pj = (j0 + u < n) ? __shfl_sync(0xffffffffu, p, (j0 + u) & 31) : 0.f;
        const float2 a = unpack_bf16x2(vv[u].x);
        acc[0] += pj * a.x; acc[1] += pj * a.y;
        if (PER == 4) {
          const float2 c = unpack_bf16x2(vv[u].y);
          acc[2] += pj * c.x; acc[3] += pj * c.y;
        }
      }
    }
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < PER; ++i) s_acc[warp][lane * PER + i] = acc[i];
  __syncthreads();
  const float M = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
  float L = 0.f;
  float w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) { w[k] = s_m[k] == -INFINITY ? 0.f : fast_exp2(s_m[k] - M); L += s_l[k] * w[k]; }
  for (int d = threadIdx.x; d < HD; d += 128) {
    const float v = s_acc[0][d] * w[0] + s_acc[1][d] * w[1] + s_acc[2][d] * w[2] + s_acc[3][d] * w[3];
    out[(long long)b * out_stride + h * HD + d] = __float2bfloat16_rn(L > 0.f ? v / L : 0.f);
  }
}

}  // namespace oa

using namespace oa;

extern "C" int oa_kv_append(const void* k_src, const void* v_src, long long src_stride, void* k_cache, void* v_cache, int batch,
                            int s_new, int heads, int head_dim, int pos0, int max_seq, const int* pos_dev, void* stream) {
  if (head_dim % 8 || src_stride % 8) return OA_ERR_ALIGN;
  if (pos0 < 0 || (!pos_dev && pos0 + s_new > max_seq)) return OA_ERR_ARG;
  if (batch <= 0 || s_new <= 0) return OA_OK;
  const long long total = (long long)batch * s_new * heads * (head_dim / 8);
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  kv_append_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)k_src, (const __nv_bfloat16*)v_src, src_stride,
                                                                 (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, batch, s_new, heads,
                                                                 head_dim, pos0, max_seq, pos_dev);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_decode_attn(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out, long long out_stride,
                              int batch, int heads, int head_dim, int len, int max_seq, float scale, const int* pos_dev,
                              void* stream) {
  if (len <= 0 || len > max_seq) return OA_ERR_ARG;
  if (batch <= 0) return OA_OK;
  const float sl2 = scale * 1.4426950408889634f;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = batch * heads;
  if (head_dim == 128)
    decode_attn_kernel<128><<<grid, 128, 0, st>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                                                  (__nv_bfloat16*)out, out_stride, heads, len, max_seq, sl2, pos_dev);
  else if (head_dim == 64)
    decode_attn_kernel<64><<<grid, 128, 0, st>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                                                 (__nv_bfloat16*)out, out_stride, heads, len, max_seq, sl2, pos_dev);
  else return OA_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
