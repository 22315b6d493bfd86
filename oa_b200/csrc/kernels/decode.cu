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


// ------------------------------------------------------------------------------------------------ streamed decode attention
// The cache of one (sequence, head) is contiguous, so a tile of TILE positions is one 16 KB block of K and one of V.  A
// producer thread streams those blocks into a 3-stage shared-memory ring with bulk asynchronous copies (completion counted
// on an mbarrier), four consumer warps compute out of shared memory: the memory system always has about 96 KB per CTA in
// flight, independent of how fast the arithmetic warps issue.  CTAs are persistent over (sequence, head, split) items; each
// item leaves an unnormalised partial (acc, m, l) that `decode_merge_kernel` combines.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

constexpr int DA_STAGES = 3;
constexpr int DA_TILE_BYTES = 16384;

template <int HD>
__global__ void __launch_bounds__(160)
decode_attn_stream_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ kc,
                          const __nv_bfloat16* __restrict__ vc, float* __restrict__ partial, int heads, int n_bh, int splits, int len,
                          int max_seq, float scale_log2, const int* __restrict__ pos_dev, int* __restrict__ status) {
  constexpr int LPR = HD / 64;            // lanes that share one row in the q.k phase (64 head-dim elements each)
  constexpr int RW = 32 / LPR;            // rows per warp and tile
  constexpr int TILE = 4 * RW;            // positions per tile: 64 (HD 128) or 128 (HD 64) -> 16 KB of K and of V
  constexpr int CH = HD / 8;              // 16-byte chunks per row
  constexpr int RG = 32 / CH;             // rows handled at once in the p.v phase
  static_assert(TILE * HD * 2 == DA_TILE_BYTES, "tile size");
  extern __shared__ __align__(128) unsigned char da_smem[];
  __shared__ uint64_t full_bar[DA_STAGES], empty_bar[DA_STAGES];
  __shared__ float4 s_qlo[16], s_qhi[16];
  __shared__ float s_m[4], s_l[4];
  __shared__ float s_acc[4][HD];
  __shared__ int s_fail;
  if (pos_dev) len = min(len + *pos_dev, max_seq);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = n_bh * splits;
  const int per = (((len + splits - 1) / splits + TILE - 1) / TILE) * TILE;     // positions per split, whole tiles
  if (threadIdx.x == 0) {
    for (int i = 0; i < DA_STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 4); }
    mbar_fence_init();
    s_fail = 0;
  }
  __syncthreads();
  unsigned char* tiles = da_smem;

  if (warp == 4) {
    // ---------------------------------------------------------------- producer (one thread)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const int bh = item / splits, sp = item - bh * splits;
        const int lo = sp * per, hi = min(len, lo + per);
        const __nv_bfloat16* kb = kc + (long long)bh * max_seq * HD;
        const __nv_bfloat16* vb = vc + (long long)bh * max_seq * HD;
        for (int pos = lo; pos < hi; pos += TILE, ++it) {
          const uint32_t stage = it % DA_STAGES, phase = (it / DA_STAGES) & 1u;
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) { report_error(status, OA_KERR_WAIT_EMPTY); ok = false; break; }
          const uint32_t bytes = (uint32_t)min(TILE, hi - pos) * HD * 2u;
          mbar_expect_tx(&full_bar[stage], 2u * bytes);
          bulk_load_1d(tiles + stage * 2 * DA_TILE_BYTES, kb + (long long)pos * HD, bytes, &full_bar[stage]);
          bulk_load_1d(tiles + stage * 2 * DA_TILE_BYTES + DA_TILE_BYTES, vb + (long long)pos * HD, bytes, &full_bar[stage]);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- consumers (four warps)
    const int r = lane % RW, hh = lane / RW;            // q.k: row within the warp's rows, 64-element half of the row
    const int pc = lane % CH, pg = lane / CH;           // p.v: 16-byte chunk of the head dim, row group
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      const int bh = item / splits, sp = item - bh * splits;
      const int b = bh / heads, h = bh - b * heads;
      const int lo = sp * per, hi = min(len, lo + per);
      if (threadIdx.x < HD / 4) {
        const __nv_bfloat16* qp = q + (long long)b * q_stride + h * HD + threadIdx.x * 4;
        const float4 v = make_float4(__bfloat162float(qp[0]), __bfloat162float(qp[1]), __bfloat162float(qp[2]), __bfloat162float(qp[3]));
        if (threadIdx.x & 1) s_qhi[threadIdx.x >> 1] = v; else s_qlo[threadIdx.x >> 1] = v;
      }
      consumer_sync();
      float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int pos = lo; pos < hi && ok; pos += TILE, ++it) {
        const uint32_t stage = it % DA_STAGES, phase = (it / DA_STAGES) & 1u;
        if (!warp_wait(&full_bar[stage], phase)) { report_error(status, OA_KERR_WAIT_FULL); ok = false; break; }
        const unsigned char* sk = tiles + stage * 2 * DA_TILE_BYTES;
        const unsigned char* sv = sk + DA_TILE_BYTES;
        const int row0 = warp * RW;                       // this warp's first row of the tile
        const int valid_rows = min(TILE, hi - pos) - row0; // rows of this warp that hold cached positions (may be <= 0)
        // q.k: each lane takes eight 16-byte chunks of its row, starting at a row-dependent chunk (no bank conflicts)
        float dot = 0.f;
        const unsigned char* krow = sk + (row0 + r) * (HD * 2);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = 8 * hh + ((j + r) & 7);
          const uint4 kv = *reinterpret_cast<const uint4*>(krow + c * 16);
          const float4 ql = s_qlo[c], qh = s_qhi[c];
          const float2 a = unpack_bf16x2(kv.x), e = unpack_bf16x2(kv.y), f = unpack_bf16x2(kv.z), g = unpack_bf16x2(kv.w);
          dot += a.x * ql.x + a.y * ql.y + e.x * ql.z + e.y * ql.w + f.x * qh.x + f.y * qh.y + g.x * qh.z + g.y * qh.w;
        }
        if (LPR == 2) dot += __shfl_xor_sync(0xffffffffu, dot, 16);
        const bool live = r < valid_rows;
        const float sc = live ? dot * scale_log2 : -INFINITY;
        const float m_new = fmaxf(m, warp_max(sc));
        const float p = (live && m_new != -INFINITY) ? fast_exp2(sc - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : fast_exp2(m - m_new);
        l = l * corr + warp_sum(p) * (1.f / LPR);
        m = m_new;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= corr;
        // p.v: a quarter warp reads 128 contiguous bytes of one value row
#pragma unroll
        for (int i = 0; i < RW / RG; ++i) {
          const int row = i * RG + pg;
          const float pj = __shfl_sync(0xffffffffu, p, row);
          if (pj != 0.f) {
            const uint4 vv = *reinterpret_cast<const uint4*>(sv + (row0 + row) * (HD * 2) + pc * 16);
            const float2 a = unpack_bf16x2(vv.x), e = unpack_bf16x2(vv.y), f = unpack_bf16x2(vv.z), g = unpack_bf16x2(vv.w);
            acc[0] += pj * a.x; acc[1] += pj * a.y; acc[2] += pj * e.x; acc[3] += pj * e.y;
            acc[4] += pj * f.x; acc[5] += pj * f.y; acc[6] += pj * g.x; acc[7] += pj * g.y;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
      }
      // row groups of the p.v phase hold partial sums of the same chunk
#pragma unroll
      for (int o = CH; o < 32; o <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
      if (lane == 0) { s_m[warp] = m; s_l[warp] = l; if (!ok) s_fail = 1; }
      if (pg == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) s_acc[warp][pc * 8 + i] = acc[i];
      }
      consumer_sync();
      const float M = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
      float w[4], L = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) { w[k] = s_m[k] == -INFINITY ? 0.f : fast_exp2(s_m[k] - M); L += s_l[k] * w[k]; }
      float* dst = partial + (long long)item * (HD + 2);
      if (threadIdx.x < HD) {
        const int d = threadIdx.x;
        dst[d] = s_acc[0][d] * w[0] + s_acc[1][d] * w[1] + s_acc[2][d] * w[2] + s_acc[3][d] * w[3];
      }
      if (threadIdx.x == 0) { dst[HD] = M; dst[HD + 1] = L; }
      const bool stop = s_fail != 0;                      // the same for all four warps: they leave together
      consumer_sync();
      if (stop) break;
    }
  }
  __syncthreads();
}

// out[b, h, :] = sum_s acc_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)
template <int HD>
__global__ void decode_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, long long out_stride, int heads,
                                    int splits) {
  const int bh = blockIdx.x, b = bh / heads, h = bh - b * heads, d = threadIdx.x;
  const float* src = partial + (long long)bh * splits * (HD + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, src[s * (HD + 2) + HD]);
  float L = 0.f, v = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = src[s * (HD + 2) + HD];
    const float w = ms == -INFINITY ? 0.f : fast_exp2(ms - M);
    L += src[s * (HD + 2) + HD + 1] * w;
    v += src[s * (HD + 2) + d] * w;
  }
  out[(long long)b * out_stride + h * HD + d] = __float2bfloat16_rn(L > 0.f ? v / L : 0.f);
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

// Streamed variant: `partial` holds batch*heads*splits*(head_dim+2) floats.  Both kernels are captured together in a graph.
extern "C" size_t oa_decode_attn_stream_scratch_bytes(int batch, int heads, int head_dim, int splits) {
  return (size_t)batch * heads * splits * (head_dim + 2) * sizeof(float);
}

template <int HD>
static int launch_decode_stream(const void* q, long long q_stride, const void* kc, const void* vc, void* out, long long out_stride, int batch,
                                int heads, int len, int max_seq, float sl2, const int* pos_dev, void* partial, int splits, int* status,
                                cudaStream_t st) {
  static bool set = false;
  const int smem = DA_STAGES * 2 * DA_TILE_BYTES;
  if (!set) {
    if (cudaFuncSetAttribute(decode_attn_stream_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return OA_ERR_LAUNCH;
    set = true;
  }
  const int n_bh = batch * heads, items = n_bh * splits;
  const int grid = items < 2 * 148 ? items : 2 * 148;
  decode_attn_stream_kernel<HD><<<grid, 160, smem, st>>>((const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                                                         (float*)partial, heads, n_bh, splits, len, max_seq, sl2, pos_dev, status);
  decode_merge_kernel<HD><<<n_bh, HD, 0, st>>>((const float*)partial, (__nv_bfloat16*)out, out_stride, heads, splits);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_decode_attn_stream(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                     long long out_stride, int batch, int heads, int head_dim, int len, int max_seq, float scale,
                                     const int* pos_dev, void* partial, int splits, int* status, void* stream) {
  if (len <= 0 || len > max_seq || splits < 1 || splits > 64) return OA_ERR_ARG;
  if ((((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0) return OA_ERR_ALIGN;
  if (batch <= 0) return OA_OK;
  const float sl2 = scale * 1.4426950408889634f;
  if (head_dim == 128)
    return launch_decode_stream<128>(q, q_stride, k_cache, v_cache, out, out_stride, batch, heads, len, max_seq, sl2, pos_dev, partial, splits,
                                     status, (cudaStream_t)stream);
  if (head_dim == 64)
    return launch_decode_stream<64>(q, q_stride, k_cache, v_cache, out, out_stride, batch, heads, len, max_seq, sl2, pos_dev, partial, splits,
                                    status, (cudaStream_t)stream);
  return OA_ERR_UNSUPPORTED;
}
