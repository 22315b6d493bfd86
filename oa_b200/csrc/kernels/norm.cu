// RMSNorm and LayerNorm, forward and backward (fp32 or bf16 storage, fp32 math).
//   RMSNorm:   y = x * rsqrt(mean(x^2) + eps) * w                  (Nn/RmsNorm/RmsNorm.slang:26-30)
//   LayerNorm: y = (x - mean) * rsqrt(var + eps) * w + b, biased variance, two passes
//              (Nn/LayerNorm/LayerNorm.slang:41-58)
// One warp per row.  The forward can add a residual stream first (ResidualRmsNorm); the backward
// can add the gradient that arrives through the residual path, so that no separate add kernels run.
// Weight / bias gradients: each warp keeps private column partials in shared memory over the rows it
// owns, each CTA writes one partial row to a scratch buffer, and a second kernel sums the partial
// rows in a fixed order (deterministic, no atomics).
#include "common.cuh"
#include "api.h"

namespace oa {

template <typename T> struct NIO;
template <> struct NIO<float> {
  static constexpr int VEC = 4;
  __device__ static void load(const float* p, float* v) {
    float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  __device__ static void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct NIO<__nv_bfloat16> {
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
};

constexpr int NORM_THREADS = 256;
constexpr int NORM_WARPS = NORM_THREADS / 32;

template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, float* __restrict__ rstd_out,
                   long long rows, int cols, float eps, const T* __restrict__ res_in, T* __restrict__ res_out) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = NIO<T>::VEC;
  const int lane = threadIdx.x & 31;
  const long long warp_global = (long long)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * NORM_WARPS;
  for (long long row = warp_global; row < rows; row += warp_stride) {
    const T* px = x + row * cols;
    float ss = 0.f;
    for (int c = lane * V; c < cols; c += 32 * V) {
      float v[V];
      NIO<T>::load(px + c, v);
      if (res_in) {
        float r[V];
        NIO<T>::load(res_in + row * cols + c, r);
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] += r[j];
        NIO<T>::store(res_out + row * cols + c, v);
      }
#pragma unroll
      for (int j = 0; j < V; ++j) ss += v[j] * v[j];
    }
    ss = warp_sum(ss);
    float rstd = rsqrtf(ss / (float)cols + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    const T* src = res_in ? res_out + row * cols : px;
    if (res_in) __syncwarp();
    for (int c = lane * V; c < cols; c += 32 * V) {
      float v[V], g[V];
      NIO<T>::load(src + c, v);
      NIO<T>::load(w + c, g);
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = v[j] * rstd * g[j];
      NIO<T>::store(y + row * cols + c, v);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres);   dw partial += dy * xhat
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ dy,
                   const float* __restrict__ rstd_in, T* __restrict__ dx, long long rows, int cols,
                   const T* __restrict__ dres, float* __restrict__ partial, int warps_used) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float s_dw[];  // [warps_used][cols]
  constexpr int V = NIO<T>::VEC;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < warps_used * cols; i += blockDim.x) s_dw[i] = 0.f;
  __syncthreads();
  if (warp < warps_used) {
    float* my = s_dw + (size_t)warp * cols;
    const long long warp_global = (long long)blockIdx.x * warps_used + warp;
    const long long warp_stride = (long long)gridDim.x * warps_used;
    for (long long row = warp_global; row < rows; row += warp_stride) {
      const T* px = x + row * cols;
      const T* pd = dy + row * cols;
      const float rstd = rstd_in[row];
      float dot = 0.f;
      for (int c = lane * V; c < cols; c += 32 * V) {
        float v[V], d[V], g[V];
        NIO<T>::load(px + c, v);
        NIO<T>::load(pd + c, d);
        NIO<T>::load(w + c, g);
#pragma unroll
        for (int j = 0; j < V; ++j) dot += d[j] * g[j] * v[j] * rstd;
      }
      dot = warp_sum(dot) / (float)cols;
      for (int c = lane * V; c < cols; c += 32 * V) {
        float v[V], d[V], g[V], o[V];
        NIO<T>::load(px + c, v);
        NIO<T>::load(pd + c, d);
        NIO<T>::load(w + c, g);
        if (dres) NIO<T>::load(dres + row * cols + c, o);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float xh = v[j] * rstd;
          my[c + j] += d[j] * xh;
          float r = rstd * (d[j] * g[j] - xh * dot);
          o[j] = dres ? o[j] + r : r;
        }
        NIO<T>::store(dx + row * cols + c, o);
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < warps_used; ++k) s += s_dw[(size_t)k * cols + c];
    partial[(size_t)blockIdx.x * cols + c] = s;
  }
}

// bf16 fast path for cols = ITER * 256: a lane always owns the same 8 * ITER columns, so the row stays in registers
// between the two passes (packed bf16), the weight is loaded once, and the dw partial sums live in registers across all
// rows of the warp instead of read-modify-write traffic on shared memory.
template <int ITER>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                       const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx, long long rows, const __nv_bfloat16* __restrict__ dres,
                       float* __restrict__ partial) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float s_dw[];  // [NORM_WARPS][cols]
  constexpr int cols = ITER * 256;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4 wp[ITER];
  float acc[ITER][8];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    wp[it] = *reinterpret_cast<const uint4*>(w + it * 256 + lane * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[it][j] = 0.f;
  }
  const long long warp_global = (long long)blockIdx.x * NORM_WARPS + warp;
  const long long warp_stride = (long long)gridDim.x * NORM_WARPS;
  for (long long row = warp_global; row < rows; row += warp_stride) {
    uint4 xp[ITER], dp[ITER], rp[ITER];
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      xp[it] = *reinterpret_cast<const uint4*>(x + row * cols + it * 256 + lane * 8);
      dp[it] = *reinterpret_cast<const uint4*>(dy + row * cols + it * 256 + lane * 8);
      if (dres) rp[it] = *reinterpret_cast<const uint4*>(dres + row * cols + it * 256 + lane * 8);
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const uint32_t xs[4] = {xp[it].x, xp[it].y, xp[it].z, xp[it].w}, ds[4] = {dp[it].x, dp[it].y, dp[it].z, dp[it].w},
                     ws[4] = {wp[it].x, wp[it].y, wp[it].z, wp[it].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 xv = unpack_bf16x2(xs[k]), dv = unpack_bf16x2(ds[k]), wv = unpack_bf16x2(ws[k]);
        dot += dv.x * wv.x * xv.x + dv.y * wv.y * xv.y;
      }
    }
    dot = warp_sum(dot) * rstd / (float)cols;
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const uint32_t xs[4] = {xp[it].x, xp[it].y, xp[it].z, xp[it].w}, ds[4] = {dp[it].x, dp[it].y, dp[it].z, dp[it].w},
                     ws[4] = {wp[it].x, wp[it].y, wp[it].z, wp[it].w}, rs[4] = {rp[it].x, rp[it].y, rp[it].z, rp[it].w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 xv = unpack_bf16x2(xs[k]), dv = unpack_bf16x2(ds[k]), wv = unpack_bf16x2(ws[k]);
        const float xh0 = xv.x * rstd, xh1 = xv.y * rstd;
        acc[it][2 * k] += dv.x * xh0;
        acc[it][2 * k + 1] += dv.y * xh1;
        float r0 = rstd * (dv.x * wv.x - xh0 * dot), r1 = rstd * (dv.y * wv.y - xh1 * dot);
        if (dres) { const float2 rv = unpack_bf16x2(rs[k]); r0 += rv.x; r1 += rv.y; }
        o[k] = pack_bf16x2(r0, r1);
      }
      *reinterpret_cast<uint4*>(dx + row * cols + it * 256 + lane * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
#pragma unroll
  for (int it = 0; it < ITER; ++it)
#pragma unroll
    for (int j = 0; j < 8; ++j) s_dw[(size_t)warp * cols + it * 256 + lane * 8 + j] = acc[it][j];
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_WARPS; ++k) s += s_dw[(size_t)k * cols + c];
    partial[(size_t)blockIdx.x * cols + c] = s;
  }
}

template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b, T* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, long long rows, int cols, float eps) {
  constexpr int V = NIO<T>::VEC;
  const int lane = threadIdx.x & 31;
  const long long warp_global = (long long)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
  const long long warp_stride = (long long)gridDim.x * NORM_WARPS;
  for (long long row = warp_global; row < rows; row += warp_stride) {
    const T* px = x + row * cols;
    float s = 0.f;
    for (int c = lane * V; c < cols; c += 32 * V) {
      float v[V];
      NIO<T>::load(px + c, v);
#pragma unroll
      for (int j = 0; j < V; ++j) s += v[j];
    }
    float mean = warp_sum(s) / (float)cols;
    float ss = 0.f;
    for (int c = lane * V; c < cols; c += 32 * V) {
      float v[V];
      NIO<T>::load(px + c, v);
#pragma unroll
      for (int j = 0; j < V; ++j) ss += (v[j] - mean) * (v[j] - mean);
    }
    float rstd = rsqrtf(warp_sum(ss) / (float)cols + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    for (int c = lane * V; c < cols; c += 32 * V) {
      float v[V], g[V], bb[V];
      NIO<T>::load(px + c, v);
      NIO<T>::load(w + c, g);
      if (b) NIO<T>::load(b + c, bb);
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = (v[j] - mean) * rstd * g[j] + (b ? bb[j] : 0.f);
      NIO<T>::store(y + row * cols + c, v);
    }
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) with g = dy * w;  dw += dy * xhat;  db += dy
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ dy,
                     const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
                     long long rows, int cols, float* __restrict__ partial, int warps_used, int nblocks_total) {
  extern __shared__ float s_acc[];  // [warps_used][2][cols]
  constexpr int V = NIO<T>::VEC;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < warps_used * 2 * cols; i += blockDim.x) s_acc[i] = 0.f;
  __syncthreads();
  if (warp < warps_used) {
    float* my_dw = s_acc + (size_t)warp * 2 * cols;
    float* my_db = my_dw + cols;
    const long long warp_global = (long long)blockIdx.x * warps_used + warp;
    const long long warp_stride = (long long)gridDim.x * warps_used;
    for (long long row = warp_global; row < rows; row += warp_stride) {
      const T* px = x + row * cols;
      const T* pd = dy + row * cols;
      const float mean = mean_in[row], rstd = rstd_in[row];
      float sg = 0.f, sgx = 0.f;
      for (int c = lane * V; c < cols; c += 32 * V) {
        float v[V], d[V], g[V];
        NIO<T>::load(px + c, v);
        NIO<T>::load(pd + c, d);
        NIO<T>::load(w + c, g);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float gg = d[j] * g[j];
          sg += gg;
          sgx += gg * (v[j] - mean) * rstd;
        }
      }
      sg = warp_sum(sg) / (float)cols;
      sgx = warp_sum(sgx) / (float)cols;
      for (int c = lane * V; c < cols; c += 32 * V) {
        float v[V], d[V], g[V], o[V];
        NIO<T>::load(px + c, v);
        NIO<T>::load(pd + c, d);
        NIO<T>::load(w + c, g);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float xh = (v[j] - mean) * rstd;
          my_dw[c + j] += d[j] * xh;
          my_db[c + j] += d[j];
          o[j] = rstd * (d[j] * g[j] - sg - xh * sgx);
        }
        NIO<T>::store(dx + row * cols + c, o);
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float s0 = 0.f, s1 = 0.f;
    for (int k = 0; k < warps_used; ++k) {
      s0 += s_acc[(size_t)k * 2 * cols + c];
      s1 += s_acc[(size_t)k * 2 * cols + cols + c];
    }
    partial[(size_t)blockIdx.x * cols + c] = s0;
    partial[((size_t)nblocks_total + blockIdx.x) * cols + c] = s1;
  }
}

// out[c] (+)= sum_p partial[p, c]: 32 columns x 8 row groups per CTA (block 256), shared-memory reduce over the groups.
template <typename D>
__global__ void __launch_bounds__(256)
partial_rows_sum_kernel(const float* __restrict__ partial, D* __restrict__ out, int nparts, int cols, int accumulate) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < cols)
    for (int p = ry; p < nparts; p += 8) s += partial[(size_t)p * cols + c];
  red[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][cx];
    if constexpr (sizeof(D) == 4) {
      if (accumulate) t += out[c];
      out[c] = t;
    } else {
      if (accumulate) t += __bfloat162float(out[c]);
      out[c] = __float2bfloat16_rn(t);
    }
  }
}

static int norm_bwd_blocks(long long rows) {
  long long b = (rows + NORM_WARPS - 1) / NORM_WARPS;
  if (b > 148 * 2) b = 148 * 2;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace oa

using namespace oa;
#define ST ((cudaStream_t)stream)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH)

// Scratch for the weight (and bias) gradient partial rows: float[2 * blocks * cols].
extern "C" size_t oa_norm_bwd_scratch_bytes(long long rows, int cols) {
  return (size_t)2 * norm_bwd_blocks(rows) * cols * sizeof(float);
}

extern "C" int oa_rmsnorm_fwd(int dtype, const void* x, const void* w, void* y, float* rstd, long long rows, int cols,
                              float eps, const void* residual_in, void* residual_out, void* stream) {
  if (rows <= 0) return OA_OK;
  if (cols % 8) return OA_ERR_ALIGN;
  long long b = (rows + NORM_WARPS - 1) / NORM_WARPS;
  if (b > 148 * 8) b = 148 * 8;
  if (dtype == OA_F32)
    rmsnorm_fwd_kernel<float><<<(int)b, NORM_THREADS, 0, ST>>>((const float*)x, (const float*)w, (float*)y, rstd, rows, cols, eps, (const float*)residual_in, (float*)residual_out);
  else if (dtype == OA_BF16)
    launch_pdl(rmsnorm_fwd_kernel<__nv_bfloat16>, dim3((unsigned)b), dim3(NORM_THREADS), 0, ST, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, rows, cols, eps, (const __nv_bfloat16*)residual_in, (__nv_bfloat16*)residual_out);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) return OA_ERR_LAUNCH;
  }
  return OA_OK;
}

extern "C" int oa_rmsnorm_bwd(int dtype, const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                              void* dw, int dw_dtype, long long rows, int cols, const void* dres, float* scratch,
                              int accumulate_dw, void* stream) {
  if (rows <= 0) return OA_OK;
  if (cols % 8) return OA_ERR_ALIGN;
  int warps = NORM_WARPS;
  while (warps > 1 && (size_t)warps * cols * 4 > 200 * 1024) warps >>= 1;
  size_t smem = (size_t)warps * cols * 4;
  if (smem > 200 * 1024) return OA_ERR_TOO_LARGE;
  int blocks = norm_bwd_blocks(rows);
  int rc;
  if (dtype == OA_F32) {
    if ((rc = set_smem(rmsnorm_bwd_kernel<float>, smem))) return rc;
    rmsnorm_bwd_kernel<float><<<blocks, NORM_THREADS, smem, ST>>>((const float*)x, (const float*)w, (const float*)dy, rstd, (float*)dx, rows, cols, (const float*)dres, scratch, warps);
  } else if (dtype == OA_BF16 && warps == NORM_WARPS && cols % 256 == 0 && cols / 256 <= 4 &&
             ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(w) |
               reinterpret_cast<uintptr_t>(dres)) & 15) == 0) {
    const __nv_bfloat16 *bx = (const __nv_bfloat16*)x, *bw = (const __nv_bfloat16*)w, *bd = (const __nv_bfloat16*)dy, *br = (const __nv_bfloat16*)dres;
    __nv_bfloat16* bo = (__nv_bfloat16*)dx;
#define OA_RMS_BWD_REG(IT)                                                                          \
    if ((rc = set_smem(rmsnorm_bwd_reg_kernel<IT>, smem))) return rc;                                \
    launch_pdl(rmsnorm_bwd_reg_kernel<IT>, dim3(blocks), dim3(NORM_THREADS), smem, ST, bx, bw, bd, rstd, bo, rows, br, scratch)
    switch (cols / 256) {
      case 1: OA_RMS_BWD_REG(1); break;
      case 2: OA_RMS_BWD_REG(2); break;
      case 3: OA_RMS_BWD_REG(3); break;
      default: OA_RMS_BWD_REG(4); break;
    }
#undef OA_RMS_BWD_REG
  } else if (dtype == OA_BF16) {
    if ((rc = set_smem(rmsnorm_bwd_kernel<__nv_bfloat16>, smem))) return rc;
    rmsnorm_bwd_kernel<__nv_bfloat16><<<blocks, NORM_THREADS, smem, ST>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, rstd, (__nv_bfloat16*)dx, rows, cols, (const __nv_bfloat16*)dres, scratch, warps);
  } else return OA_ERR_UNSUPPORTED;
  if (dw) {
    if (dw_dtype == OA_F32) launch_pdl(partial_rows_sum_kernel<float>, dim3((cols + 31) / 32), dim3(256), 0, ST, scratch, (float*)dw, blocks, cols, accumulate_dw);
    else launch_pdl(partial_rows_sum_kernel<__nv_bfloat16>, dim3((cols + 31) / 32), dim3(256), 0, ST, scratch, (__nv_bfloat16*)dw, blocks, cols, accumulate_dw);
  }
  return CHECK_LAUNCH();
}

extern "C" int oa_layernorm_fwd(int dtype, const void* x, const void* w, const void* b, void* y, float* mean,
                                float* rstd, long long rows, int cols, float eps, void* stream) {
  if (rows <= 0) return OA_OK;
  if (cols % 8) return OA_ERR_ALIGN;
  long long nb = (rows + NORM_WARPS - 1) / NORM_WARPS;
  if (nb > 148 * 8) nb = 148 * 8;
  if (dtype == OA_F32)
    layernorm_fwd_kernel<float><<<(int)nb, NORM_THREADS, 0, ST>>>((const float*)x, (const float*)w, (const float*)b, (float*)y, mean, rstd, rows, cols, eps);
  else if (dtype == OA_BF16)
    layernorm_fwd_kernel<__nv_bfloat16><<<(int)nb, NORM_THREADS, 0, ST>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, mean, rstd, rows, cols, eps);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}

extern "C" int oa_layernorm_bwd(int dtype, const void* x, const void* w, const void* dy, const float* mean,
                                const float* rstd, void* dx, void* dw, void* db, int dw_dtype, long long rows, int cols,
                                float* scratch, int accumulate_dw, void* stream) {
  if (rows <= 0) return OA_OK;
  if (cols % 8) return OA_ERR_ALIGN;
  int warps = NORM_WARPS;
  while (warps > 1 && (size_t)warps * 2 * cols * 4 > 200 * 1024) warps >>= 1;
  size_t smem = (size_t)warps * 2 * cols * 4;
  if (smem > 200 * 1024) return OA_ERR_TOO_LARGE;
  int blocks = norm_bwd_blocks(rows);
  int rc;
  if (dtype == OA_F32) {
    if ((rc = set_smem(layernorm_bwd_kernel<float>, smem))) return rc;
    layernorm_bwd_kernel<float><<<blocks, NORM_THREADS, smem, ST>>>((const float*)x, (const float*)w, (const float*)dy, mean, rstd, (float*)dx, rows, cols, scratch, warps, blocks);
  } else if (dtype == OA_BF16) {
    if ((rc = set_smem(layernorm_bwd_kernel<__nv_bfloat16>, smem))) return rc;
    layernorm_bwd_kernel<__nv_bfloat16><<<blocks, NORM_THREADS, smem, ST>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, mean, rstd, (__nv_bfloat16*)dx, rows, cols, scratch, warps, blocks);
  } else return OA_ERR_UNSUPPORTED;
  float* part_db = scratch + (size_t)blocks * cols;
  if (dw_dtype == OA_F32) {
    if (dw) partial_rows_sum_kernel<float><<<(cols + 31) / 32, 256, 0, ST>>>(scratch, (float*)dw, blocks, cols, accumulate_dw);
    if (db) partial_rows_sum_kernel<float><<<(cols + 31) / 32, 256, 0, ST>>>(part_db, (float*)db, blocks, cols, accumulate_dw);
  } else {
    if (dw) partial_rows_sum_kernel<__nv_bfloat16><<<(cols + 31) / 32, 256, 0, ST>>>(scratch, (__nv_bfloat16*)dw, blocks, cols, accumulate_dw);
    if (db) partial_rows_sum_kernel<__nv_bfloat16><<<(cols + 31) / 32, 256, 0, ST>>>(part_db, (__nv_bfloat16*)db, blocks, cols, accumulate_dw);
  }
  return CHECK_LAUNCH();
}
