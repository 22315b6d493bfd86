// Causal depthwise convolution + SiLU over a column range of the projected rows of a Mamba block, in place, and the
// learned-decay fill of the dd_A columns.  These are the options of the benchmark's Mamba-3 configuration (convolution
// width 4 before the scan, A = -exp(A_log)); the reference's mixer has neither (Source/Private/Oa/Ml/Nn/Mamba3/Mamba3.cpp).
//
//   forward   y[t, c] = silu(sum_k w[k, c] * x[t - k, c])   (x = 0 before the start of the sequence), written over x
//   backward  g[t, c] = dy[t, c] * silu'(pre[t, c]) with pre recomputed from the saved x;
//             dx[t, c] = sum_k w[k, c] * g[t + k, c];  dw[k, c] = sum_t g[t, c] * x[t - k, c]
// One thread owns one column and walks a block of TB tokens with the last K-1 inputs in registers, so global memory is read
// in whole rows; weight-gradient partials are written per token block and reduced in a fixed order by the caller.
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr int MC_TB = 64;      // tokens per block
constexpr int MC_MAXK = 8;

template <typename T> __device__ __forceinline__ float mc_ld(const T* p);
template <> __device__ __forceinline__ float mc_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float mc_ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void mc_st(T* p, float v);
template <> __device__ __forceinline__ void mc_st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void mc_st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// grid (ceil(C / 128), B * ceil(L / TB)); x: [B*L, ld] column range [col0, col0 + C); saved: [B*L, C] copy of the inputs
template <typename T>
__global__ void __launch_bounds__(128)
mamba3_conv_fwd_kernel(T* __restrict__ x, long long ld, int col0, T* __restrict__ saved, const float* __restrict__ w, int B, int L, int C,
                       int Kw) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= C) return;
  const int nb = (L + MC_TB - 1) / MC_TB;
  const int b = blockIdx.y / nb, t0 = (blockIdx.y % nb) * MC_TB;
  float wk[MC_MAXK], win[MC_MAXK];
#pragma unroll
  for (int k = 0; k < MC_MAXK; ++k) {
    wk[k] = k < Kw ? w[(long long)k * C + c] : 0.f;
    const int t = t0 - 1 - k;                    // win[k] = x[t0 - 1 - k]
    win[k] = (k < Kw - 1 && t >= 0) ? mc_ld(saved + ((long long)b * L + t) * C + c) : 0.f;
  }
  // Inputs (also the halo, which another block overwrites) are read from `saved`, the copy made by the launch before this one.
  const int t1 = min(L, t0 + MC_TB);
  for (int t = t0; t < t1; ++t) {
    const long long row = (long long)b * L + t;
    const float xt = mc_ld(saved + row * C + c);
    float acc = wk[0] * xt;
#pragma unroll
    for (int k = 1; k < MC_MAXK; ++k) acc = fmaf(wk[k], win[k - 1], acc);
#pragma unroll
    for (int k = MC_MAXK - 1; k > 0; --k) win[k] = win[k - 1];
    win[0] = xt;
    mc_st(x + row * ld + col0 + c, silu_f(acc));
  }
}

template <typename T>
__global__ void mamba3_cols_copy_kernel(const T* __restrict__ x, long long ld, int col0, T* __restrict__ out, long long rows, int C) {
  const long long total = rows * C;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
    out[i] = x[(i / C) * ld + col0 + (i % C)];
}

// dy: [B*L, ld] column range (gradient of the convolved columns), overwritten by dx; saved: the forward inputs;
// dw_part: float[B * nb][Kw][C]
template <typename T>
__global__ void __launch_bounds__(128)
mamba3_conv_bwd_kernel(T* __restrict__ dy, long long ld, int col0, const T* __restrict__ saved, const float* __restrict__ w,
                       float* __restrict__ dw_part, T* __restrict__ gbuf, int B, int L, int C, int Kw) {
  // pass A (gbuf != null, dy read-only): g = dy * silu'(pre) -> gbuf [B*L, C];   pass B (gbuf read-only): dx and dw from g
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= C) return;
  const int nb = (L + MC_TB - 1) / MC_TB;
  const int b = blockIdx.y / nb, t0 = (blockIdx.y % nb) * MC_TB;
  const int t1 = min(L, t0 + MC_TB);
  float wk[MC_MAXK];
#pragma unroll
  for (int k = 0; k < MC_MAXK; ++k) wk[k] = k < Kw ? w[(long long)k * C + c] : 0.f;
  if (dw_part == nullptr) {
    float win[MC_MAXK];
#pragma unroll
    for (int k = 0; k < MC_MAXK; ++k) {
      const int t = t0 - 1 - k;
      win[k] = (k < Kw - 1 && t >= 0) ? mc_ld(saved + ((long long)b * L + t) * C + c) : 0.f;
    }
    for (int t = t0; t < t1; ++t) {
      const long long row = (long long)b * L + t;
      const float xt = mc_ld(saved + row * C + c);
      float pre = wk[0] * xt;
#pragma unroll
      for (int k = 1; k < MC_MAXK; ++k) pre = fmaf(wk[k], win[k - 1], pre);
#pragma unroll
      for (int k = MC_MAXK - 1; k > 0; --k) win[k] = win[k - 1];
      win[0] = xt;
      const float sg = sigmoid_f(pre);
      mc_st(gbuf + row * C + c, mc_ld(dy + row * ld + col0 + c) * sg * (1.f + pre * (1.f - sg)));
    }
    return;
  }
  // pass B: dx[t] = sum_k w[k] g[t + k];  dw[k] += g[t] x[t - k]
  float dwk[MC_MAXK];
#pragma unroll
  for (int k = 0; k < MC_MAXK; ++k) dwk[k] = 0.f;
  for (int t = t0; t < t1; ++t) {
    const long long row = (long long)b * L + t;
    float dx = 0.f;
    const float gt = mc_ld(gbuf + row * C + c);
#pragma unroll
    for (int k = 0; k < MC_MAXK; ++k) {
      if (k < Kw) {
        if (t + k < L) dx = fmaf(wk[k], mc_ld(gbuf + (row + k) * C + c), dx);
        if (t - k >= 0) dwk[k] = fmaf(gt, mc_ld(saved + (row - k) * C + c), dwk[k]);
      }
    }
    mc_st(dy + row * ld + col0 + c, dx);
  }
  for (int k = 0; k < Kw; ++k) dw_part[((long long)blockIdx.y * Kw + k) * C + c] = dwk[k];
}

// x[row, col0 + h] = exp(a_log[h]) - 1
template <typename T>
__global__ void mamba3_alog_fill_kernel(T* __restrict__ x, long long ld, int col0, const float* __restrict__ a_log, long long rows, int H) {
  const long long total = rows * H;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int h = (int)(i % H);
    mc_st(x + (i / H) * ld + col0 + h, __expf(a_log[h]) - 1.f);
  }
}

static inline int mc_grid(long long n) {
  long long b = (n + 255) / 256;
  if (b > 148 * 8) b = 148 * 8;
  return (int)(b < 1 ? 1 : b);
}

}  // namespace oa

using namespace oa;
#define ST ((cudaStream_t)stream)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH)

extern "C" int oa_mamba3_conv_fwd(int dtype, void* x, long long ld, int col0, void* saved, const float* w, int B, int L, int C,
                                  int Kw, void* stream) {
  if (Kw < 1 || Kw > MC_MAXK || B <= 0 || L <= 0 || C <= 0) return OA_ERR_ARG;
  const long long rows = (long long)B * L;
  dim3 grid((C + 127) / 128, B * ((L + MC_TB - 1) / MC_TB));
  if (dtype == OA_F32) {
    mamba3_cols_copy_kernel<float><<<mc_grid(rows * C), 256, 0, ST>>>((const float*)x, ld, col0, (float*)saved, rows, C);
    mamba3_conv_fwd_kernel<float><<<grid, 128, 0, ST>>>((float*)x, ld, col0, (float*)saved, w, B, L, C, Kw);
  } else if (dtype == OA_BF16) {
    mamba3_cols_copy_kernel<__nv_bfloat16><<<mc_grid(rows * C), 256, 0, ST>>>((const __nv_bfloat16*)x, ld, col0, (__nv_bfloat16*)saved, rows, C);
    mamba3_conv_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, ST>>>((__nv_bfloat16*)x, ld, col0, (__nv_bfloat16*)saved, w, B, L, C, Kw);
  } else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}

// gbuf: [B*L, C] scratch of the data type; dw_part: float[B * ceil(L / 64) * Kw * C] (reduce over its first axis afterwards)
extern "C" int oa_mamba3_conv_bwd(int dtype, void* dy, long long ld, int col0, const void* saved, const float* w, float* dw_part,
                                  void* gbuf, int B, int L, int C, int Kw, void* stream) {
  if (Kw < 1 || Kw > MC_MAXK || B <= 0 || L <= 0 || C <= 0) return OA_ERR_ARG;
  dim3 grid((C + 127) / 128, B * ((L + MC_TB - 1) / MC_TB));
  if (dtype == OA_F32) {
    mamba3_conv_bwd_kernel<float><<<grid, 128, 0, ST>>>((float*)dy, ld, col0, (const float*)saved, w, nullptr, (float*)gbuf, B, L, C, Kw);
    mamba3_conv_bwd_kernel<float><<<grid, 128, 0, ST>>>((float*)dy, ld, col0, (const float*)saved, w, dw_part, (float*)gbuf, B, L, C, Kw);
  } else if (dtype == OA_BF16) {
    mamba3_conv_bwd_kernel<__nv_bfloat16><<<grid, 128, 0, ST>>>((__nv_bfloat16*)dy, ld, col0, (const __nv_bfloat16*)saved, w, nullptr,
                                                                (__nv_bfloat16*)gbuf, B, L, C, Kw);
    mamba3_conv_bwd_kernel<__nv_bfloat16><<<grid, 128, 0, ST>>>((__nv_bfloat16*)dy, ld, col0, (const __nv_bfloat16*)saved, w, dw_part,
                                                                (__nv_bfloat16*)gbuf, B, L, C, Kw);
  } else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}

extern "C" int oa_mamba3_alog_fill(int dtype, void* x, long long ld, int col0, const float* a_log, long long rows, int H, void* stream) {
  if (rows <= 0 || H <= 0) return OA_OK;
  if (dtype == OA_F32) mamba3_alog_fill_kernel<float><<<mc_grid(rows * H), 256, 0, ST>>>((float*)x, ld, col0, a_log, rows, H);
  else if (dtype == OA_BF16) mamba3_alog_fill_kernel<__nv_bfloat16><<<mc_grid(rows * H), 256, 0, ST>>>((__nv_bfloat16*)x, ld, col0, a_log, rows, H);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}
