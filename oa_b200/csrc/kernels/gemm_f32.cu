// Exact-fp32 SIMT GEMM with arbitrary element strides, a batch dimension and the bias / activation
// epilogues.  It backs the engine's FP32 precision mode (the reference's only fully exercised
// precision) and the finite-difference gradient checks, where TF32/bf16 rounding is not acceptable.
// The bf16 path uses gemm_tcgen05.cu instead.
//   C[b][m,n] = act(alpha * sum_k A[b][m*sam + k*sak] * B[b][n*sbn + k*sbk] + bias[n]) (+ C)
// 64x64x16 tiles, 256 threads, 4x4 outputs per thread: the same tiling class as the reference's
// GemmTiled (Source/Private/Oa/Core/Shader/Compute/Blas/Gemm/GemmTiled.slang:1-110), here with
// runtime strides so that NT / NN / TN products and Bmm need no transposed copies.
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr int FT = 64, FK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                long long sam, long long sak, long long sbn, long long sbk, int ldc, long long batch_a,
                long long batch_b, long long batch_c, const float* __restrict__ bias, int act, int accumulate,
                float alpha) {
  __shared__ float sA[FK][FT + 1];
  __shared__ float sB[FK][FT + 1];
  const int b = blockIdx.z;
  A += (long long)b * batch_a;
  B += (long long)b * batch_b;
  C += (long long)b * batch_c;
  const int m0 = blockIdx.y * FT, n0 = blockIdx.x * FT;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += FK) {
    // 64x16 elements per operand, 256 threads -> 4 loads each
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int idx = threadIdx.x + i * 256;
      int r, kk;
      // choose the faster-varying index to follow the contiguous dimension of each operand
      if (sak == 1) { kk = idx & 15; r = idx >> 4; } else { r = idx & 63; kk = idx >> 6; }
      int gm = m0 + r, gk = k0 + kk;
      sA[kk][r] = (gm < M && gk < K) ? A[gm * sam + gk * sak] : 0.f;
      if (sbk == 1) { kk = idx & 15; r = idx >> 4; } else { r = idx & 63; kk = idx >> 6; }
      int gn = n0 + r;
      gk = k0 + kk;
      sB[kk][r] = (gn < N && gk < K) ? B[gn * sbn + gk * sbk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < FK; ++kk) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sA[kk][ty * 4 + i]; bb[i] = sB[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j] * alpha;
      if (bias) v += bias[gn];
      if (act == OA_ACT_GELU) v = gelu_tanh(v);
      else if (act == OA_ACT_RELU) v = fmaxf(v, 0.f);
      else if (act == OA_ACT_SILU) v = silu_f(v);
      float* c = C + (long long)gm * ldc + gn;
      if (accumulate) v += *c;
      *c = v;
    }
  }
}

}  // namespace oa

extern "C" int oa_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, long long sam, long long sak,
                           long long sbn, long long sbk, int ldc, int batch, long long batch_a, long long batch_b,
                           long long batch_c, const float* bias, int act, int accumulate, float alpha, void* stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return OA_OK;
  if (K < 0 || batch > 65535) return OA_ERR_ARG;
  dim3 grid((N + oa::FT - 1) / oa::FT, (M + oa::FT - 1) / oa::FT, batch);
  oa::gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, B, C, M, N, K, sam, sak, sbn, sbk, ldc, batch_a, batch_b,
                                                              batch_c, bias, act, accumulate, alpha);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
