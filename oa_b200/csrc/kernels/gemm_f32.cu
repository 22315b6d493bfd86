// Exact-fp32 SIMT GEMM with arbitrary element strides, a batch dimension and the bias / activation
// epilogues.  It backs the engine's FP32 precision mode (the reference's only fully exercised
// precision) and the finite-difference gradient checks, where TF32/bf16 rounding is not acceptable.
// The bf16 path uses gemm_tcgen05.cu instead.
//   C[b][m,n] = act(alpha * sum_k A[b][m*sam + k*sak] * B[b][n*sbn + k*sbk] + bias[n]) (+ C)
// 64x64x16 tiles, 256 threads, 4x4 outputs per thread with 16-byte shared-memory reads and the next
// K tile prefetched into registers (the reference's GemmTiled,
// Source/Private/Oa/Core/Shader/Compute/Blas/Gemm/GemmTiled.slang:1-110, is the same tiling class), here
// with runtime strides so that NT / NN / TN products and Bmm need no transposed copies.
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr int FT = 64, FK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N, int K,
                long long sam, long long sak, long long sbn, long long sbk, int ldc, long long batch_a,
                long long batch_b, long long batch_c, const float* __restrict__ bias, int act, int accumulate,
                float alpha, int k_chunk) {
  __shared__ __align__(16) float sA[FK][FT + 4];
  __shared__ __align__(16) float sB[FK][FT + 4];
  const int b = blockIdx.z;
  // k_chunk > 0: split-K mode - blockIdx.z is the K slice (batch 1) and C is the slice's own [M, ldc] partial buffer
  const int k_lo = k_chunk > 0 ? b * k_chunk : 0;
  const int k_hi = k_chunk > 0 ? min(K, k_lo + k_chunk) : K;
  if (k_chunk > 0) {
    C += (long long)b * batch_c;
  } else {
    A += (long long)b * batch_a;
    B += (long long)b * batch_b;
    C += (long long)b * batch_c;
  }
  const int m0 = blockIdx.y * FT, n0 = blockIdx.x * FT;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  // 64x16 elements per operand, 256 threads -> 4 loads each; the faster-varying index follows the contiguous dimension
  int ar[4], ak[4], br[4], bk[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = threadIdx.x + i * 256;
    if (sak == 1) { ak[i] = idx & 15; ar[i] = idx >> 4; } else { ar[i] = idx & 63; ak[i] = idx >> 6; }
    if (sbk == 1) { bk[i] = idx & 15; br[i] = idx >> 4; } else { br[i] = idx & 63; bk[i] = idx >> 6; }
  }
  float ra[4], rb[4];
  auto fetch = [&](int k0) {       // global -> registers (the next tile is in flight while this one is multiplied)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gm = m0 + ar[i], gka = k0 + ak[i], gn = n0 + br[i], gkb = k0 + bk[i];
      ra[i] = (gm < M && gka < k_hi) ? A[gm * sam + gka * sak] : 0.f;
      rb[i] = (gn < N && gkb < k_hi) ? B[gn * sbn + gkb * sbk] : 0.f;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int i = 0; i < 4; ++i) { sA[ak[i]][ar[i]] = ra[i]; sB[bk[i]][br[i]] = rb[i]; }
  };
  float acc[4][4] = {};
  if (k_lo < k_hi) fetch(k_lo);
  for (int k0 = k_lo; k0 < k_hi; k0 += FK) {
    stash();
    __syncthreads();
    if (k0 + FK < k_hi) fetch(k0 + FK);
#pragma unroll
    for (int kk = 0; kk < FK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&sA[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&sB[kk][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w};
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

// C[m,n] = alpha * sum_s part[s][m,n] (+ C): fixed slice order, so the split-K result is reproducible
__global__ void gemm_f32_splitk_reduce_kernel(const float* __restrict__ part, float* __restrict__ C, int M, int N, int ldc, int splits,
                                              int accumulate, float alpha) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * N) return;
  const int m = (int)(i / N), n = (int)(i % N);
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += part[((long long)k * M + m) * N + n];
  float* c = C + (long long)m * ldc + n;
  *c = accumulate ? *c + s * alpha : s * alpha;
}

// Scratch for split-K partials: allocated outside stream capture only, sizes rounded up to a power of two, and an outgrown
// buffer is kept (a captured graph may still hold its address), so at most 64 + 32 + ... MB are ever held.
static float* g_splitk_buf = nullptr;
static size_t g_splitk_bytes = 0;

static float* splitk_scratch(size_t bytes, cudaStream_t st) {
  if (bytes <= g_splitk_bytes) return g_splitk_buf;
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return nullptr;
  if (bytes > (64u << 20)) return nullptr;
  size_t cap = 1u << 20;
  while (cap < bytes) cap <<= 1;
  float* p = nullptr;
  if (cudaMalloc(&p, cap) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  g_splitk_buf = p; g_splitk_bytes = cap;
  return p;
}

}  // namespace oa

extern "C" int oa_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, long long sam, long long sak,
                           long long sbn, long long sbk, int ldc, int batch, long long batch_a, long long batch_b,
                           long long batch_c, const float* bias, int act, int accumulate, float alpha, void* stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return OA_OK;
  if (K < 0 || batch > 65535) return OA_ERR_ARG;
  dim3 grid((N + oa::FT - 1) / oa::FT, (M + oa::FT - 1) / oa::FT, batch);
  cudaStream_t st = (cudaStream_t)stream;
  // Few output tiles and a long reduction (weight gradients of small models): slice K over more CTAs, then reduce the slices
  const int tiles = (int)(grid.x * grid.y);
  if (batch == 1 && !bias && act == OA_ACT_NONE && tiles < 64 && K >= 512) {
    int splits = (256 + tiles - 1) / tiles;
    if (splits > K / 128) splits = K / 128;
    if (splits > 64) splits = 64;
    if (splits >= 2) {
      const int k_chunk = (((K + splits - 1) / splits) + oa::FK - 1) / oa::FK * oa::FK;
      splits = (K + k_chunk - 1) / k_chunk;
      float* part = oa::splitk_scratch((size_t)splits * M * N * sizeof(float), st);
      if (part && splits >= 2) {
        grid.z = splits;
        oa::gemm_f32_kernel<<<grid, 256, 0, st>>>(A, B, part, M, N, K, sam, sak, sbn, sbk, N, 0, 0, (long long)M * N, nullptr,
                                                  OA_ACT_NONE, 0, 1.0f, k_chunk);
        const long long n = (long long)M * N;
        oa::gemm_f32_splitk_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(part, C, M, N, ldc, splits, accumulate, alpha);
        return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
      }
    }
  }
  oa::gemm_f32_kernel<<<grid, 256, 0, st>>>(A, B, C, M, N, K, sam, sak, sbn, sbk, ldc, batch_a, batch_b, batch_c, bias, act,
                                            accumulate, alpha, 0);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
