// Vector-quantisation kernels (VQ-VAE bottleneck): nearest-code assignment and the EMA codebook update with dead-code
// revival.  Contract: Source/Private/Oa/Ml/Shader/Compute/Ops/VqAssign.slang and VqEmaUpdate.slang of the reference.
// The assignment is GEMM-shaped: argmin_k |z - e_k|^2 = argmin_k (|e_k|^2 - 2 z.e_k), so the dot products come from the
// GEMM kernel and this file only does the per-row argmin + gather.  The EMA update is one CTA per code and adds the rows
// assigned to it in row order (no atomics: the result is bit-reproducible).
#include "common.cuh"
#include "api.h"

namespace oa {

// One warp per row: lanes stride over the codes, lowest index wins ties, then the warp copies the winning code.
__global__ void vq_argmin_gather_kernel(const float* __restrict__ dot, const float* __restrict__ enorm,
                                        const float* __restrict__ codebook, int* __restrict__ idx, float* __restrict__ zq, int N,
                                        int Kc, int D) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= N) return;
  float best = 3.402823466e+38f;
  int arg = 0x7fffffff;
  for (int k = lane; k < Kc; k += 32) {
    const float d = enorm[k] - 2.f * dot[(long long)row * Kc + k];
    if (d < best) { best = d; arg = k; }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa_ = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ob < best || (ob == best && oa_ < arg)) { best = ob; arg = oa_; }
  }
  if (arg == 0x7fffffff) arg = 0;                 // every distance was NaN / inf: fall back to code 0
  if (lane == 0) idx[row] = arg;
  for (int d = lane; d < D; d += 32) zq[(long long)row * D + d] = codebook[(long long)arg * D + d];
}

// |e_k|^2 per code
__global__ void vq_code_norm_kernel(const float* __restrict__ codebook, float* __restrict__ enorm, int Kc, int D) {
  const int k = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (k >= Kc) return;
  float s = 0.f;
  for (int d = lane; d < D; d += 32) { const float v = codebook[(long long)k * D + d]; s += v * v; }
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) enorm[k] = s;
}

// One CTA per code k.  N_k <- g N_k + (1-g) count; m_k <- g m_k + (1-g) sum of assigned rows; e_k = m_k / max(N_k, eps);
// optional rescale of e_k to unit RMS; codes with N_k < dead_thresh restart from the encoder row hash(k, seed) mod N.
__global__ void vq_ema_update_kernel(const float* __restrict__ ze, const int* __restrict__ idx, float* __restrict__ embed_sum,
                                     float* __restrict__ cluster_size, float* __restrict__ codebook, int N, int D, float decay,
                                     float eps, float dead_thresh, unsigned seed, int normalize) {
  const int k = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  __shared__ int s_match[256];
  __shared__ int s_cnt;
  __shared__ float s_red[32];
  extern __shared__ float s_sum[];                 // D running sums
  for (int d = tid; d < D; d += nt) s_sum[d] = 0.f;
  int count = 0;
  for (int base = 0; base < N; base += nt) {
    __syncthreads();
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    const int n = base + tid;
    const bool hit = n < N && idx[n] == k;
    // compact the matching rows of this tile in row order: ballot per warp + warp offsets
    const unsigned bal = __ballot_sync(0xffffffffu, hit);
    const int warp = tid >> 5, lane = tid & 31;
    if (lane == 0) s_red[warp] = __int_as_float(__popc(bal));
    __syncthreads();
    int off = 0;
    for (int w = 0; w < warp; ++w) off += __float_as_int(s_red[w]);
    if (hit) s_match[off + __popc(bal & ((1u << lane) - 1u))] = n;
    if (tid == nt - 1) s_cnt = off + __popc(bal);
    __syncthreads();
    const int m = s_cnt;
    count += m;
    for (int d = tid; d < D; d += nt) {
      float s = s_sum[d];
      for (int j = 0; j < m; ++j) s += ze[(long long)s_match[j] * D + d];
      s_sum[d] = s;
    }
  }
  __syncthreads();
  const float Nk = decay * cluster_size[k] + (1.f - decay) * (float)count;
  float sq = 0.f;
  for (int d = tid; d < D; d += nt) {
    const float mk = decay * embed_sum[(long long)k * D + d] + (1.f - decay) * s_sum[d];
    embed_sum[(long long)k * D + d] = mk;
    const float ek = mk / fmaxf(Nk, eps);
    s_sum[d] = ek;
    sq += ek * ek;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  __syncthreads();
  if ((tid & 31) == 0) s_red[tid >> 5] = sq;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < (nt >> 5); ++w) total += s_red[w];
  float inv = 1.f;
  if (normalize) {
    const float rms = sqrtf(total / (float)D);
    if (rms > eps) inv = 1.f / rms;
  }
  const bool dead = Nk < dead_thresh;
  unsigned h = ((unsigned)(k + 1) * 2654435761u) ^ (seed * 2246822519u) ^ (seed >> 15);
  h ^= h >> 13; h *= 3266489917u; h ^= h >> 16;
  const long long r = (long long)(h % (unsigned)N) * D;
  for (int d = tid; d < D; d += nt) {
    if (dead) {
      const float v = ze[r + d];
      codebook[(long long)k * D + d] = v;
      embed_sum[(long long)k * D + d] = v;
    } else {
      codebook[(long long)k * D + d] = s_sum[d] * inv;
    }
  }
  if (tid == 0) cluster_size[k] = dead ? 1.f : Nk;
}

}  // namespace oa

using namespace oa;

extern "C" {

int oa_vq_code_norm(const void* codebook, void* enorm, int K, int D, void* stream) {
  if (K <= 0 || D <= 0) return OA_ERR_ARG;
  vq_code_norm_kernel<<<(K + 7) / 8, 256, 0, (cudaStream_t)stream>>>((const float*)codebook, (float*)enorm, K, D);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

int oa_vq_argmin_gather(const void* dot, const void* enorm, const void* codebook, void* idx, void* zq, int N, int K, int D,
                        void* stream) {
  if (N <= 0 || K <= 0 || D <= 0) return OA_ERR_ARG;
  vq_argmin_gather_kernel<<<(N + 7) / 8, 256, 0, (cudaStream_t)stream>>>((const float*)dot, (const float*)enorm,
                                                                         (const float*)codebook, (int*)idx, (float*)zq, N, K, D);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

int oa_vq_ema_update(const void* ze, const void* idx, void* embed_sum, void* cluster_size, void* codebook, int N, int D, int K,
                     float decay, float eps, float dead_thresh, unsigned seed, int normalize, void* stream) {
  if (N <= 0 || K <= 0 || D <= 0 || D > 8192) return OA_ERR_ARG;
  vq_ema_update_kernel<<<K, 256, D * sizeof(float), (cudaStream_t)stream>>>((const float*)ze, (const int*)idx, (float*)embed_sum,
                                                                          (float*)cluster_size, (float*)codebook, N, D, decay, eps,
                                                                          dead_thresh, seed, normalize);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

}  // extern "C"
