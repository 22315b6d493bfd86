// Whole-sequence GRU / RNN recurrent scans, forward and backward, one launch per layer.
//
// Contracts (Source/Private/Oa/Ml/Shader/Compute/Nn/Gru/GruScan.slang:8-15,73-86, Nn/Rnn/RnnScan.slang:8-12):
//   GRU:  r = sigmoid(i_r + h_r); z = sigmoid(i_z + h_z); n = tanh(i_n + r * h_n); h' = (1 - z) * n + z * h
//         with [h_r | h_z | h_n] = W_hh h + b_hh, gate order reset | update | candidate, h(0) = 0
//   RNN:  h' = tanh(i + W_hh h + b_hh)
// The input projection i = W_ih x + b_ih for all time steps is one GEMM done by the caller; only the serial part
// runs here.  The reference runs one work-group per batch element with h in shared memory; here a CTA owns a tile
// of BT batch rows so that every W_hh row fetched from L2 / shared memory is reused BT times, h and the gate
// pre-activations live in shared memory, math is fp32.  The backward pass walks time in reverse from the saved
// h(t-1), emits the gate gradients dGi (for the input projection) and dGh; the weight gradient
// dW_hh = dGh^T Hprev and db_hh are then ordinary (tensor-core) GEMM / column-sum calls.
#include "common.cuh"
#include "api.h"

namespace oa {

template <typename T> __device__ __forceinline__ float rld(const T* p);
template <> __device__ __forceinline__ float rld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float rld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void rst(T* p, float v);
template <> __device__ __forceinline__ void rst<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void rst<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int RNN_BT = 4;        // batch rows per CTA
constexpr int RNN_THREADS = 256;

// G = number of gates (3 = GRU, 1 = RNN).  Shared: h[BT][H], gh[BT][G*H].
template <typename T, int G>
__global__ void __launch_bounds__(RNN_THREADS)
rnn_scan_fwd_kernel(const T* __restrict__ gates_i, const T* __restrict__ w_hh, const T* __restrict__ b_hh, const T* __restrict__ h0,
                    T* __restrict__ out, T* __restrict__ hprev, int batch, int seq, int H) {
  extern __shared__ float sm[];
  float* sh = sm;                       // [BT][H]
  float* sg = sm + RNN_BT * H;          // [BT][G*H]
  const int b0 = blockIdx.x * RNN_BT;
  const int nb = min(RNN_BT, batch - b0);
  for (int i = threadIdx.x; i < RNN_BT * H; i += blockDim.x) {
    int bb = i / H, j = i % H;
    sh[i] = (h0 && bb < nb) ? rld<T>(h0 + (long long)(b0 + bb) * H + j) : 0.f;
  }
  __syncthreads();
  for (int t = 0; t < seq; ++t) {
    // recurrent projection: gh[b][j] = b_hh[j] + sum_k W_hh[j][k] * h[b][k]
    for (int j = threadIdx.x; j < G * H; j += blockDim.x) {
      float acc[RNN_BT];
      const float bj = b_hh ? rld<T>(b_hh + j) : 0.f;
#pragma unroll
      for (int bb = 0; bb < RNN_BT; ++bb) acc[bb] = bj;
      const T* wr = w_hh + (long long)j * H;
      for (int k = 0; k < H; ++k) {
        const float w = rld<T>(wr + k);
#pragma unroll
        for (int bb = 0; bb < RNN_BT; ++bb) acc[bb] = fmaf(w, sh[bb * H + k], acc[bb]);
      }
#pragma unroll
      for (int bb = 0; bb < RNN_BT; ++bb) sg[bb * G * H + j] = acc[bb];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nb * H; i += blockDim.x) {
      const int bb = i / H, j = i % H;
      const long long row = ((long long)(b0 + bb) * seq + t);
      const T* gi = gates_i + row * G * H;
      const float hp = sh[bb * H + j];
      float hn;
      if (G == 3) {
        const float r = sigmoid_f(rld<T>(gi + j) + sg[bb * 3 * H + j]);
        const float z = sigmoid_f(rld<T>(gi + H + j) + sg[bb * 3 * H + H + j]);
        const float n = tanhf(rld<T>(gi + 2 * H + j) + r * sg[bb * 3 * H + 2 * H + j]);
        hn = (1.f - z) * n + z * hp;
      } else {
        hn = tanhf(rld<T>(gi + j) + sg[bb * H + j]);
      }
      if (hprev) rst<T>(hprev + row * H + j, hp);
      rst<T>(out + row * H + j, hn);
      sh[bb * H + j] = hn;
    }
    __syncthreads();
  }
}

// Shared: h[BT][H] (saved h(t-1)), gh[BT][G*H], dh[BT][H] (running gradient), dgh[BT][G*H].
template <typename T, int G>
__global__ void __launch_bounds__(RNN_THREADS)
rnn_scan_bwd_kernel(const T* __restrict__ gates_i, const T* __restrict__ w_hh, const T* __restrict__ b_hh,
                    const T* __restrict__ hprev, const T* __restrict__ dout, T* __restrict__ dgi, T* __restrict__ dgh,
                    T* __restrict__ dh0, int batch, int seq, int H) {
  extern __shared__ float sm[];
  float* sh = sm;
  float* sg = sh + RNN_BT * H;
  float* sdh = sg + RNN_BT * G * H;
  float* sdg = sdh + RNN_BT * H;
  const int b0 = blockIdx.x * RNN_BT;
  const int nb = min(RNN_BT, batch - b0);
  for (int i = threadIdx.x; i < RNN_BT * H; i += blockDim.x) sdh[i] = 0.f;
  for (int i = threadIdx.x; i < RNN_BT * G * H; i += blockDim.x) sdg[i] = 0.f;
  __syncthreads();
  for (int t = seq - 1; t >= 0; --t) {
    for (int i = threadIdx.x; i < RNN_BT * H; i += blockDim.x) {
      int bb = i / H, j = i % H;
      sh[i] = bb < nb ? rld<T>(hprev + ((long long)(b0 + bb) * seq + t) * H + j) : 0.f;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < G * H; j += blockDim.x) {
      float acc[RNN_BT];
      const float bj = b_hh ? rld<T>(b_hh + j) : 0.f;
#pragma unroll
      for (int bb = 0; bb < RNN_BT; ++bb) acc[bb] = bj;
      const T* wr = w_hh + (long long)j * H;
      for (int k = 0; k < H; ++k) {
        const float w = rld<T>(wr + k);
#pragma unroll
        for (int bb = 0; bb < RNN_BT; ++bb) acc[bb] = fmaf(w, sh[bb * H + k], acc[bb]);
      }
#pragma unroll
      for (int bb = 0; bb < RNN_BT; ++bb) sg[bb * G * H + j] = acc[bb];
    }
    __syncthreads();
    // pointwise backward; dh_total = dout[t] + carried dh
    for (int i = threadIdx.x; i < nb * H; i += blockDim.x) {
      const int bb = i / H, j = i % H;
      const long long row = ((long long)(b0 + bb) * seq + t);
      const T* gi = gates_i + row * G * H;
      const float hp = sh[bb * H + j];
      const float d = rld<T>(dout + row * H + j) + sdh[bb * H + j];
      if (G == 3) {
        const float hr = sg[bb * 3 * H + j], hz = sg[bb * 3 * H + H + j], hn_ = sg[bb * 3 * H + 2 * H + j];
        const float r = sigmoid_f(rld<T>(gi + j) + hr);
        const float z = sigmoid_f(rld<T>(gi + H + j) + hz);
        const float n = tanhf(rld<T>(gi + 2 * H + j) + r * hn_);
        const float dn = d * (1.f - z);
        const float dz = d * (hp - n);
        const float dn_pre = dn * (1.f - n * n);
        const float dr = dn_pre * hn_;
        const float dr_pre = dr * r * (1.f - r);
        const float dz_pre = dz * z * (1.f - z);
        rst<T>(dgi + row * 3 * H + j, dr_pre);
        rst<T>(dgi + row * 3 * H + H + j, dz_pre);
        rst<T>(dgi + row * 3 * H + 2 * H + j, dn_pre);
        const float dhn = dn_pre * r;
        rst<T>(dgh + row * 3 * H + j, dr_pre);
        rst<T>(dgh + row * 3 * H + H + j, dz_pre);
        rst<T>(dgh + row * 3 * H + 2 * H + j, dhn);
        sdg[bb * 3 * H + j] = dr_pre; sdg[bb * 3 * H + H + j] = dz_pre; sdg[bb * 3 * H + 2 * H + j] = dhn;
        sdh[bb * H + j] = d * z;          // direct path h -> h'
      } else {
        const float hn = tanhf(rld<T>(gi + j) + sg[bb * H + j]);
        const float dpre = d * (1.f - hn * hn);
        rst<T>(dgi + row * H + j, dpre);
        rst<T>(dgh + row * H + j, dpre);
        sdg[bb * H + j] = dpre;
        sdh[bb * H + j] = 0.f;
      }
    }
    __syncthreads();
    // dh(t-1) += W_hh^T dgh
    for (int k = threadIdx.x; k < H; k += blockDim.x) {
      float acc[RNN_BT];
#pragma unroll
      for (int bb = 0; bb < RNN_BT; ++bb) acc[bb] = 0.f;
      for (int j = 0; j < G * H; ++j) {
        const float w = rld<T>(w_hh + (long long)j * H + k);
#pragma unroll
        for (int bb = 0; bb < RNN_BT; ++bb) acc[bb] = fmaf(w, sdg[bb * G * H + j], acc[bb]);
      }
#pragma unroll
      for (int bb = 0; bb < RNN_BT; ++bb) sdh[bb * H + k] += acc[bb];
    }
    __syncthreads();
  }
  if (dh0)
    for (int i = threadIdx.x; i < nb * H; i += blockDim.x) rst<T>(dh0 + (long long)(b0 + i / H) * H + i % H, sdh[(i / H) * H + i % H]);
}

template <typename K>
static int rnn_set_smem(K kernel, size_t bytes) {
  if (bytes > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) return OA_ERR_LAUNCH;
  return OA_OK;
}

}  // namespace oa

using namespace oa;
#define ST ((cudaStream_t)stream)

// gates = 3 (GRU) or 1 (RNN).  gates_i [B, S, gates*H], w_hh [gates*H, H], b_hh [gates*H] or null, h0 [B, H] or null,
// out [B, S, H], hprev [B, S, H] or null (needed for the backward pass).
extern "C" int oa_rnn_scan_fwd(int dtype, int gates, const void* gates_i, const void* w_hh, const void* b_hh, const void* h0,
                               void* out, void* hprev, int batch, int seq, int H, void* stream) {
  if (gates != 1 && gates != 3) return OA_ERR_ARG;
  if (batch <= 0 || seq <= 0) return OA_OK;
  size_t smem = (size_t)RNN_BT * H * (1 + gates) * sizeof(float);
  if (smem > 200 * 1024) return OA_ERR_TOO_LARGE;
  int blocks = (batch + RNN_BT - 1) / RNN_BT, rc;
#define LAUNCH_FWD(T, G)                                                                                         \
  {                                                                                                              \
    if ((rc = rnn_set_smem(rnn_scan_fwd_kernel<T, G>, smem))) return rc;                                         \
    rnn_scan_fwd_kernel<T, G><<<blocks, RNN_THREADS, smem, ST>>>((const T*)gates_i, (const T*)w_hh, (const T*)b_hh, \
                                                                 (const T*)h0, (T*)out, (T*)hprev, batch, seq, H); \
  }
  if (dtype == OA_F32) { if (gates == 3) LAUNCH_FWD(float, 3) else LAUNCH_FWD(float, 1) }
  else if (dtype == OA_BF16) { if (gates == 3) LAUNCH_FWD(__nv_bfloat16, 3) else LAUNCH_FWD(__nv_bfloat16, 1) }
  else return OA_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_rnn_scan_bwd(int dtype, int gates, const void* gates_i, const void* w_hh, const void* b_hh, const void* hprev,
                               const void* dout, void* dgi, void* dgh, void* dh0, int batch, int seq, int H, void* stream) {
  if (gates != 1 && gates != 3) return OA_ERR_ARG;
  if (batch <= 0 || seq <= 0) return OA_OK;
  size_t smem = (size_t)RNN_BT * H * (2 + 2 * gates) * sizeof(float);
  if (smem > 200 * 1024) return OA_ERR_TOO_LARGE;
  int blocks = (batch + RNN_BT - 1) / RNN_BT, rc;
#define LAUNCH_BWD(T, G)                                                                                           \
  {                                                                                                                \
    if ((rc = rnn_set_smem(rnn_scan_bwd_kernel<T, G>, smem))) return rc;                                           \
    rnn_scan_bwd_kernel<T, G><<<blocks, RNN_THREADS, smem, ST>>>((const T*)gates_i, (const T*)w_hh, (const T*)b_hh,   \
                                                                 (const T*)hprev, (const T*)dout, (T*)dgi, (T*)dgh,  \
                                                                 (T*)dh0, batch, seq, H);                           \
  }
  if (dtype == OA_F32) { if (gates == 3) LAUNCH_BWD(float, 3) else LAUNCH_BWD(float, 1) }
  else if (dtype == OA_BF16) { if (gates == 3) LAUNCH_BWD(__nv_bfloat16, 3) else LAUNCH_BWD(__nv_bfloat16, 1) }
  else return OA_ERR_UNSUPPORTED;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
