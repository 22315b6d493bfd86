// Block quantisation kernels (llama.cpp-compatible layouts): Q4_0 with separate per-block scales, Q8_0 blocks
// (fp16 scale + 32 int8 = 34 bytes) and per-tensor int8.  Contract: Source/Private/Oa/Ml/Shader/Compute/Quantize/
// {ComputeScaleQ4_0,QuantizeQ4_0,DequantizeQ4_0,QuantizeQ8_0,DequantizeQ8_0,QuantizeInt8,DequantizeInt8}.slang.
// One warp owns one 32-element block: the block maximum is a shuffle reduction and nibble pairs are packed with one
// shuffle, so every byte is written exactly once (no read-modify-write of the packed buffer).
#include <cuda_fp16.h>

#include "common.cuh"
#include "api.h"

namespace oa {

// scale[b] = max|x| / 7 over the block (1 when the block is ~zero)
__global__ void q4_0_scale_kernel(const float* __restrict__ x, float* __restrict__ scale, long long count) {
  const long long b = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b * 32 >= count) return;
  const long long i = b * 32 + lane;
  const float m = warp_max(i < count ? fabsf(x[i]) : 0.f);
  if (lane == 0) { float s = m / 7.0f; scale[b] = s < 1e-6f ? 1.0f : s; }
}

// q = clamp(round(x / scale), -7, 7) + 7; even lanes take the low nibble, odd lanes the high nibble of byte lane / 2
__global__ void q4_0_quantize_kernel(const float* __restrict__ x, const float* __restrict__ scale, unsigned char* __restrict__ out,
                                     long long count) {
  const long long b = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b * 32 >= count) return;
  const long long i = b * 32 + lane;
  int q = 7;
  if (i < count) q = min(max(__float2int_rn(x[i] / scale[b]), -7), 7) + 7;
  const int hi = __shfl_down_sync(0xffffffffu, q, 1);
  if ((lane & 1) == 0) out[b * 16 + (lane >> 1)] = (unsigned char)(q | (hi << 4));
}

__global__ void q4_0_dequantize_kernel(const unsigned char* __restrict__ in, const float* __restrict__ scale, float* __restrict__ out,
                                       long long count) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const long long b = i >> 5;
  const int lane = (int)(i & 31);
  const unsigned p = in[b * 16 + (lane >> 1)];
  const int q = (int)((lane & 1) ? (p >> 4) & 0xF : p & 0xF) - 7;
  out[i] = (float)q * scale[b];
}

// Q8_0 block: fp16 d = max|x| / 127, then 32 int8 q = clamp(round(x / d), -127, 127)
__global__ void q8_0_quantize_kernel(const float* __restrict__ x, unsigned char* __restrict__ out, long long blocks) {
  const long long b = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (b >= blocks) return;
  const float v = x[b * 32 + lane];
  const float d = warp_max(fabsf(v)) / 127.0f;
  const float id = d != 0.f ? 1.0f / d : 0.f;
  unsigned char* o = out + b * 34;
  if (lane == 0) { const __half h = __float2half_rn(d); *reinterpret_cast<unsigned short*>(o) = __half_as_ushort(h); }
  o[2 + lane] = (unsigned char)(signed char)min(max(__float2int_rn(v * id), -127), 127);
}

__global__ void q8_0_dequantize_kernel(const unsigned char* __restrict__ in, float* __restrict__ out, long long blocks) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= blocks * 32) return;
  const unsigned char* p = in + (i >> 5) * 34;
  const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(p)));
  out[i] = d * (float)(signed char)p[2 + (i & 31)];
}

// per-tensor int8: the scale is one device-resident float
__global__ void int8_quantize_kernel(const float* __restrict__ x, const float* __restrict__ scale, signed char* __restrict__ out,
                                     long long count) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = (signed char)min(max(__float2int_rn(x[i] / scale[0]), -127), 127);
}

__global__ void int8_dequantize_kernel(const signed char* __restrict__ in, const float* __restrict__ scale, float* __restrict__ out,
                                       long long count) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = (float)in[i] * scale[0];
}

}  // namespace oa

using namespace oa;

extern "C" {

// op: 0 Q4_0 scales, 1 Q4_0 quantize, 2 Q4_0 dequantize, 3 Q8_0 quantize, 4 Q8_0 dequantize, 5 int8 quantize,
// 6 int8 dequantize.  `count` is the number of fp32 elements (a multiple of 32 for Q8_0).
int oa_quantize(int op, const void* in, const void* scale, void* out, long long count, void* stream) {
  if (count <= 0) return OA_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const long long blocks = (count + 31) / 32;
  const int wg = (int)((blocks + 7) / 8), eg = (int)((count + 255) / 256);
  switch (op) {
    case 0: q4_0_scale_kernel<<<wg, 256, 0, s>>>((const float*)in, (float*)out, count); break;
    case 1: q4_0_quantize_kernel<<<wg, 256, 0, s>>>((const float*)in, (const float*)scale, (unsigned char*)out, count); break;
    case 2: q4_0_dequantize_kernel<<<eg, 256, 0, s>>>((const unsigned char*)in, (const float*)scale, (float*)out, count); break;
    case 3: if (count % 32) return OA_ERR_ARG; q8_0_quantize_kernel<<<wg, 256, 0, s>>>((const float*)in, (unsigned char*)out, blocks); break;
    case 4: if (count % 32) return OA_ERR_ARG; q8_0_dequantize_kernel<<<eg, 256, 0, s>>>((const unsigned char*)in, (float*)out, blocks); break;
    case 5: int8_quantize_kernel<<<eg, 256, 0, s>>>((const float*)in, (const float*)scale, (signed char*)out, count); break;
    case 6: int8_dequantize_kernel<<<eg, 256, 0, s>>>((const signed char*)in, (const float*)scale, (float*)out, count); break;
    default: return OA_ERR_ARG;
  }
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

}  // extern "C"
