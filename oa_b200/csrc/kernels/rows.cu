// Row compaction / scatter with a device-resident row count, accuracy counters, stochastic rounding to bf16 and the
// int8 matrix product.
//
// Contracts (reference kernels): Ml/Shader/Compute/Ops/CompactRows*.slang and ScatterRows*.slang (the reference writes
// indirect-dispatch arguments on the GPU; here the consumers read the row count from device memory and size their loop
// by it, so no host round trip is needed either), Flat/ScatterAddRows, Nn/Reduction/CategoricalAccuracyCount and
// MaskedCategoricalAccuracyCount, Sr/SrRoundBf16.slang, Quantize/GemmInt8.slang.
#include "common.cuh"
#include "api.h"

namespace oa {

template <typename T> __device__ __forceinline__ T zero_of() { return T(0); }
template <> __device__ __forceinline__ uint4 zero_of<uint4>() { return make_uint4(0u, 0u, 0u, 0u); }
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

// Exclusive prefix sum of a 0/1 mask: position[r] = number of selected rows before r, count[0] = total.  Three launches
// without any wait between blocks: (1) every block counts its 16,384 rows, (2) one block turns the block counts into
// block offsets, (3) every block scans its own rows and adds its offset.  The order is stable and the result does not
// depend on the launch shape.
constexpr int SCAN_PER_THREAD = 16;
constexpr int SCAN_BLOCK_ROWS = 1024 * SCAN_PER_THREAD;

__device__ __forceinline__ unsigned scan_flags(const unsigned char* __restrict__ mask, int r0, int rows) {
  unsigned flags = 0;                                  // bit i = row r0 + i is selected
#pragma unroll
  for (int i = 0; i < SCAN_PER_THREAD; ++i)
    if (r0 + i < rows && mask[r0 + i] != 0) flags |= 1u << i;
  return flags;
}

// Inclusive sum over the 1024 threads of a block; every thread gets its own inclusive value, *total the block's sum.
__device__ __forceinline__ int block_inclusive_scan(int mine, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int s = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += up;
    }
    warp_sums[lane] = s;
  }
  __syncthreads();
  const int out = incl + (warp > 0 ? warp_sums[warp - 1] : 0);
  *total = warp_sums[31];
  __syncthreads();                                      // warp_sums may be reused by the caller's next round
  return out;
}

__global__ void __launch_bounds__(1024)
rows_block_count_kernel(const unsigned char* __restrict__ mask, int* __restrict__ block_counts, int rows) {
  __shared__ int warp_sums[32];
  const int r0 = blockIdx.x * SCAN_BLOCK_ROWS + threadIdx.x * SCAN_PER_THREAD;
  int total;
  block_inclusive_scan(__popc(scan_flags(mask, r0, rows)), warp_sums, &total);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = total;
}

__global__ void __launch_bounds__(1024)
rows_block_offsets_kernel(const int* __restrict__ block_counts, int* __restrict__ block_offsets, int* __restrict__ count, int nblocks) {
  __shared__ int warp_sums[32];
  int carry = 0;                                        // identical in every thread
  for (int base = 0; base < nblocks; base += 1024) {
    const int b = base + threadIdx.x;
    const int mine = b < nblocks ? block_counts[b] : 0;
    int total;
    const int incl = block_inclusive_scan(mine, warp_sums, &total);
    if (b < nblocks) block_offsets[b] = carry + incl - mine;
    carry += total;
  }
  if (threadIdx.x == 0) count[0] = carry;
}

__global__ void __launch_bounds__(1024)
rows_block_positions_kernel(const unsigned char* __restrict__ mask, const int* __restrict__ block_offsets, int* __restrict__ position, int rows) {
  __shared__ int warp_sums[32];
  const int r0 = blockIdx.x * SCAN_BLOCK_ROWS + threadIdx.x * SCAN_PER_THREAD;
  const unsigned flags = scan_flags(mask, r0, rows);
  const int mine = __popc(flags);
  int total;
  const int before = block_offsets[blockIdx.x] + block_inclusive_scan(mine, warp_sums, &total) - mine;
#pragma unroll
  for (int i = 0; i < SCAN_PER_THREAD; ++i)
    if (r0 + i < rows) position[r0 + i] = before + __popc(flags & ((1u << i) - 1u));
}

// packed[position[r], :] = x[r, :] and index[position[r]] = r for every selected row r.
template <typename T>
__global__ void rows_compact_kernel(const T* __restrict__ x, const unsigned char* __restrict__ mask, const int* __restrict__ position,
                                    T* __restrict__ packed, int* __restrict__ index, int rows, int width) {
  const long long total = (long long)rows * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i - (long long)r * width);
    if (mask[r] == 0) continue;
    const int p = position[r];
    packed[(long long)p * width + c] = x[i];
    if (c == 0) index[p] = r;
  }
}

// out[index[i], :] (=|+=) packed[i, :] for i < count[0]; rows of `out` that no index names keep their value.
template <typename T, bool ADD>
__global__ void rows_scatter_kernel(const T* __restrict__ packed, const int* __restrict__ index, const int* __restrict__ count,
                                    T* __restrict__ out, int capacity, int out_rows, int width) {
  const int n = min(count[0], capacity);
  const long long total = (long long)n * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i / width), c = (int)(i - (long long)p * width);
    const int r = index[p];
    if (r < 0 || r >= out_rows) continue;
    if constexpr (ADD) atomicAdd(&out[(long long)r * width + c], packed[i]);
    else out[(long long)r * width + c] = packed[i];
  }
}

// packed[i, :] = src[index[i], :] for i < count[0], zero for the remaining rows of the fixed-capacity output.
template <typename T>
__global__ void rows_gather_kernel(const T* __restrict__ src, const int* __restrict__ index, const int* __restrict__ count, T* __restrict__ packed,
                                   int capacity, int src_rows, int width) {
  const int n = min(count[0], capacity);
  const long long total = (long long)capacity * width;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i / width), c = (int)(i - (long long)p * width);
    T v = zero_of<T>();
    if (p < n) {
      const int r = index[p];
      if (r >= 0 && r < src_rows) v = src[(long long)r * width + c];
    }
    packed[i] = v;
  }
}

// One warp per row: arg-max over the row (lowest index on ties), compared with the target.  out[0] += correct rows,
// out[1] += rows considered (mask == nullptr: every row).  Integer atomics: the result does not depend on the order.
template <typename T>
__global__ void accuracy_count_kernel(const T* __restrict__ logits, const int* __restrict__ targets, const unsigned char* __restrict__ mask,
                                      int* __restrict__ out, int rows, int vocab) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  int correct = 0, considered = 0;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    if (mask != nullptr && mask[r] == 0) continue;
    const T* row = logits + (long long)r * vocab;
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int c = lane; c < vocab; c += 32) {
      const float v = to_float(row[c]);
      if (v > best || (v == best && c < arg)) { best = v; arg = c; }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, d);
      const int oa_ = __shfl_xor_sync(0xffffffffu, arg, d);
      if (ob > best || (ob == best && oa_ < arg)) { best = ob; arg = oa_; }
    }
    if (lane == 0) { considered += 1; correct += arg == targets[r] ? 1 : 0; }
  }
  if (lane == 0 && considered > 0) { atomicAdd(&out[0], correct); atomicAdd(&out[1], considered); }
}

__device__ __forceinline__ unsigned sr_mix32(unsigned v) {
  v ^= v >> 16; v *= 0x7feb352du; v ^= v >> 15; v *= 0x846ca68bu; v ^= v >> 16;
  return v;
}

// fp32 -> bf16 with stochastic rounding: add 16 uniform random bits below the kept mantissa, then truncate.  The
// expectation of the result equals the input; infinities and NaNs are truncated unchanged.
__global__ void sr_round_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long n, unsigned seed_lo, unsigned seed_hi) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    unsigned bits = __float_as_uint(x[i]);
    if ((bits & 0x7f800000u) != 0x7f800000u) {
      const unsigned r = sr_mix32(seed_lo ^ sr_mix32(seed_hi + (unsigned)i * 0x9e3779b9u + (unsigned)(i >> 32))) & 0xffffu;
      bits += r;
    }
    out[i] = __ushort_as_bfloat16((unsigned short)(bits >> 16));
  }
}

// C[m, n] = sum_k A[m, k] * B[n, k] over int8 with int32 accumulation (4 products per instruction when K is a
// multiple of 4 and the rows are 4-byte aligned); optional fp32 output scaled by row_scale[m] * col_scale[n].
__global__ void __launch_bounds__(256)
gemm_int8_kernel(const signed char* __restrict__ a, const signed char* __restrict__ b, int* __restrict__ c_i32, float* __restrict__ c_f32,
                 const float* __restrict__ row_scale, const float* __restrict__ col_scale, int M, int N, int K, int vec) {
  const int n = blockIdx.x * 16 + (threadIdx.x & 15), m = blockIdx.y * 16 + (threadIdx.x >> 4);
  if (m >= M || n >= N) return;
  const signed char* ar = a + (long long)m * K;
  const signed char* br = b + (long long)n * K;
  int acc = 0, k = 0;
  if (vec) {
    const int* a4 = reinterpret_cast<const int*>(ar);
    const int* b4 = reinterpret_cast<const int*>(br);
    for (; k + 4 <= K; k += 4) acc = __dp4a(a4[k >> 2], b4[k >> 2], acc);
  }
  for (; k < K; ++k) acc += (int)ar[k] * (int)br[k];
  if (c_i32 != nullptr) c_i32[(long long)m * N + n] = acc;
  if (c_f32 != nullptr) c_f32[(long long)m * N + n] = (float)acc * (row_scale ? row_scale[m] : 1.f) * (col_scale ? col_scale[n] : 1.f);
}

// Rows whose byte width is a multiple of 16 (and whose buffers are 16-byte aligned) move as 16-byte vectors.
static inline bool rows_vectorisable(const void* a, const void* b, int width, int elem_bytes) {
  return ((long long)width * elem_bytes) % 16 == 0 && (((uintptr_t)a | (uintptr_t)b) & 15) == 0;
}

static inline int rows_grid(long long n) {
  long long g = (n + 255) / 256;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

extern "C" {

size_t oa_rows_scan_scratch_ints(int rows) { return 2 * (size_t)((rows + SCAN_BLOCK_ROWS - 1) / SCAN_BLOCK_ROWS) + 2; }

// scratch: oa_rows_scan_scratch_ints(rows) int32 values of device memory
int oa_rows_scan(const void* mask, void* position, void* count, void* scratch, int rows, void* stream) {
  if (rows < 0) return OA_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int nblocks = (rows + SCAN_BLOCK_ROWS - 1) / SCAN_BLOCK_ROWS;
  int* block_counts = (int*)scratch;
  int* block_offsets = block_counts + nblocks + 1;
  if (nblocks > 0) rows_block_count_kernel<<<nblocks, 1024, 0, s>>>((const unsigned char*)mask, block_counts, rows);
  rows_block_offsets_kernel<<<1, 1024, 0, s>>>(block_counts, block_offsets, (int*)count, nblocks);
  if (nblocks > 0) rows_block_positions_kernel<<<nblocks, 1024, 0, s>>>((const unsigned char*)mask, block_offsets, (int*)position, rows);
  return (int)cudaGetLastError();
}

// elem_bytes: 2 (bf16 / fp16) or 4 (fp32 / int32)
int oa_rows_compact(const void* x, const void* mask, const void* position, void* packed, void* index, int rows, int width, int elem_bytes,
                    void* stream) {
  if (rows <= 0 || width <= 0) return rows == 0 ? 0 : OA_ERR_ARG;
  if (rows_vectorisable(x, packed, width, elem_bytes)) {
    const int vecs = (int)((long long)width * elem_bytes / 16);
    rows_compact_kernel<uint4><<<rows_grid((long long)rows * vecs), 256, 0, (cudaStream_t)stream>>>(
        (const uint4*)x, (const unsigned char*)mask, (const int*)position, (uint4*)packed, (int*)index, rows, vecs);
    return (int)cudaGetLastError();
  }
  const int g = rows_grid((long long)rows * width);
  if (elem_bytes == 4)
    rows_compact_kernel<float><<<g, 256, 0, (cudaStream_t)stream>>>((const float*)x, (const unsigned char*)mask, (const int*)position, (float*)packed,
                                                                     (int*)index, rows, width);
  else if (elem_bytes == 2)
    rows_compact_kernel<unsigned short><<<g, 256, 0, (cudaStream_t)stream>>>((const unsigned short*)x, (const unsigned char*)mask, (const int*)position,
                                                                              (unsigned short*)packed, (int*)index, rows, width);
  else return OA_ERR_UNSUPPORTED;
  return (int)cudaGetLastError();
}

// dtype: OA_F32 or OA_BF16; add != 0 accumulates (atomic, so rows named twice sum in no fixed order)
int oa_rows_scatter(const void* packed, const void* index, const void* count, void* out, int capacity, int out_rows, int width, int dtype, int add,
                    void* stream) {
  if (capacity <= 0 || width <= 0) return capacity == 0 ? 0 : OA_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int eb = dtype == OA_F32 ? 4 : 2;
  if (!add && (dtype == OA_F32 || dtype == OA_BF16) && rows_vectorisable(packed, out, width, eb)) {
    const int vecs = (int)((long long)width * eb / 16);
    rows_scatter_kernel<uint4, false><<<rows_grid((long long)capacity * vecs), 256, 0, s>>>((const uint4*)packed, (const int*)index, (const int*)count,
                                                                                          (uint4*)out, capacity, out_rows, vecs);
    return (int)cudaGetLastError();
  }
  const int g = rows_grid((long long)capacity * width);
  if (dtype == OA_F32) {
    if (add) rows_scatter_kernel<float, true><<<g, 256, 0, s>>>((const float*)packed, (const int*)index, (const int*)count, (float*)out, capacity, out_rows, width);
    else rows_scatter_kernel<float, false><<<g, 256, 0, s>>>((const float*)packed, (const int*)index, (const int*)count, (float*)out, capacity, out_rows, width);
  } else if (dtype == OA_BF16) {
    if (add) rows_scatter_kernel<__nv_bfloat16, true><<<g, 256, 0, s>>>((const __nv_bfloat16*)packed, (const int*)index, (const int*)count,
                                                                          (__nv_bfloat16*)out, capacity, out_rows, width);
    else rows_scatter_kernel<__nv_bfloat16, false><<<g, 256, 0, s>>>((const __nv_bfloat16*)packed, (const int*)index, (const int*)count,
                                                                      (__nv_bfloat16*)out, capacity, out_rows, width);
  } else return OA_ERR_UNSUPPORTED;
  return (int)cudaGetLastError();
}

// elem_bytes: 2 or 4
int oa_rows_gather(const void* src, const void* index, const void* count, void* packed, int capacity, int src_rows, int width, int elem_bytes,
                   void* stream) {
  if (capacity <= 0 || width <= 0) return capacity == 0 ? 0 : OA_ERR_ARG;
  if (rows_vectorisable(src, packed, width, elem_bytes)) {
    const int vecs = (int)((long long)width * elem_bytes / 16);
    rows_gather_kernel<uint4><<<rows_grid((long long)capacity * vecs), 256, 0, (cudaStream_t)stream>>>(
        (const uint4*)src, (const int*)index, (const int*)count, (uint4*)packed, capacity, src_rows, vecs);
    return (int)cudaGetLastError();
  }
  const int g = rows_grid((long long)capacity * width);
  if (elem_bytes == 4)
    rows_gather_kernel<float><<<g, 256, 0, (cudaStream_t)stream>>>((const float*)src, (const int*)index, (const int*)count, (float*)packed, capacity,
                                                                    src_rows, width);
  else if (elem_bytes == 2)
    rows_gather_kernel<unsigned short><<<g, 256, 0, (cudaStream_t)stream>>>((const unsigned short*)src, (const int*)index, (const int*)count,
                                                                             (unsigned short*)packed, capacity, src_rows, width);
  else return OA_ERR_UNSUPPORTED;
  return (int)cudaGetLastError();
}

// out2 = {correct, considered} (int32, accumulated: zero it first); mask may be null
int oa_accuracy_count(const void* logits, const void* targets, const void* mask, void* out2, int rows, int vocab, int dtype, void* stream) {
  if (rows <= 0 || vocab <= 0) return rows == 0 ? 0 : OA_ERR_ARG;
  const int blocks = min((rows + 7) / 8, 148 * 8);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == OA_F32)
    accuracy_count_kernel<float><<<blocks, 256, 0, s>>>((const float*)logits, (const int*)targets, (const unsigned char*)mask, (int*)out2, rows, vocab);
  else if (dtype == OA_BF16)
    accuracy_count_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)logits, (const int*)targets, (const unsigned char*)mask, (int*)out2,
                                                                 rows, vocab);
  else return OA_ERR_UNSUPPORTED;
  return (int)cudaGetLastError();
}

int oa_sr_round_bf16(const void* x, void* out, long long n, unsigned seed_lo, unsigned seed_hi, void* stream) {
  if (n <= 0) return n == 0 ? 0 : OA_ERR_ARG;
  sr_round_bf16_kernel<<<rows_grid(n), 256, 0, (cudaStream_t)stream>>>((const float*)x, (__nv_bfloat16*)out, n, seed_lo, seed_hi);
  return (int)cudaGetLastError();
}

int oa_gemm_int8(const void* a, const void* b, void* c_i32, void* c_f32, const void* row_scale, const void* col_scale, int M, int N, int K,
                 void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return OA_ERR_ARG;
  const int vec = (K % 4 == 0) && (((uintptr_t)a | (uintptr_t)b) % 4 == 0);
  dim3 grid((N + 15) / 16, (M + 15) / 16);
  gemm_int8_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const signed char*)a, (const signed char*)b, (int*)c_i32, (float*)c_f32,
                                                           (const float*)row_scale, (const float*)col_scale, M, N, K, vec);
  return (int)cudaGetLastError();
}

}  // extern "C"

}  // namespace oa
