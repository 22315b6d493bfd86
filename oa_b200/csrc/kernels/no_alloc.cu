// Allocation-free column sum: see no_alloc.h for who this is for and the full contract.
// (No counterpart in the reference.)
#include "common.cuh"
#include "api.h"
#include "no_alloc.h"
#include <mutex>

namespace {

// Scratch for the per-block partial sums, owned by the library image (4 MiB on every device that
// loads the library).  In HOST code this name is only a stand-in for the symbol, never a device
// pointer: the device address is obtained once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_col_sum_scratch[OA_COL_SUM_STATIC_MAX_FLOATS];

constexpr int kRowsPerBlock = 256;
constexpr int kMaxDevices = 64;

template <typename T> __device__ __forceinline__ float ld_as_float(const T* p);
template <> __device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// Stage 1: block (bx, by) sums rows [by*256, by*256+256) of 128 columns into partial[by, c].
// Every partial that stage 2 reads is written here, so stale contents of the shared array never matter.
template <typename T>
__global__ void static_col_sum_partial(const T* __restrict__ x, float* __restrict__ partial, long long rows, int cols) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  long long r0 = (long long)blockIdx.y * kRowsPerBlock;
  long long r1 = r0 + kRowsPerBlock < rows ? r0 + kRowsPerBlock : rows;
  float s = 0.f;
  for (long long r = r0; r < r1; ++r) s += ld_as_float<T>(x + r * cols + c);
  partial[(long long)blockIdx.y * cols + c] = s;
}

// Stage 2: fixed-order sum over the partial rows.
template <typename D>
__global__ void static_col_sum_final(const float* __restrict__ partial, D* __restrict__ out, int nparts, int cols,
                                     int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * cols + c];
  if constexpr (sizeof(D) == 4) {
    if (accumulate) s += out[c];
    out[c] = s;
  } else {
    if (accumulate) s += __bfloat162float(out[c]);
    out[c] = __float2bfloat16_rn(s);
  }
}

std::mutex g_mu;
float* g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the current device; resolved on the first call per device.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return OA_ERR_DRIVER;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_col_sum_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();  // leave no sticky-looking error behind for the caller's next check
      return OA_ERR_DRIVER;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return OA_OK;
}

}  // namespace

extern "C" size_t oa_col_sum_static_max_floats(void) { return (size_t)OA_COL_SUM_STATIC_MAX_FLOATS; }

extern "C" int oa_col_sum_static(int dtype, const void* x, void* out, int out_dtype, long long rows, int cols,
                                 int accumulate, void* stream) {
  if (rows <= 0 || cols <= 0 || !x || !out) return OA_ERR_ARG;
  if ((dtype != OA_F32 && dtype != OA_BF16) || (out_dtype != OA_F32 && out_dtype != OA_BF16)) return OA_ERR_UNSUPPORTED;
  const long long nparts = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  if (nparts > 65535 || nparts * (long long)cols > (long long)OA_COL_SUM_STATIC_MAX_FLOATS) return OA_ERR_TOO_LARGE;
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != OA_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 g1((cols + 127) / 128, (unsigned)nparts);
  if (dtype == OA_F32) static_col_sum_partial<float><<<g1, 128, 0, st>>>((const float*)x, scratch, rows, cols);
  else static_col_sum_partial<__nv_bfloat16><<<g1, 128, 0, st>>>((const __nv_bfloat16*)x, scratch, rows, cols);
  if (out_dtype == OA_F32)
    static_col_sum_final<float><<<(cols + 127) / 128, 128, 0, st>>>(scratch, (float*)out, (int)nparts, cols, accumulate);
  else
    static_col_sum_final<__nv_bfloat16><<<(cols + 127) / 128, 128, 0, st>>>(scratch, (__nv_bfloat16*)out, (int)nparts, cols, accumulate);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
