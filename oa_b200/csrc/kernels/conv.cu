// Convolution and pooling support kernels.  The reference lowers convolutions to im2col + GEMM (Conv1dGemm / Im2Col1d /
// Col2Im1d / Conv2d* / ConvTranspose2d* in Source/Private/Oa/Ml/Shader/Compute/Nn/Conv*), and has max / average pooling
// and nearest up-sampling shaders.  Here im2col / col2im are the two data-movement kernels around the tensor-core GEMM
// (col2im is written as a gather: every input element sums the column entries that cover it, so there are no atomics and
// the result is deterministic), and the pooling kernels are gathers as well.  Layout NCHW, columns
// [N*Ho*Wo, C*kh*kw] with (c, ky, kx) fastest last.
#include "common.cuh"
#include "api.h"

namespace oa {

struct ConvGeom {
  int N, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, Ho, Wo;
};

template <typename T> __device__ __forceinline__ float cld(const T* p);
template <> __device__ __forceinline__ float cld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float cld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void cst(T* p, float v);
template <> __device__ __forceinline__ void cst<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void cst<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename T>
__global__ void im2col_kernel(const T* __restrict__ x, T* __restrict__ cols, ConvGeom g) {
  const long long K = (long long)g.C * g.kh * g.kw;
  const long long total = (long long)g.N * g.Ho * g.Wo * K;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(i % K);
    long long r = i / K;
    const int ox = (int)(r % g.Wo); r /= g.Wo;
    const int oy = (int)(r % g.Ho);
    const int n = (int)(r / g.Ho);
    const int kx = k % g.kw, ky = (k / g.kw) % g.kh, c = k / (g.kw * g.kh);
    const int iy = oy * g.sh - g.ph + ky * g.dh, ix = ox * g.sw - g.pw + kx * g.dw;
    T v;
    if (iy >= 0 && iy < g.H && ix >= 0 && ix < g.W) v = x[(((long long)n * g.C + c) * g.H + iy) * g.W + ix];
    else cst<T>(&v, 0.f);
    cols[i] = v;
  }
}

// dx[n,c,iy,ix] = sum over (ky,kx) with a valid output position of cols[(n,oy,ox), (c,ky,kx)]
template <typename T>
__global__ void col2im_kernel(const T* __restrict__ cols, T* __restrict__ x, ConvGeom g) {
  const long long K = (long long)g.C * g.kh * g.kw;
  const long long total = (long long)g.N * g.C * g.H * g.W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ix = (int)(i % g.W);
    long long r = i / g.W;
    const int iy = (int)(r % g.H); r /= g.H;
    const int c = (int)(r % g.C);
    const int n = (int)(r / g.C);
    float s = 0.f;
    for (int ky = 0; ky < g.kh; ++ky) {
      const int ty = iy + g.ph - ky * g.dh;
      if (ty < 0 || ty % g.sh) continue;
      const int oy = ty / g.sh;
      if (oy >= g.Ho) continue;
      for (int kx = 0; kx < g.kw; ++kx) {
        const int tx = ix + g.pw - kx * g.dw;
        if (tx < 0 || tx % g.sw) continue;
        const int ox = tx / g.sw;
        if (ox >= g.Wo) continue;
        s += cld<T>(cols + (((long long)n * g.Ho + oy) * g.Wo + ox) * K + ((long long)c * g.kh + ky) * g.kw + kx);
      }
    }
    cst<T>(x + i, s);
  }
}

// mode 0 max (idx receives the flat input offset inside the plane, or -1), mode 1 average (count includes padding = false)
template <typename T>
__global__ void pool2d_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int* __restrict__ idx, ConvGeom g, int mode) {
  const long long total = (long long)g.N * g.C * g.Ho * g.Wo;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ox = (int)(i % g.Wo);
    long long r = i / g.Wo;
    const int oy = (int)(r % g.Ho);
    const long long plane = r / g.Ho;
    const T* px = x + plane * g.H * g.W;
    float best = -INFINITY, sum = 0.f;
    int bi = -1, cnt = 0;
    for (int ky = 0; ky < g.kh; ++ky) {
      const int iy = oy * g.sh - g.ph + ky;
      if (iy < 0 || iy >= g.H) continue;
      for (int kx = 0; kx < g.kw; ++kx) {
        const int ix = ox * g.sw - g.pw + kx;
        if (ix < 0 || ix >= g.W) continue;
        const float v = cld<T>(px + iy * g.W + ix);
        if (v > best) { best = v; bi = iy * g.W + ix; }
        sum += v; ++cnt;
      }
    }
    if (mode == 0) { cst<T>(y + i, bi >= 0 ? best : 0.f); if (idx) idx[i] = bi; }
    else cst<T>(y + i, cnt ? sum / cnt : 0.f);
  }
}

template <typename T>
__global__ void pool2d_bwd_kernel(const T* __restrict__ dy, const int* __restrict__ idx, T* __restrict__ dx, ConvGeom g, int mode) {
  const long long total = (long long)g.N * g.C * g.H * g.W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ix = (int)(i % g.W);
    long long r = i / g.W;
    const int iy = (int)(r % g.H);
    const long long plane = r / g.H;
    float s = 0.f;
    // output positions whose window covers (iy, ix)
    const int oy_lo = max(0, (iy + g.ph - g.kh + g.sh) / g.sh), oy_hi = min(g.Ho - 1, (iy + g.ph) / g.sh);
    const int ox_lo = max(0, (ix + g.pw - g.kw + g.sw) / g.sw), ox_hi = min(g.Wo - 1, (ix + g.pw) / g.sw);
    for (int oy = oy_lo; oy <= oy_hi; ++oy)
      for (int ox = ox_lo; ox <= ox_hi; ++ox) {
        const long long o = (plane * g.Ho + oy) * g.Wo + ox;
        if (mode == 0) {
          if (idx[o] == iy * g.W + ix) s += cld<T>(dy + o);
        } else {
          const int y0 = max(0, oy * g.sh - g.ph), y1 = min(g.H, oy * g.sh - g.ph + g.kh);
          const int x0 = max(0, ox * g.sw - g.pw), x1 = min(g.W, ox * g.sw - g.pw + g.kw);
          s += cld<T>(dy + o) / (float)((y1 - y0) * (x1 - x0));
        }
      }
    cst<T>(dx + i, s);
  }
}

// nearest-neighbour up-sampling by integer factors; backward sums each fy x fx block
template <typename T>
__global__ void upsample_kernel(const T* __restrict__ in, T* __restrict__ out, long long planes, int H, int W, int fy, int fx, int backward) {
  const long long total = backward ? planes * H * W : planes * H * fy * W * fx;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    if (!backward) {
      const int ox = (int)(i % (W * fx));
      long long r = i / (W * fx);
      const int oy = (int)(r % (H * fy));
      const long long pl = r / (H * fy);
      out[i] = in[(pl * H + oy / fy) * W + ox / fx];
    } else {
      const int ix = (int)(i % W);
      long long r = i / W;
      const int iy = (int)(r % H);
      const long long pl = r / H;
      float s = 0.f;
      for (int a = 0; a < fy; ++a)
        for (int b = 0; b < fx; ++b) s += cld<T>(in + (pl * H * fy + iy * fy + a) * (long long)(W * fx) + ix * fx + b);
      cst<T>(out + i, s);
    }
  }
}

static inline int cgrid(long long n) {
  long long b = (n + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  return (int)(b < 1 ? 1 : b);
}

}  // namespace oa

using namespace oa;

static int conv_geom(ConvGeom& g, int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw, int dh, int dw) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0 || ph < 0 || pw < 0) return OA_ERR_ARG;
  g = ConvGeom{N, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw, (H + 2 * ph - dh * (kh - 1) - 1) / sh + 1, (W + 2 * pw - dw * (kw - 1) - 1) / sw + 1};
  return (g.Ho > 0 && g.Wo > 0) ? OA_OK : OA_ERR_ARG;
}

#define CONV_DISPATCH(dtype, EXPR_F32, EXPR_BF16)   \
  if ((dtype) == OA_F32) { EXPR_F32; }              \
  else if ((dtype) == OA_BF16) { EXPR_BF16; }       \
  else return OA_ERR_UNSUPPORTED;

extern "C" int oa_im2col(int dtype, const void* x, void* cols, int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw,
                         int dh, int dw, void* stream) {
  ConvGeom g;
  if (int rc = conv_geom(g, N, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw)) return rc;
  const long long total = (long long)N * g.Ho * g.Wo * C * kh * kw;
  cudaStream_t st = (cudaStream_t)stream;
  CONV_DISPATCH(dtype, (im2col_kernel<float><<<cgrid(total), 256, 0, st>>>((const float*)x, (float*)cols, g)),
                (im2col_kernel<__nv_bfloat16><<<cgrid(total), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)cols, g)));
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_col2im(int dtype, const void* cols, void* x, int N, int C, int H, int W, int kh, int kw, int sh, int sw, int ph, int pw,
                         int dh, int dw, void* stream) {
  ConvGeom g;
  if (int rc = conv_geom(g, N, C, H, W, kh, kw, sh, sw, ph, pw, dh, dw)) return rc;
  const long long total = (long long)N * C * H * W;
  cudaStream_t st = (cudaStream_t)stream;
  CONV_DISPATCH(dtype, (col2im_kernel<float><<<cgrid(total), 256, 0, st>>>((const float*)cols, (float*)x, g)),
                (col2im_kernel<__nv_bfloat16><<<cgrid(total), 256, 0, st>>>((const __nv_bfloat16*)cols, (__nv_bfloat16*)x, g)));
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_pool2d_fwd(int dtype, int mode, const void* x, void* y, int* idx, int N, int C, int H, int W, int kh, int kw, int sh,
                             int sw, int ph, int pw, void* stream) {
  ConvGeom g;
  if (int rc = conv_geom(g, N, C, H, W, kh, kw, sh, sw, ph, pw, 1, 1)) return rc;
  const long long total = (long long)N * C * g.Ho * g.Wo;
  cudaStream_t st = (cudaStream_t)stream;
  CONV_DISPATCH(dtype, (pool2d_fwd_kernel<float><<<cgrid(total), 256, 0, st>>>((const float*)x, (float*)y, idx, g, mode)),
                (pool2d_fwd_kernel<__nv_bfloat16><<<cgrid(total), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, idx, g, mode)));
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_pool2d_bwd(int dtype, int mode, const void* dy, const int* idx, void* dx, int N, int C, int H, int W, int kh, int kw,
                             int sh, int sw, int ph, int pw, void* stream) {
  ConvGeom g;
  if (int rc = conv_geom(g, N, C, H, W, kh, kw, sh, sw, ph, pw, 1, 1)) return rc;
  const long long total = (long long)N * C * H * W;
  cudaStream_t st = (cudaStream_t)stream;
  CONV_DISPATCH(dtype, (pool2d_bwd_kernel<float><<<cgrid(total), 256, 0, st>>>((const float*)dy, idx, (float*)dx, g, mode)),
                (pool2d_bwd_kernel<__nv_bfloat16><<<cgrid(total), 256, 0, st>>>((const __nv_bfloat16*)dy, idx, (__nv_bfloat16*)dx, g, mode)));
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_upsample_nearest(int dtype, const void* in, void* out, long long planes, int H, int W, int fy, int fx, int backward,
                                   void* stream) {
  if (planes <= 0 || H <= 0 || W <= 0 || fy <= 0 || fx <= 0) return OA_ERR_ARG;
  const long long total = backward ? planes * H * W : planes * H * fy * W * fx;
  cudaStream_t st = (cudaStream_t)stream;
  CONV_DISPATCH(dtype, (upsample_kernel<float><<<cgrid(total), 256, 0, st>>>((const float*)in, (float*)out, planes, H, W, fy, fx, backward)),
                (upsample_kernel<__nv_bfloat16><<<cgrid(total), 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, planes, H, W, fy, fx, backward)));
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
