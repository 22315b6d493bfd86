// Image kernels on planar fp32 NCHW tensors: pointwise intensity maps, channel transforms, blends and overlays, counter-based
// noise, shared-memory tile filters (2-D and separable correlation, rectangular morphology, median, bilateral, adaptive
// thresholds), index maps (crop / flip / rotate / pad), resize and warps.  Contract: the 50 OaFnImage operations of the
// reference (Tools/FnAutogen/Schema/Vision/VisionFnImage{Pixel,Filter,Geometric,Color,Resize}.toml and the shaders under
// Source/Private/Oa/Vision/Shader/Compute/{Color,Filter,Geometric}).  The reference runs one global-memory thread per output
// sample for every filter; here a 32x32 output tile and its halo are staged once in shared memory with the border rule applied
// during staging, so separable filters and rectangular morphology run both passes out of shared memory in one launch.
#include "common.cuh"
#include "api.h"

namespace oa {

enum : int { BORDER_CONSTANT = 0, BORDER_REPLICATE = 1, BORDER_REFLECT = 2, BORDER_REFLECT101 = 3, BORDER_WRAP = 4 };

// Source index for coordinate i of an axis of length n; -1 = outside (constant border).
__device__ __forceinline__ int border_index(int i, int n, int mode) {
  if (i >= 0 && i < n) return i;
  switch (mode) {
    case BORDER_REPLICATE: return i < 0 ? 0 : n - 1;
    case BORDER_REFLECT: {
      const int p = 2 * n;
      int m = i % p;
      if (m < 0) m += p;
      return m < n ? m : p - 1 - m;
    }
    case BORDER_REFLECT101: {
      if (n == 1) return 0;
      const int p = 2 * n - 2;
      int m = i % p;
      if (m < 0) m += p;
      return m < n ? m : p - m;
    }
    case BORDER_WRAP: {
      int m = i % n;
      return m < 0 ? m + n : m;
    }
    default: return -1;
  }
}

__device__ __forceinline__ float load_border(const float* __restrict__ plane, int y, int x, int H, int W, int mode, float value) {
  const int sy = border_index(y, H, mode), sx = border_index(x, W, mode);
  return (sy < 0 || sx < 0) ? value : plane[(long long)sy * W + sx];
}

// ------------------------------------------------------------------------------------------------ pointwise
enum : int { PW_BINARY = 0, PW_BINARY_INV, PW_TRUNCATE, PW_TOZERO, PW_TOZERO_INV, PW_INRANGE, PW_CLAMP, PW_INVERT, PW_CONTRAST,
             PW_GAMMA, PW_SOLARIZE, PW_POSTERIZE };

__device__ __forceinline__ float pointwise_value(float v, int op, float p0, float p1, float p2) {
  switch (op) {
    case PW_BINARY: return v > p0 ? p1 : 0.f;
    case PW_BINARY_INV: return v > p0 ? 0.f : p1;
    case PW_TRUNCATE: return fminf(v, p0);
    case PW_TOZERO: return v > p0 ? v : 0.f;
    case PW_TOZERO_INV: return v > p0 ? 0.f : v;
    case PW_INRANGE: return (v >= p0 && v <= p1) ? p2 : 0.f;
    case PW_CLAMP: return fminf(fmaxf(v, p0), p1);
    case PW_INVERT: return p0 - v;
    case PW_CONTRAST: return v * p0 + p1;
    case PW_GAMMA: return powf(fmaxf(v, 0.f), p0) * p1;
    case PW_SOLARIZE: return v >= p0 ? p1 - v : v;
    case PW_POSTERIZE: {
      const float levels = fmaxf(p0, 2.f);
      const float t = fminf(fmaxf((v - p1) / (p2 - p1), 0.f), 1.f);
      return floorf(t * (levels - 1.f) + 0.5f) / (levels - 1.f) * (p2 - p1) + p1;   // round half up, stable for ties
    }
    default: return v;
  }
}

__global__ void image_pointwise_kernel(const float* __restrict__ x, float* __restrict__ out, long long n, int op, float p0, float p1,
                                       float p2, int vec) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, step = (long long)gridDim.x * blockDim.x;
  if (vec) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (long long i = tid; i < n / 4; i += step) {
      float4 v = x4[i];
      v.x = pointwise_value(v.x, op, p0, p1, p2);
      v.y = pointwise_value(v.y, op, p0, p1, p2);
      v.z = pointwise_value(v.z, op, p0, p1, p2);
      v.w = pointwise_value(v.w, op, p0, p1, p2);
      o4[i] = v;
    }
    return;
  }
  for (long long i = tid; i < n; i += step) out[i] = pointwise_value(x[i], op, p0, p1, p2);
}

// ------------------------------------------------------------------------------------------------ channel transforms
struct ChannelMatrix {
  float m[4][5];     // out[c] = sum_j m[c][j] * in[j] + m[c][cin]
  int sel[4];        // select mode: out[c] = in[sel[c]]
};

// mode 0: matrix by value; 1: channel selection (exact copies); 2: 3x4 colour matrix read from device memory, channels >= 3 pass through
__global__ void image_channel_kernel(const float* __restrict__ x, float* __restrict__ out, int batch, int cin, int cout, long long plane,
                                     ChannelMatrix cm, const float* __restrict__ twist, int mode) {
  const long long total = (long long)batch * plane;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / plane, p = i - b * plane;
    const float* src = x + b * cin * plane + p;
    float* dst = out + b * cout * plane + p;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < cin; ++c) v[c] = src[(long long)c * plane];
    for (int c = 0; c < cout; ++c) {
      float r;
      if (mode == 1) {
        r = v[cm.sel[c]];
      } else if (mode == 2) {
        r = c < 3 ? twist[c * 4] * v[0] + twist[c * 4 + 1] * v[1] + twist[c * 4 + 2] * v[2] + twist[c * 4 + 3] : v[c];
      } else {
        r = cm.m[c][cin];
        for (int j = 0; j < cin; ++j) r = fmaf(cm.m[c][j], v[j], r);
      }
      dst[(long long)c * plane] = r;
    }
  }
}

// ------------------------------------------------------------------------------------------------ blends
// op 0: a*(1-alpha) + b*alpha; 1: per-pixel mask (1 or C mask channels, values clamped to [0,1]); 2: rectangle fill
__global__ void image_blend_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ mask,
                                   float* __restrict__ out, int batch, int channels, int H, int W, int op, float alpha,
                                   int mask_channels, int rx, int ry, int rw, int rh, float value) {
  const long long plane = (long long)H * W, total = (long long)batch * channels * plane;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const float av = a[i];
    float r = av;
    if (op == 0) {
      r = av * (1.f - alpha) + b[i] * alpha;
    } else if (op == 1) {
      const long long p = i % plane, bc = i / plane;
      const int c = (int)(bc % channels);
      const long long n = bc / channels;
      const int mc = mask_channels == 1 ? 0 : c;
      const float m = fminf(fmaxf(mask[(n * mask_channels + mc) * plane + p], 0.f), 1.f);
      r = av * (1.f - m) + b[i] * m;
    } else {
      const long long p = i % plane;
      const int y = (int)(p / W), xx = (int)(p % W);
      if (xx >= rx && xx < rx + rw && y >= ry && y < ry + rh) r = value;
    }
    out[i] = r;
  }
}

// labels [N,H,W] int32, palette [K,3]; colour channels blend toward the label colour, a fourth channel is copied
__global__ void image_overlay_kernel(const float* __restrict__ img, const int* __restrict__ labels, const float* __restrict__ palette,
                                     float* __restrict__ out, int batch, int channels, long long plane, int classes, float alpha) {
  const long long total = (long long)batch * channels * plane;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long p = i % plane, bc = i / plane;
    const int c = (int)(bc % channels);
    const long long n = bc / channels;
    const int label = labels[n * plane + p];
    float r = img[i];
    if (c < 3 && label >= 0 && label < classes) r = r * (1.f - alpha) + palette[label * 3 + c] * alpha;
    out[i] = r;
  }
}

// ------------------------------------------------------------------------------------------------ noise
__device__ __forceinline__ unsigned image_mix32(unsigned v) {
  v ^= v >> 16; v *= 0x85ebca6bu; v ^= v >> 13; v *= 0xc2b2ae35u; v ^= v >> 16;
  return v;
}
// uniform in [0,1) with 24 bits, keyed by (seed, element, stream)
__device__ __forceinline__ float image_uniform(unsigned seed_lo, unsigned seed_hi, unsigned long long i, unsigned stream) {
  unsigned v = image_mix32(seed_lo ^ image_mix32(seed_hi + 0x9e3779b9u));
  v = image_mix32(v ^ image_mix32((unsigned)i + 0x85ebca6bu));
  v = image_mix32(v ^ image_mix32((unsigned)(i >> 32) + 0xc2b2ae35u));
  v = image_mix32(v ^ image_mix32(stream + 0x27d4eb2fu));
  return (float)(v >> 8) * (1.f / 16777216.f);
}

// op 0: x + mean + std * N(0,1) (Box-Muller); op 1: pepper below p/2, salt at or above 1 - p/2
__global__ void image_noise_kernel(const float* __restrict__ x, float* __restrict__ out, long long n, int op, float p0, float p1, float p2,
                                   unsigned seed_lo, unsigned seed_hi) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = x[i];
    const float u0 = image_uniform(seed_lo, seed_hi, (unsigned long long)i, 0u);
    if (op == 0) {
      const float u1 = image_uniform(seed_lo, seed_hi, (unsigned long long)i, 1u);
      const float r = sqrtf(-2.f * logf(1.f - u0));          // 1 - u0 in (0, 1]
      v += p0 + p1 * r * cosf(6.283185307179586f * u1);
    } else {
      const float half = p0 * 0.5f;
      if (u0 < half) v = p2;
      else if (u0 >= 1.f - half) v = p1;
    }
    out[i] = v;
  }
}

// ------------------------------------------------------------------------------------------------ tile filters
enum : int { TF_CONV2D = 0, TF_SEPARABLE, TF_MIN, TF_MAX, TF_MEDIAN, TF_BILATERAL, TF_ADAPTIVE_MEAN, TF_ADAPTIVE_GAUSS };
constexpr int TF_TILE = 32, TF_MAXR = 15, TF_HALO = TF_TILE + 2 * TF_MAXR;

__device__ __forceinline__ unsigned float_order_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float float_from_key(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ void sort2(float& a, float& b) {
  const float lo = fminf(a, b), hi = fmaxf(a, b);
  a = lo; b = hi;
}

// Median of a K x K window (K = 3, 5, 7) by forgetful selection: a working set of K*K/2 + 2 samples lives in registers; its
// minimum and maximum can never be the median, so each step drops both and takes the next sample from shared memory.  All
// loops unroll, every index is a compile-time constant.
template <int K>
__device__ __forceinline__ float median_small(const float (*halo)[TF_HALO + 1], int r, int tx) {
  constexpr int N = K * K, M0 = N / 2 + 2;
  float w[M0];
#pragma unroll
  for (int j = 0; j < M0; ++j) w[j] = halo[r + j / K][tx + j % K];
#pragma unroll
  for (int m = M0; m >= 3; --m) {
#pragma unroll
    for (int i = 0; i + 1 < m; ++i) sort2(w[i], w[i + 1]);            // maximum to w[m-1]
#pragma unroll
    for (int i = m - 2; i > 0; --i) sort2(w[i - 1], w[i]);            // minimum to w[0]
    if (m > 3) {
      const int j = M0 + (M0 - m);                                    // next unread sample (constant after unrolling)
      w[0] = halo[r + j / K][tx + j % K];
    }
  }
  return w[1];
}

// One CTA (32 x 8 threads) per 32x32 output tile of one plane.  kw x kh window (odd, <= 31), coefficient pointers by mode:
// TF_CONV2D k0 = [kh, kw]; TF_SEPARABLE k0 = horizontal [kw], k1 = vertical [kh].  p0..p2: bilateral (sigma_space, sigma_color),
// adaptive (sigma_space, offset C, max value).
// HEAVY = false compiles only the correlation and morphology modes (fewer registers, more resident CTAs); HEAVY = true the
// neighbourhood modes (median, bilateral, adaptive thresholds).
template <bool HEAVY>
__global__ void __launch_bounds__(256) image_tile_filter_kernel(const float* __restrict__ x, float* __restrict__ out, int planes, int H,
                                                                int W, int kw, int kh, int mode, int border, float border_value,
                                                                const float* __restrict__ k0, const float* __restrict__ k1, float p0,
                                                                float p1, float p2) {
  __shared__ float halo[TF_HALO][TF_HALO + 1];
  __shared__ float rows[TF_HALO][TF_TILE + 1];
  __shared__ float coef[31 * 31];
  const int rx = kw / 2, ry = kh / 2;
  const int hw = TF_TILE + 2 * rx, hh = TF_TILE + 2 * ry;
  const int tx = threadIdx.x, ty = threadIdx.y, t = ty * 32 + tx;
  const int x0 = blockIdx.x * TF_TILE, y0 = blockIdx.y * TF_TILE;
  if (mode == TF_CONV2D) {
    for (int i = t; i < kw * kh; i += 256) coef[i] = k0[i];
  } else if (mode == TF_SEPARABLE) {
    for (int i = t; i < kw; i += 256) coef[i] = k0[i];
    for (int i = t; i < kh; i += 256) coef[32 + i] = k1[i];
  }
  for (int plane = blockIdx.z; plane < planes; plane += gridDim.z) {
    const float* src = x + (long long)plane * H * W;
    float* dst = out + (long long)plane * H * W;
    __syncthreads();
    for (int i = t; i < hw * hh; i += 256) {
      const int hy = i / hw, hx = i - hy * hw;
      halo[hy][hx] = load_border(src, y0 + hy - ry, x0 + hx - rx, H, W, border, border_value);
    }
    __syncthreads();
    if (!HEAVY && (mode == TF_SEPARABLE || mode == TF_MIN || mode == TF_MAX)) {
      // horizontal pass over every halo row, then the vertical pass over the 32 columns
      for (int i = t; i < hh * TF_TILE; i += 256) {
        const int hy = i / TF_TILE, cx = i - hy * TF_TILE;
        float acc;
        if (mode == TF_SEPARABLE) {
          acc = 0.f;
          for (int k = 0; k < kw; ++k) acc = fmaf(coef[k], halo[hy][cx + k], acc);
        } else {
          acc = halo[hy][cx];
          for (int k = 1; k < kw; ++k) acc = mode == TF_MIN ? fminf(acc, halo[hy][cx + k]) : fmaxf(acc, halo[hy][cx + k]);
        }
        rows[hy][cx] = acc;
      }
      __syncthreads();
      for (int r = ty; r < TF_TILE; r += 8) {
        const int oy = y0 + r, ox = x0 + tx;
        if (oy >= H || ox >= W) continue;
        float acc;
        if (mode == TF_SEPARABLE) {
          acc = 0.f;
          for (int k = 0; k < kh; ++k) acc = fmaf(coef[32 + k], rows[r + k][tx], acc);
        } else {
          acc = rows[r][tx];
          for (int k = 1; k < kh; ++k) acc = mode == TF_MIN ? fminf(acc, rows[r + k][tx]) : fmaxf(acc, rows[r + k][tx]);
        }
        dst[(long long)oy * W + ox] = acc;
      }
      continue;
    }
    for (int r = ty; r < TF_TILE; r += 8) {
      const int oy = y0 + r, ox = x0 + tx;
      if (oy >= H || ox >= W) continue;
      float result;
      if constexpr (!HEAVY) {
        float acc = 0.f;
        for (int ky = 0; ky < kh; ++ky)
          for (int kx = 0; kx < kw; ++kx) acc = fmaf(coef[ky * kw + kx], halo[r + ky][tx + kx], acc);
        result = acc;
      } else if (mode == TF_MEDIAN && kw == kh && kw <= 7) {
        result = kw == 1 ? halo[r][tx] : kw == 3 ? median_small<3>(halo, r, tx) : kw == 5 ? median_small<5>(halo, r, tx) : median_small<7>(halo, r, tx);
      } else if (mode == TF_MEDIAN) {
        // rank selection by bisection over the order-preserving bit pattern: no per-thread sample array
        const int rank = (kw * kh) / 2;
        unsigned key = 0u;
        for (int bit = 31; bit >= 0; --bit) {
          const unsigned cand = key | (1u << bit);
          int below = 0;
          for (int ky = 0; ky < kh; ++ky)
            for (int kx = 0; kx < kw; ++kx) below += float_order_key(halo[r + ky][tx + kx]) < cand ? 1 : 0;
          if (below <= rank) key = cand;
        }
        result = float_from_key(key);
      } else {
        const float center = halo[r + ry][tx + rx];
        const float ss = fmaxf(p0, 1e-6f), sc = fmaxf(p1, 1e-6f);
        float weighted = 0.f, wsum = 0.f;
        for (int ky = 0; ky < kh; ++ky) {
          const int dy = ky - ry;
          for (int kx = 0; kx < kw; ++kx) {
            const int dx = kx - rx;
            const float s = halo[r + ky][tx + kx];
            float w = 1.f;
            if (mode == TF_BILATERAL) {
              const float d = s - center;
              w = __expf(-(float)(dx * dx + dy * dy) / (2.f * ss * ss) - d * d / (2.f * sc * sc));
            } else if (mode == TF_ADAPTIVE_GAUSS) {
              w = __expf(-(float)(dx * dx + dy * dy) / (2.f * ss * ss));
            }
            weighted = fmaf(s, w, weighted);
            wsum += w;
          }
        }
        const float filtered = weighted / fmaxf(wsum, 1e-20f);
        result = mode == TF_BILATERAL ? filtered : (center > filtered - p1 ? p2 : 0.f);
      }
      dst[(long long)oy * W + ox] = result;
    }
  }
}

// ------------------------------------------------------------------------------------------------ index maps
// op 0 crop (a0 = x, a1 = y); 1 flip (a0 = horizontal, a1 = vertical); 2 rotate clockwise (a0 = degrees); 3 pad (a0 = left, a1 = top)
__global__ void image_index_map_kernel(const float* __restrict__ x, float* __restrict__ out, int planes, int Hi, int Wi, int Ho, int Wo,
                                       int op, int a0, int a1, int border, float border_value) {
  const long long plane_o = (long long)Ho * Wo, total = (long long)planes * plane_o;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long pl = i / plane_o, p = i - pl * plane_o;
    const int y = (int)(p / Wo), xx = (int)(p % Wo);
    const float* src = x + pl * Hi * Wi;
    int sx = xx, sy = y;
    if (op == 0) {
      sx = xx + a0; sy = y + a1;
    } else if (op == 1) {
      if (a0) sx = Wi - 1 - xx;
      if (a1) sy = Hi - 1 - y;
    } else if (op == 2) {
      if (a0 == 90) { sx = y; sy = Hi - 1 - xx; }
      else if (a0 == 180) { sx = Wi - 1 - xx; sy = Hi - 1 - y; }
      else if (a0 == 270) { sx = Wi - 1 - y; sy = xx; }
    } else {
      out[i] = load_border(src, y - a1, xx - a0, Hi, Wi, border, border_value);
      continue;
    }
    out[i] = src[(long long)sy * Wi + sx];
  }
}

// mode 0 nearest (floor(out * in / out_size)), 1 bilinear with half-pixel centres and edge clamping; optional per-channel
// (v - mean[c]) / std[c] applied to the sample (mean == nullptr: none)
__global__ void image_resize_kernel(const float* __restrict__ x, float* __restrict__ out, int planes, int channels, int Hi, int Wi, int Ho,
                                    int Wo, int mode, float m0, float m1, float m2, float s0, float s1, float s2, int normalize) {
  const long long plane_o = (long long)Ho * Wo, total = (long long)planes * plane_o;
  const float scale_y = (float)Hi / (float)Ho, scale_x = (float)Wi / (float)Wo;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long pl = i / plane_o, p = i - pl * plane_o;
    const int y = (int)(p / Wo), xx = (int)(p % Wo);
    const float* src = x + pl * Hi * Wi;
    float v;
    if (mode == 0) {
      const int sy = min((int)floorf((float)y * scale_y), Hi - 1), sx = min((int)floorf((float)xx * scale_x), Wi - 1);
      v = src[(long long)sy * Wi + sx];
    } else {
      const float fy = fminf(fmaxf(((float)y + 0.5f) * scale_y - 0.5f, 0.f), (float)(Hi - 1));
      const float fx = fminf(fmaxf(((float)xx + 0.5f) * scale_x - 0.5f, 0.f), (float)(Wi - 1));
      const int yy0 = (int)floorf(fy), xx0 = (int)floorf(fx);
      const int yy1 = min(yy0 + 1, Hi - 1), xx1 = min(xx0 + 1, Wi - 1);
      const float wy = fy - (float)yy0, wx = fx - (float)xx0;
      const float v00 = src[(long long)yy0 * Wi + xx0], v01 = src[(long long)yy0 * Wi + xx1];
      const float v10 = src[(long long)yy1 * Wi + xx0], v11 = src[(long long)yy1 * Wi + xx1];
      const float top = v00 + (v01 - v00) * wx, bot = v10 + (v11 - v10) * wx;
      v = top + (bot - top) * wy;
    }
    if (normalize) {
      const int c = (int)(pl % channels);
      const float mean = c == 0 ? m0 : (c == 1 ? m1 : m2), sd = c == 0 ? s0 : (c == 1 ? s1 : s2);
      if (c < 3) v = (v - mean) / sd;
    }
    out[i] = v;
  }
}

// (m0 * x + m1 * y) + m2 with every product and sum rounded on its own (no contraction into fused multiply-adds), so that
// nearest-neighbour warps pick the same source pixel as the same expression evaluated elsewhere in fp32
__device__ __forceinline__ float affine_row(const float* __restrict__ m, float x, float y) {
  return __fadd_rn(__fadd_rn(__fmul_rn(m[0], x), __fmul_rn(m[1], y)), m[2]);
}

// op 0 remap (map [Nm,2,Ho,Wo]: x plane then y plane, Nm = 1 or N); 1 inverse affine 2x3; 2 inverse perspective 3x3
__global__ void image_warp_kernel(const float* __restrict__ x, const float* __restrict__ map, float* __restrict__ out, int batch,
                                  int channels, int Hi, int Wi, int Ho, int Wo, int op, int map_batch, int interp, int border,
                                  float border_value) {
  const long long plane_o = (long long)Ho * Wo, total = (long long)batch * channels * plane_o;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long pl = i / plane_o, p = i - pl * plane_o;
    const int y = (int)(p / Wo), xx = (int)(p % Wo);
    const long long b = pl / channels;
    float sx, sy;
    bool valid = true;
    if (op == 0) {
      const long long base = (map_batch == 1 ? 0 : b) * 2 * plane_o + p;
      sx = map[base]; sy = map[base + plane_o];
    } else if (op == 1) {
      sx = affine_row(map, (float)xx, (float)y);
      sy = affine_row(map + 3, (float)xx, (float)y);
    } else {
      const float den = affine_row(map + 6, (float)xx, (float)y);
      valid = fabsf(den) > 1e-12f;
      sx = valid ? __fdiv_rn(affine_row(map, (float)xx, (float)y), den) : 0.f;
      sy = valid ? __fdiv_rn(affine_row(map + 3, (float)xx, (float)y), den) : 0.f;
    }
    const float* src = x + pl * Hi * Wi;
    float v;
    if (!valid || !(sx == sx) || !(sy == sy) || fabsf(sx) > 1e9f || fabsf(sy) > 1e9f) {
      v = border_value;
    } else if (interp == 0) {
      v = load_border(src, (int)floorf(sy + 0.5f), (int)floorf(sx + 0.5f), Hi, Wi, border, border_value);
    } else {
      const int yy0 = (int)floorf(sy), xx0 = (int)floorf(sx);
      const float wy = sy - (float)yy0, wx = sx - (float)xx0;
      const float v00 = load_border(src, yy0, xx0, Hi, Wi, border, border_value);
      const float v01 = load_border(src, yy0, xx0 + 1, Hi, Wi, border, border_value);
      const float v10 = load_border(src, yy0 + 1, xx0, Hi, Wi, border, border_value);
      const float v11 = load_border(src, yy0 + 1, xx0 + 1, Hi, Wi, border, border_value);
      const float top = v00 + (v01 - v00) * wx, bot = v10 + (v11 - v10) * wx;
      v = top + (bot - top) * wy;
    }
    out[i] = v;
  }
}

// Gradient of image_resize_kernel with respect to its input, as a gather: one thread per INPUT pixel sums, in a fixed
// order, the output gradients that read it (no atomics, so the result is bit-reproducible).  The candidate output rows /
// columns come from inverting the coordinate map with a margin; each candidate is re-run through the forward map, so
// the weights are exactly the forward pass's.
__device__ __forceinline__ float resize_axis_weight(int o, int r, float scale, int n_in, int mode) {
  if (mode == 0) return min((int)floorf((float)o * scale), n_in - 1) == r ? 1.f : 0.f;
  const float f = fminf(fmaxf(((float)o + 0.5f) * scale - 0.5f, 0.f), (float)(n_in - 1));
  const int i0 = (int)floorf(f), i1 = min(i0 + 1, n_in - 1);
  const float w = f - (float)i0;
  return (i0 == r ? 1.f - w : 0.f) + (i1 == r ? w : 0.f);
}

__global__ void image_resize_bwd_kernel(const float* __restrict__ g, float* __restrict__ dx, int planes, int Hi, int Wi, int Ho, int Wo, int mode) {
  const long long plane_i = (long long)Hi * Wi, total = (long long)planes * plane_i;
  const float scale_y = (float)Hi / (float)Ho, scale_x = (float)Wi / (float)Wo;
  const float inv_y = (float)Ho / (float)Hi, inv_x = (float)Wo / (float)Wi;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long pl = i / plane_i, p = i - pl * plane_i;
    const int r = (int)(p / Wi), c = (int)(p % Wi);
    // outputs whose source coordinate lies within one input pixel of (r, c), plus one of margin; the edge pixels also
    // collect the outputs whose coordinate was clamped onto them
    int y_lo = max((int)floorf(((float)r - 0.5f) * inv_y - 0.5f) - 1, 0);
    int y_hi = min((int)ceilf(fmaxf(((float)r + 1.5f) * inv_y - 0.5f, (float)(r + 1) * inv_y)) + 1, Ho - 1);
    int x_lo = max((int)floorf(((float)c - 0.5f) * inv_x - 0.5f) - 1, 0);
    int x_hi = min((int)ceilf(fmaxf(((float)c + 1.5f) * inv_x - 0.5f, (float)(c + 1) * inv_x)) + 1, Wo - 1);
    if (r == 0) y_lo = 0;
    if (r == Hi - 1) y_hi = Ho - 1;
    if (c == 0) x_lo = 0;
    if (c == Wi - 1) x_hi = Wo - 1;
    const float* gp = g + pl * (long long)Ho * Wo;
    float acc = 0.f;
    const int nx = x_hi - x_lo + 1;
    if (nx <= 8) {                                   // the usual case: column weights once, in registers
      float wxs[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) wxs[j] = j < nx ? resize_axis_weight(x_lo + j, c, scale_x, Wi, mode) : 0.f;
      for (int y = y_lo; y <= y_hi; ++y) {
        const float wy = resize_axis_weight(y, r, scale_y, Hi, mode);
        if (wy == 0.f) continue;
        const float* grow = gp + (long long)y * Wo + x_lo;
        float row = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (wxs[j] != 0.f) row += wxs[j] * grow[j];
        acc += wy * row;
      }
    } else {
      for (int y = y_lo; y <= y_hi; ++y) {
        const float wy = resize_axis_weight(y, r, scale_y, Hi, mode);
        if (wy == 0.f) continue;
        float row = 0.f;
        for (int x = x_lo; x <= x_hi; ++x) {
          const float wx = resize_axis_weight(x, c, scale_x, Wi, mode);
          if (wx != 0.f) row += wx * gp[(long long)y * Wo + x];
        }
        acc += wy * row;
      }
    }
    dx[i] = acc;
  }
}

static inline int grid_for(long long n, int block = 256) {
  long long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace oa

using namespace oa;

extern "C" {

int oa_image_pointwise(const void* x, void* out, long long n, int op, float p0, float p1, float p2, void* stream) {
  if (n <= 0) return 0;
  const int vec = (n % 4 == 0) && (((uintptr_t)x | (uintptr_t)out) % 16 == 0);
  image_pointwise_kernel<<<grid_for(vec ? n / 4 : n), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, n, op, p0, p1, p2, vec);
  return (int)cudaGetLastError();
}

int oa_image_channels(const void* x, void* out, int batch, int cin, int cout, long long plane, const float* matrix20, const int* sel4,
                      const void* twist, int mode, void* stream) {
  if (cin < 1 || cin > 4 || cout < 1 || cout > 4) return (int)cudaErrorInvalidValue;
  ChannelMatrix cm{};
  if (matrix20) for (int c = 0; c < 4; ++c) for (int j = 0; j < 5; ++j) cm.m[c][j] = matrix20[c * 5 + j];
  if (sel4) for (int c = 0; c < 4; ++c) cm.sel[c] = sel4[c] < 0 || sel4[c] >= cin ? 0 : sel4[c];
  image_channel_kernel<<<grid_for((long long)batch * plane), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, batch, cin, cout,
                                                                                              plane, cm, (const float*)twist, mode);
  return (int)cudaGetLastError();
}

int oa_image_blend(const void* a, const void* b, const void* mask, void* out, int batch, int channels, int H, int W, int op, float alpha,
                   int mask_channels, int rx, int ry, int rw, int rh, float value, void* stream) {
  image_blend_kernel<<<grid_for((long long)batch * channels * H * W), 256, 0, (cudaStream_t)stream>>>(
      (const float*)a, (const float*)b, (const float*)mask, (float*)out, batch, channels, H, W, op, alpha, mask_channels, rx, ry, rw, rh, value);
  return (int)cudaGetLastError();
}

int oa_image_overlay(const void* img, const void* labels, const void* palette, void* out, int batch, int channels, long long plane,
                     int classes, float alpha, void* stream) {
  image_overlay_kernel<<<grid_for((long long)batch * channels * plane), 256, 0, (cudaStream_t)stream>>>(
      (const float*)img, (const int*)labels, (const float*)palette, (float*)out, batch, channels, plane, classes, alpha);
  return (int)cudaGetLastError();
}

int oa_image_noise(const void* x, void* out, long long n, int op, float p0, float p1, float p2, unsigned long long seed, void* stream) {
  if (n <= 0) return 0;
  image_noise_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, n, op, p0, p1, p2, (unsigned)seed,
                                                                      (unsigned)(seed >> 32));
  return (int)cudaGetLastError();
}

int oa_image_tile_filter(const void* x, void* out, int planes, int H, int W, int kw, int kh, int mode, int border, float border_value,
                         const void* k0, const void* k1, float p0, float p1, float p2, void* stream) {
  if (kw < 1 || kh < 1 || kw > 31 || kh > 31 || !(kw & 1) || !(kh & 1) || planes < 1) return (int)cudaErrorInvalidValue;
  dim3 grid((W + TF_TILE - 1) / TF_TILE, (H + TF_TILE - 1) / TF_TILE, planes > 4096 ? 4096 : planes);
  if (mode <= TF_MAX)
    image_tile_filter_kernel<false><<<grid, dim3(32, 8), 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, planes, H, W, kw, kh, mode,
                                                                                    border, border_value, (const float*)k0, (const float*)k1,
                                                                                    p0, p1, p2);
  else
    image_tile_filter_kernel<true><<<grid, dim3(32, 8), 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, planes, H, W, kw, kh, mode,
                                                                                   border, border_value, (const float*)k0, (const float*)k1,
                                                                                   p0, p1, p2);
  return (int)cudaGetLastError();
}

int oa_image_index_map(const void* x, void* out, int planes, int Hi, int Wi, int Ho, int Wo, int op, int a0, int a1, int border,
                       float border_value, void* stream) {
  image_index_map_kernel<<<grid_for((long long)planes * Ho * Wo), 256, 0, (cudaStream_t)stream>>>((const float*)x, (float*)out, planes, Hi, Wi,
                                                                                                   Ho, Wo, op, a0, a1, border, border_value);
  return (int)cudaGetLastError();
}

int oa_image_resize(const void* x, void* out, int planes, int channels, int Hi, int Wi, int Ho, int Wo, int mode, const float* mean3,
                    const float* std3, void* stream) {
  const int norm = mean3 != nullptr && std3 != nullptr;
  image_resize_kernel<<<grid_for((long long)planes * Ho * Wo), 256, 0, (cudaStream_t)stream>>>(
      (const float*)x, (float*)out, planes, channels, Hi, Wi, Ho, Wo, mode, norm ? mean3[0] : 0.f, norm ? mean3[1] : 0.f, norm ? mean3[2] : 0.f,
      norm ? std3[0] : 1.f, norm ? std3[1] : 1.f, norm ? std3[2] : 1.f, norm);
  return (int)cudaGetLastError();
}

int oa_image_resize_bwd(const void* grad_out, void* grad_in, int planes, int Hi, int Wi, int Ho, int Wo, int mode, void* stream) {
  image_resize_bwd_kernel<<<grid_for((long long)planes * Hi * Wi), 256, 0, (cudaStream_t)stream>>>((const float*)grad_out, (float*)grad_in, planes,
                                                                                                     Hi, Wi, Ho, Wo, mode);
  return (int)cudaGetLastError();
}

int oa_image_warp(const void* x, const void* map, void* out, int batch, int channels, int Hi, int Wi, int Ho, int Wo, int op, int map_batch,
                  int interp, int border, float border_value, void* stream) {
  image_warp_kernel<<<grid_for((long long)batch * channels * Ho * Wo), 256, 0, (cudaStream_t)stream>>>(
      (const float*)x, (const float*)map, (float*)out, batch, channels, Hi, Wi, Ho, Wo, op, map_batch, interp, border, border_value);
  return (int)cudaGetLastError();
}

}  // extern "C"
