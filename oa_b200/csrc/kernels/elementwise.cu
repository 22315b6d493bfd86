// Flat elementwise, indexing, row-reduction, softmax and RNG kernels (fp32 or bf16 storage,
// fp32 math).  These cover the reference's generated elementwise family
// (Source/Private/Oa/Core/Shader/Compute/Flat/*.slang), the activations
// (Source/Private/Oa/Ml/Shader/Compute/Nn/Activation/*.slang), Swiglu, RopeApply, Embedding /
// Gather and the Philox generators (Source/Private/Oa/Core/Shader/Compute/Math/Philox.slang:18-84).
// All are bandwidth-bound: 16-byte vector accesses, grid-stride loops sized to the SM count.
#include <cstring>
#include "common.cuh"
#include "api.h"

namespace oa {

template <typename T> struct IO;
template <> struct IO<float> {
  static constexpr int VEC = 4;
  __device__ static void load(const float* p, float* v) {
    float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  __device__ static void store(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
  __device__ static float ld1(const float* p) { return *p; }
  __device__ static void st1(float* p, float v) { *p = v; }
};
template <> struct IO<__nv_bfloat16> {
  static constexpr int VEC = 8;
  __device__ static void load(const __nv_bfloat16* p, float* v) {
    uint4 x = *reinterpret_cast<const uint4*>(p);
    float2 a = unpack_bf16x2(x.x), b = unpack_bf16x2(x.y), c = unpack_bf16x2(x.z), d = unpack_bf16x2(x.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  __device__ static void store(__nv_bfloat16* p, const float* v) {
    *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                              pack_bf16x2(v[6], v[7]));
  }
  __device__ static float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static void st1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

static inline int grid_for(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  long long cap = 148LL * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__device__ __forceinline__ float unary_apply(int op, float x, float s0, float s1) {
  switch (op) {
    case OA_U_COPY: return x;
    case OA_U_NEG: return -x;
    case OA_U_ABS: return fabsf(x);
    case OA_U_LOG: return logf(x);
    case OA_U_EXP: return expf(x);
    case OA_U_SQRT: return sqrtf(x);
    case OA_U_SIN: return sinf(x);
    case OA_U_COS: return cosf(x);
    case OA_U_RECIP: return 1.f / x;
    case OA_U_SCALE: return x * s0;
    case OA_U_ADD_SCALAR: return x + s0;
    case OA_U_POW: return powf(x, s0);
    case OA_U_CLAMP_MAX: return fminf(x, s0);
    case OA_U_CLAMP_MIN: return fmaxf(x, s0);
    case OA_U_RELU: return fmaxf(x, 0.f);
    case OA_U_GELU: return gelu_tanh(x);
    case OA_U_SILU: return silu_f(x);
    case OA_U_TANH: return tanhf(x);
    case OA_U_SIGMOID: return sigmoid_f(x);
    case OA_U_SOFTPLUS: return softplus_f(x);
    case OA_U_LEAKY_RELU: return x > 0.f ? x : s0 * x;
    case OA_U_ELU: return x > 0.f ? x : s0 * (expf(x) - 1.f);
    case OA_U_MISH: return x * tanhf(softplus_f(x));
    case OA_U_SQUARE: return x * x;
    case OA_U_RSUB_SCALAR: return s0 - x;
    case OA_U_SIGN: return (x > 0.f) - (x < 0.f);
  }
  return x;
}

// a = saved tensor (input x unless noted), b = upstream gradient.
__device__ __forceinline__ float binary_apply(int op, float a, float b, float s0) {
  switch (op) {
    case OA_B_ADD: return a + b;
    case OA_B_SUB: return a - b;
    case OA_B_MUL: return a * b;
    case OA_B_DIV: return a / b;
    case OA_B_MAX: return fmaxf(a, b);
    case OA_B_MIN: return fminf(a, b);
    case OA_B_EQ: return a == b ? 1.f : 0.f;
    case OA_B_GE: return a >= b ? 1.f : 0.f;
    case OA_B_RELU_BWD: return a > 0.f ? b : 0.f;
    case OA_B_GELU_BWD: return b * gelu_tanh_grad(a);
    case OA_B_SILU_BWD: { float s = sigmoid_f(a); return b * s * (1.f + a * (1.f - s)); }
    case OA_B_TANH_BWD: return b * (1.f - a * a);          // a = forward OUTPUT
    case OA_B_SIGMOID_BWD: return b * a * (1.f - a);       // a = forward OUTPUT
    case OA_B_SOFTPLUS_BWD: return b * sigmoid_f(a);
    case OA_B_LEAKY_RELU_BWD: return a > 0.f ? b : s0 * b;
    case OA_B_ELU_BWD: return a > 0.f ? b : b * s0 * expf(a);
    case OA_B_MISH_BWD: {
      float sp = softplus_f(a), t = tanhf(sp), s = sigmoid_f(a);
      return b * (t + a * (1.f - t * t) * s);
    }
    case OA_B_ABS_BWD: return a > 0.f ? b : (a < 0.f ? -b : 0.f);
    case OA_B_LOG_BWD: return b / a;
    case OA_B_SQRT_BWD: return b * 0.5f / a;                // a = forward OUTPUT
    case OA_B_RECIP_BWD: return -b * a * a;                 // a = forward OUTPUT
    case OA_B_SILU_MUL: return silu_f(a) * b;
  }
  return a;
}

template <typename T>
__global__ void unary_kernel(int op, const T* __restrict__ x, T* __restrict__ y, long long n, float s0, float s1) {
  constexpr int V = IO<T>::VEC;
  long long nv = n / V;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float v[V];
    IO<T>::load(x + i * V, v);
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = unary_apply(op, v[j], s0, s1);
    IO<T>::store(y + i * V, v);
  }
  for (long long i = nv * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    IO<T>::st1(y + i, unary_apply(op, IO<T>::ld1(x + i), s0, s1));
}

template <typename T>
__global__ void binary_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long long n,
                              long long inner, int mode, float s0) {
  long long stride = (long long)gridDim.x * blockDim.x;
  if (mode == OA_BC_NONE) {
    constexpr int V = IO<T>::VEC;
    long long nv = n / V;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
      float va[V], vb[V];
      IO<T>::load(a + i * V, va);
      IO<T>::load(b + i * V, vb);
#pragma unroll
      for (int j = 0; j < V; ++j) va[j] = binary_apply(op, va[j], vb[j], s0);
      IO<T>::store(y + i * V, va);
    }
    for (long long i = nv * V + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
      IO<T>::st1(y + i, binary_apply(op, IO<T>::ld1(a + i), IO<T>::ld1(b + i), s0));
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      long long bi = mode == OA_BC_ROW ? (i % inner) : (mode == OA_BC_COL ? (i / inner) : 0);
      IO<T>::st1(y + i, binary_apply(op, IO<T>::ld1(a + i), IO<T>::ld1(b + bi), s0));
    }
  }
}

template <typename S, typename D>
__global__ void cast_kernel(const S* __restrict__ x, D* __restrict__ y, long long n) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    IO<D>::st1(y + i, IO<S>::ld1(x + i));
}

template <typename T>
__global__ void fill_kernel(T* y, long long n, float value) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) IO<T>::st1(y + i, value);
}

// 16 bytes per store for the bulk of an aligned fill (the element-wise kernel above writes 2 or 4 bytes per thread)
__global__ void fill_vec_kernel(uint4* y, long long n16, uint4 pattern) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) y[i] = pattern;
}

// Swiglu on a packed [rows, 2F] tensor: out = silu(A[:, :F]) * A[:, F:]
// (Source/Private/Oa/Core/FnMatrix/.../FnMatrixActivation.gen.h:47-60).
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int F) {
  constexpr int V = IO<T>::VEC;
  long long per_row = F / V;
  long long total = rows * per_row;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long r = i / per_row;
    int c = (int)(i % per_row) * V;
    float g[V], u[V];
    IO<T>::load(gu + r * 2 * F + c, g);
    IO<T>::load(gu + r * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < V; ++j) g[j] = silu_f(g[j]) * u[j];
    IO<T>::store(out + r * F + c, g);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dout, T* __restrict__ dgu,
                                  long long rows, int F) {
  constexpr int V = IO<T>::VEC;
  long long per_row = F / V;
  long long total = rows * per_row;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long r = i / per_row;
    int c = (int)(i % per_row) * V;
    float g[V], u[V], d[V], dg[V], du[V];
    IO<T>::load(gu + r * 2 * F + c, g);
    IO<T>::load(gu + r * 2 * F + F + c, u);
    IO<T>::load(dout + r * F + c, d);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float s = sigmoid_f(g[j]);
      du[j] = d[j] * g[j] * s;
      dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
    }
    IO<T>::store(dgu + r * 2 * F + c, dg);
    IO<T>::store(dgu + r * 2 * F + F + c, du);
  }
}

// Rotate-half RoPE applied in place on heads laid out side by side in a row:
// pairs (i, i + hd/2), angle = pos * theta^(-2i/hd)  (Nn/Rope/RopeApply.slang:39-56).
// `backward` applies the inverse rotation (the transpose of the forward one).
template <typename T>
__global__ void rope_kernel(T* x, long long rows, int row_stride, int n_heads, int hd, int seq_len, int pos_offset,
                            float theta, int backward, const int* __restrict__ pos_dev) {
  if (pos_dev) pos_offset += *pos_dev;           // device-resident position (graph-replayed decode steps)
  int half = hd / 2;
  long long total = rows * n_heads * half;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int j = (int)(i % half);
    long long t = i / half;
    int h = (int)(t % n_heads);
    long long r = t / n_heads;
    int pos = (int)(r % seq_len) + pos_offset;
    float freq = __powf(theta, -2.f * (float)j / (float)hd);
    float s, c;
    sincosf((float)pos * freq, &s, &c);
    if (backward) s = -s;
    T* p = x + r * row_stride + h * hd + j;
    float a = IO<T>::ld1(p), b = IO<T>::ld1(p + half);
    IO<T>::st1(p, a * c - b * s);
    IO<T>::st1(p + half, b * c + a * s);
  }
}

// bf16 fast path: one thread owns 8 consecutive pair indices j of one row, computes their 8 (cos, sin) once and applies
// them to every head of the row with 16-byte accesses (the angle depends on the position and on j only).
__global__ void __launch_bounds__(256)
rope_bf16_vec_kernel(__nv_bfloat16* x, long long rows, int row_stride, int n_heads, int hd, int seq_len, int pos_offset, float theta,
                     int backward, const int* __restrict__ pos_dev) {
  pdl_launch_dependents();
  pdl_wait();
  if (pos_dev) pos_offset += *pos_dev;
  const int half = hd >> 1, jv = half >> 3;                 // 8-wide vectors per half head
  const long long total = rows * jv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % jv);
    const long long r = i / jv;
    const float pos = (float)((int)(r % seq_len) + pos_offset);
    float c[8], s[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float freq = __powf(theta, -2.f * (float)(v * 8 + k) / (float)hd);
      sincosf(pos * freq, &s[k], &c[k]);
      if (backward) s[k] = -s[k];
    }
    __nv_bfloat16* row = x + r * row_stride + v * 8;
    // four heads per round: their eight 16-byte loads are issued before the first use, so one thread keeps 128 bytes in flight
    constexpr int HB = 4;
    for (int h0 = 0; h0 < n_heads; h0 += HB) {
      uint4 ua[HB], ub[HB];
#pragma unroll
      for (int u = 0; u < HB; ++u) {
        if (h0 + u < n_heads) {
          ua[u] = *reinterpret_cast<const uint4*>(row + (h0 + u) * hd);
          ub[u] = *reinterpret_cast<const uint4*>(row + (h0 + u) * hd + half);
        }
      }
#pragma unroll
      for (int u = 0; u < HB; ++u) {
        if (h0 + u < n_heads) {
          const uint32_t wa[4] = {ua[u].x, ua[u].y, ua[u].z, ua[u].w}, wb[4] = {ub[u].x, ub[u].y, ub[u].z, ub[u].w};
          uint32_t oa[4], ob[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 a = unpack_bf16x2(wa[k]), b = unpack_bf16x2(wb[k]);
            oa[k] = pack_bf16x2(a.x * c[2 * k] - b.x * s[2 * k], a.y * c[2 * k + 1] - b.y * s[2 * k + 1]);
            ob[k] = pack_bf16x2(b.x * c[2 * k] + a.x * s[2 * k], b.y * c[2 * k + 1] + a.y * s[2 * k + 1]);
          }
          *reinterpret_cast<uint4*>(row + (h0 + u) * hd) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
          *reinterpret_cast<uint4*>(row + (h0 + u) * hd + half) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
        }
      }
    }
  }
}

// out[i,:] = table[ids[i],:] (+ pos_table[i % seq_len,:])
template <typename T>
__global__ void embedding_fwd_kernel(const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out,
                                     long long n_ids, int dim, int vocab, const T* __restrict__ pos, int seq_len) {
  constexpr int V = IO<T>::VEC;
  int per_row = dim / V;
  long long total = n_ids * per_row;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long r = i / per_row;
    int c = (int)(i % per_row) * V;
    int id = ids[r];
    float v[V];
    if (id < 0 || id >= vocab) {
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] = __int_as_float(0x7fc00000);
    } else {
      IO<T>::load(table + (long long)id * dim + c, v);
    }
    if (pos) {
      float pv[V];
      IO<T>::load(pos + (r % seq_len) * dim + c, pv);
#pragma unroll
      for (int j = 0; j < V; ++j) v[j] += pv[j];
    }
    IO<T>::store(out + r * dim + c, v);
  }
}
// fp32 scatter-add of the output gradient into the table gradient.
template <typename T>
__global__ void embedding_bwd_kernel(const T* __restrict__ dout, const int* __restrict__ ids, float* __restrict__ dtable,
                                     long long n_ids, int dim, int vocab) {
  long long total = n_ids * dim;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    long long r = i / dim;
    int c = (int)(i % dim);
    int id = ids[r];
    if (id >= 0 && id < vocab) atomicAdd(dtable + (long long)id * dim + c, IO<T>::ld1(dout + i));
  }
}

// Column sums (bias gradient): stage 1 writes per-block partials, stage 2 reduces them in a fixed order.
// Block = 128 columns x 4 row lanes; a lane walks every fourth row of the block's slab with four independent partial sums
// (16 loads in flight per column), the lanes are then added in a fixed order, so the result does not depend on scheduling.
template <typename T>
__global__ void __launch_bounds__(512)
col_sum_partial_kernel(const T* __restrict__ x, float* __restrict__ partial, long long rows, int cols, int rows_per_block) {
  __shared__ float sm[4][128];
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int lane = threadIdx.y;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < cols) {
    long long r = r0 + lane;
    // a lane's 64 rows of a full block as 16 independent loads: small matrices give few blocks, so the time of this kernel is
    // the latency of its dependent rounds, not bandwidth
    for (; r + 60 < r1; r += 64) {
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = IO<T>::ld1(x + (r + 4 * u) * cols + c);
#pragma unroll
      for (int u = 0; u < 16; u += 4) { s0 += v[u]; s1 += v[u + 1]; s2 += v[u + 2]; s3 += v[u + 3]; }
    }
    for (; r + 12 < r1; r += 16) {
      s0 += IO<T>::ld1(x + r * cols + c);
      s1 += IO<T>::ld1(x + (r + 4) * cols + c);
      s2 += IO<T>::ld1(x + (r + 8) * cols + c);
      s3 += IO<T>::ld1(x + (r + 12) * cols + c);
    }
    for (; r < r1; r += 4) s0 += IO<T>::ld1(x + r * cols + c);
  }
  sm[lane][threadIdx.x] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (lane == 0 && c < cols)
    partial[(long long)blockIdx.y * cols + c] = (sm[0][threadIdx.x] + sm[1][threadIdx.x]) + (sm[2][threadIdx.x] + sm[3][threadIdx.x]);
}
template <typename D>
__global__ void col_sum_final_kernel(const float* __restrict__ partial, D* __restrict__ out, int nparts, int cols,
                                     int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * cols + c];
  if (accumulate) s += IO<D>::ld1(out + c);
  IO<D>::st1(out + c, s);
}

template <typename T>
__global__ void bias_add_kernel(T* x, const T* __restrict__ bias, long long rows, int cols) {
  long long total = rows * cols;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
    IO<T>::st1(x + i, IO<T>::ld1(x + i) + IO<T>::ld1(bias + i % cols));
}

// One warp per row: sum / mean / max / argmax (ties -> lower index, like Flat/TopK.slang:39-77).
template <typename T>
__global__ void row_reduce_kernel(int op, const T* __restrict__ x, void* __restrict__ y, long long rows, int cols) {
  long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const T* p = x + row * cols;
  if (op == OA_R_SUM || op == OA_R_MEAN) {
    float s = 0.f;
    for (int c = lane; c < cols; c += 32) s += IO<T>::ld1(p + c);
    s = warp_sum(s);
    if (op == OA_R_MEAN) s /= (float)cols;
    if (lane == 0) IO<T>::st1(reinterpret_cast<T*>(y) + row, s);
  } else {
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int c = lane; c < cols; c += 32) {
      float v = IO<T>::ld1(p + c);
      if (v > m || (v == m && c < mi)) { m = v; mi = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, m, o);
      int oi = __shfl_xor_sync(0xffffffffu, mi, o);
      if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
    }
    if (lane == 0) {
      if (op == OA_R_MAX) IO<T>::st1(reinterpret_cast<T*>(y) + row, m);
      else reinterpret_cast<int*>(y)[row] = mi;
    }
  }
}

// Row softmax / log-softmax of (x * scale + mask), one CTA per row.
template <typename T>
__global__ void softmax_kernel(const T* __restrict__ x, T* __restrict__ y, int cols, int log_mode, float scale,
                               const T* __restrict__ mask, long long mask_rows) {
  __shared__ float red[32];
  long long row = blockIdx.x;
  const T* p = x + row * cols;
  const T* mk = mask ? mask + (row % mask_rows) * cols : nullptr;   // the mask repeats every mask_rows rows
  float m = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = IO<T>::ld1(p + c) * scale + (mk ? IO<T>::ld1(mk + c) : 0.f);
    m = fmaxf(m, v);
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
  __syncthreads();
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = IO<T>::ld1(p + c) * scale + (mk ? IO<T>::ld1(mk + c) : 0.f);
    s += expf(v - m);
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  s = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) s += red[w];
  float lse = m + logf(s);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = IO<T>::ld1(p + c) * scale + (mk ? IO<T>::ld1(mk + c) : 0.f);
    IO<T>::st1(y + row * cols + c, log_mode ? v - lse : expf(v - lse));
  }
}
// softmax: dx = scale * y * (dy - sum(dy*y));  log-softmax: dx = scale * (dy - exp(y) * sum(dy))
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, int cols,
                                   int log_mode, float scale) {
  __shared__ float red[32];
  long long row = blockIdx.x;
  const T* py = y + row * cols;
  const T* pd = dy + row * cols;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float d = IO<T>::ld1(pd + c);
    s += log_mode ? d : d * IO<T>::ld1(py + c);
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  s = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) s += red[w];
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float d = IO<T>::ld1(pd + c), yy = IO<T>::ld1(py + c);
    IO<T>::st1(dx + row * cols + c, scale * (log_mode ? d - expf(yy) * s : yy * (d - s)));
  }
}

// Philox4x32-10, key (seed, 0x87654321), counter (index + offset, 0, 0, 0); normal = Box-Muller with log(u1 + 1e-10).
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1, uint32_t* out) {
  uint32_t c[4] = {c0, c1, 0u, 0u};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}
__device__ __forceinline__ float u01(uint32_t x) { return (float)(x >> 8) * (1.0f / 16777216.0f); }

template <typename T>
__global__ void philox_kernel(T* y, long long n, unsigned long long seed, unsigned long long offset, int normal, float a,
                              float b, const unsigned long long* __restrict__ state) {
  if (state) { seed = state[0]; offset += state[1]; }     // device-resident (seed, base offset): replay-safe inside a graph
  long long stride = (long long)gridDim.x * blockDim.x;
  long long groups = (n + 3) / 4;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    unsigned long long ctr = (unsigned long long)g + offset;
    uint32_t r[4];
    philox4x32_10((uint32_t)ctr, (uint32_t)(ctr >> 32), (uint32_t)seed, 0x87654321u ^ (uint32_t)(seed >> 32), r);
    float v[4];
    if (normal) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float u1 = u01(r[2 * h]), u2 = u01(r[2 * h + 1]);
        float rad = sqrtf(-2.f * logf(u1 + 1e-10f));
        float sn, cs;
        sincosf(6.283185307179586f * u2, &sn, &cs);
        v[2 * h] = a + b * rad * cs;
        v[2 * h + 1] = a + b * rad * sn;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = a + (b - a) * u01(r[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (g * 4 + j < n) IO<T>::st1(y + g * 4 + j, v[j]);
  }
}
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float p, unsigned long long seed,
                               unsigned long long offset, const unsigned long long* __restrict__ state) {
  if (state) { seed = state[0]; offset += state[1]; }     // device-resident (seed, base offset): replay-safe inside a graph
  long long stride = (long long)gridDim.x * blockDim.x;
  long long groups = (n + 3) / 4;
  float keep_scale = 1.f / (1.f - p);
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += stride) {
    unsigned long long ctr = (unsigned long long)g + offset;
    uint32_t r[4];
    philox4x32_10((uint32_t)ctr, (uint32_t)(ctr >> 32), (uint32_t)seed, 0x87654321u ^ (uint32_t)(seed >> 32), r);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (g * 4 + j < n) {
        float keep = u01(r[j]) >= p ? keep_scale : 0.f;
        IO<T>::st1(y + g * 4 + j, IO<T>::ld1(x + g * 4 + j) * keep);
      }
  }
}

// Gather of a strided (permuted / sliced) view into a contiguous tensor, rank <= 8.
struct StridedDesc {
  long long shape[8];
  long long stride[8];
  int rank;
};
template <typename T>
__global__ void copy_strided_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, StridedDesc d) {
  long long gstride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gstride) {
    long long rem = i, off = 0;
    for (int k = d.rank - 1; k >= 0; --k) {
      long long idx = rem % d.shape[k];
      rem /= d.shape[k];
      off += idx * d.stride[k];
    }
    y[i] = x[off];
  }
}

}  // namespace oa

using namespace oa;
#define ST ((cudaStream_t)stream)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH)
#define DISPATCH_T(dtype, ...)                      \
  if ((dtype) == OA_F32) { using T = float; __VA_ARGS__; }         \
  else if ((dtype) == OA_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else return OA_ERR_UNSUPPORTED;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int oa_unary(int op, int dtype, const void* x, void* y, long long n, float s0, float s1, void* stream) {
  if (n <= 0) return OA_OK;
  if (!aligned16(x) || !aligned16(y)) return OA_ERR_ALIGN;
  DISPATCH_T(dtype, unary_kernel<T><<<grid_for(n / IO<T>::VEC + 1, 256), 256, 0, ST>>>(op, (const T*)x, (T*)y, n, s0, s1));
  return CHECK_LAUNCH();
}
extern "C" int oa_binary(int op, int dtype, const void* a, const void* b, void* y, long long n, long long inner_b,
                         int bcast_mode, void* stream) {
  if (n <= 0) return OA_OK;
  if (bcast_mode == OA_BC_NONE && (!aligned16(a) || !aligned16(b) || !aligned16(y))) return OA_ERR_ALIGN;
  long long work = bcast_mode == OA_BC_NONE ? n / 4 + 1 : n;
  // leaky-relu / elu slopes travel in `inner_b` is not possible; those backward ops use slope 0.01 / alpha 1.
  float s0 = (op == OA_B_LEAKY_RELU_BWD) ? 0.01f : 1.0f;
  DISPATCH_T(dtype, binary_kernel<T><<<grid_for(work, 256), 256, 0, ST>>>(op, (const T*)a, (const T*)b, (T*)y, n,
                                                                         inner_b > 0 ? inner_b : 1, bcast_mode, s0));
  return CHECK_LAUNCH();
}
// parts[t][i] (t < terms) = successive bf16 roundings of x[i]: x ~ sum_t parts[t], each term carrying the next 8 mantissa bits.
// Feeds the tensor-core fp32 GEMM, which multiplies the parts pairwise and accumulates in fp32.
__global__ void split_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ parts, long long n, int terms) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float r = x[i];
    for (int t = 0; t < terms; ++t) {
      const __nv_bfloat16 h = __float2bfloat16_rn(r);
      parts[(long long)t * n + i] = h;
      r -= __bfloat162float(h);
    }
  }
}

extern "C" int oa_split_bf16(const float* x, void* parts, long long n, int terms, void* stream) {
  if (n <= 0) return OA_OK;
  if (terms < 1 || terms > 3) return OA_ERR_ARG;
  split_bf16_kernel<<<grid_for(n, 256), 256, 0, ST>>>(x, (__nv_bfloat16*)parts, n, terms);
  return CHECK_LAUNCH();
}

extern "C" int oa_cast(int sd, int dd, const void* x, void* y, long long n, void* stream) {
  if (n <= 0) return OA_OK;
  int g = grid_for(n, 256);
  if (sd == OA_F32 && dd == OA_BF16) cast_kernel<float, __nv_bfloat16><<<g, 256, 0, ST>>>((const float*)x, (__nv_bfloat16*)y, n);
  else if (sd == OA_BF16 && dd == OA_F32) cast_kernel<__nv_bfloat16, float><<<g, 256, 0, ST>>>((const __nv_bfloat16*)x, (float*)y, n);
  else if (sd == OA_F32 && dd == OA_F32) cast_kernel<float, float><<<g, 256, 0, ST>>>((const float*)x, (float*)y, n);
  else if (sd == OA_BF16 && dd == OA_BF16) cast_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, ST>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}
extern "C" int oa_fill(int dtype, void* y, long long n, float value, void* stream) {
  if (n <= 0) return OA_OK;
  const int esz = dtype == OA_BF16 ? 2 : (dtype == OA_F32 ? 4 : 0);
  if (esz && n * esz >= (1 << 16) && (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
    uint32_t word;
    if (dtype == OA_BF16) {
      const __nv_bfloat16 b = __float2bfloat16(value);
      unsigned short h;
      memcpy(&h, &b, 2);
      word = (uint32_t)h | ((uint32_t)h << 16);
    } else {
      memcpy(&word, &value, 4);
    }
    const long long n16 = n * esz / 16, done = n16 * 16 / esz;
    fill_vec_kernel<<<grid_for(n16, 256), 256, 0, ST>>>((uint4*)y, n16, make_uint4(word, word, word, word));
    if (done < n) { DISPATCH_T(dtype, fill_kernel<T><<<1, 32, 0, ST>>>((T*)y + done, n - done, value)); }
    return CHECK_LAUNCH();
  }
  DISPATCH_T(dtype, fill_kernel<T><<<grid_for(n, 256), 256, 0, ST>>>((T*)y, n, value));
  return CHECK_LAUNCH();
}
extern "C" int oa_swiglu_fwd(int dtype, const void* gu, void* out, long long rows, int F, void* stream) {
  if (F % 8) return OA_ERR_ALIGN;
  DISPATCH_T(dtype, swiglu_fwd_kernel<T><<<grid_for(rows * F / IO<T>::VEC, 256), 256, 0, ST>>>((const T*)gu, (T*)out, rows, F));
  return CHECK_LAUNCH();
}
extern "C" int oa_swiglu_bwd(int dtype, const void* gu, const void* dout, void* dgu, long long rows, int F, void* stream) {
  if (F % 8) return OA_ERR_ALIGN;
  DISPATCH_T(dtype, swiglu_bwd_kernel<T><<<grid_for(rows * F / IO<T>::VEC, 256), 256, 0, ST>>>((const T*)gu, (const T*)dout, (T*)dgu, rows, F));
  return CHECK_LAUNCH();
}
extern "C" int oa_rope(int dtype, void* x, long long rows, int row_stride, int n_heads, int head_dim, int seq_len,
                       int pos_offset, float theta, int backward, const int* pos_dev, void* stream) {
  if (head_dim % 2) return OA_ERR_ARG;
  if (dtype == OA_BF16 && head_dim % 16 == 0 && row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    launch_pdl(rope_bf16_vec_kernel, dim3(grid_for(rows * (head_dim / 16), 256)), dim3(256), 0, ST, (__nv_bfloat16*)x, rows, row_stride, n_heads,
               head_dim, seq_len, pos_offset, theta, backward, pos_dev);
    return CHECK_LAUNCH();
  }
  DISPATCH_T(dtype, rope_kernel<T><<<grid_for(rows * n_heads * head_dim / 2, 256), 256, 0, ST>>>(
                        (T*)x, rows, row_stride, n_heads, head_dim, seq_len, pos_offset, theta, backward, pos_dev));
  return CHECK_LAUNCH();
}
extern "C" int oa_embedding_fwd(int dtype, const void* table, const int* ids, void* out, long long n_ids, int dim,
                                int vocab, const void* pos_table, int seq_len, void* stream) {
  if (dim % 8) return OA_ERR_ALIGN;
  DISPATCH_T(dtype, embedding_fwd_kernel<T><<<grid_for(n_ids * dim / IO<T>::VEC, 256), 256, 0, ST>>>(
                        (const T*)table, ids, (T*)out, n_ids, dim, vocab, (const T*)pos_table, seq_len > 0 ? seq_len : 1));
  return CHECK_LAUNCH();
}
extern "C" int oa_embedding_bwd(int dtype, const void* dout, const int* ids, float* dtable, long long n_ids, int dim,
                                int vocab, void* stream) {
  DISPATCH_T(dtype, embedding_bwd_kernel<T><<<grid_for(n_ids * dim, 256), 256, 0, ST>>>((const T*)dout, ids, dtable, n_ids, dim, vocab));
  return CHECK_LAUNCH();
}
// scratch: float[ceil(rows/256) * cols]
extern "C" int oa_col_sum(int dtype, const void* x, void* out, int out_dtype, long long rows, int cols, float* scratch,
                          int accumulate, void* stream) {
  const int RPB = 256;
  int nparts = (int)((rows + RPB - 1) / RPB);
  dim3 g1((cols + 127) / 128, nparts);
  DISPATCH_T(dtype, col_sum_partial_kernel<T><<<g1, dim3(128, 4), 0, ST>>>((const T*)x, scratch, rows, cols, RPB));
  if (out_dtype == OA_F32) col_sum_final_kernel<float><<<(cols + 127) / 128, 128, 0, ST>>>(scratch, (float*)out, nparts, cols, accumulate);
  else col_sum_final_kernel<__nv_bfloat16><<<(cols + 127) / 128, 128, 0, ST>>>(scratch, (__nv_bfloat16*)out, nparts, cols, accumulate);
  return CHECK_LAUNCH();
}
extern "C" int oa_bias_add(int dtype, void* x, const void* bias, long long rows, int cols, void* stream) {
  DISPATCH_T(dtype, bias_add_kernel<T><<<grid_for(rows * cols, 256), 256, 0, ST>>>((T*)x, (const T*)bias, rows, cols));
  return CHECK_LAUNCH();
}
extern "C" int oa_row_reduce(int op, int dtype, const void* x, void* y, long long rows, int cols, void* stream) {
  if (rows <= 0) return OA_OK;
  unsigned blocks = (unsigned)((rows + 7) / 8);
  DISPATCH_T(dtype, row_reduce_kernel<T><<<blocks, 256, 0, ST>>>(op, (const T*)x, y, rows, cols));
  return CHECK_LAUNCH();
}
extern "C" int oa_softmax(int dtype, const void* x, void* y, long long rows, int cols, int log_mode, float scale,
                          const void* mask, long long mask_rows, void* stream) {
  if (rows <= 0) return OA_OK;
  if (mask && mask_rows <= 0) return OA_ERR_ARG;
  int threads = cols >= 1024 ? 256 : (cols >= 128 ? 128 : 32);
  DISPATCH_T(dtype, softmax_kernel<T><<<(unsigned)rows, threads, 0, ST>>>((const T*)x, (T*)y, cols, log_mode, scale, (const T*)mask,
                                                                             mask_rows));
  return CHECK_LAUNCH();
}
extern "C" int oa_softmax_bwd(int dtype, const void* y, const void* dy, void* dx, long long rows, int cols,
                              int log_mode, float scale, void* stream) {
  if (rows <= 0) return OA_OK;
  int threads = cols >= 1024 ? 256 : (cols >= 128 ? 128 : 32);
  DISPATCH_T(dtype, softmax_bwd_kernel<T><<<(unsigned)rows, threads, 0, ST>>>((const T*)y, (const T*)dy, (T*)dx, cols, log_mode, scale));
  return CHECK_LAUNCH();
}
extern "C" int oa_philox(int dtype, void* y, long long n, unsigned long long seed, unsigned long long offset,
                         int normal, float a, float b, const unsigned long long* state, void* stream) {
  if (n <= 0) return OA_OK;
  DISPATCH_T(dtype, philox_kernel<T><<<grid_for((n + 3) / 4, 256), 256, 0, ST>>>((T*)y, n, seed, offset, normal, a, b, state));
  return CHECK_LAUNCH();
}
extern "C" int oa_dropout(int dtype, const void* x, void* y, long long n, float p, unsigned long long seed,
                          unsigned long long offset, const unsigned long long* state, void* stream) {
  if (n <= 0) return OA_OK;
  DISPATCH_T(dtype, dropout_kernel<T><<<grid_for((n + 3) / 4, 256), 256, 0, ST>>>((const T*)x, (T*)y, n, p, seed, offset, state));
  return CHECK_LAUNCH();
}
// state[1] += delta: closes a captured step, so that every replay draws the counters the eager step would have drawn
// (the reference's PhiloxGraphAdvance, Source/Private/Oa/Core/Shader/Compute/Rng/PhiloxGraphAdvance.slang).
__global__ void philox_state_advance_kernel(unsigned long long* state, unsigned long long delta) {
  if (threadIdx.x == 0 && blockIdx.x == 0) state[1] += delta;
}
extern "C" int oa_philox_state_advance(unsigned long long* state, unsigned long long delta, void* stream) {
  philox_state_advance_kernel<<<1, 32, 0, ST>>>(state, delta);
  return CHECK_LAUNCH();
}
extern "C" int oa_copy_strided(int dtype, const void* x, void* y, int rank, const long long* shape,
                               const long long* src_strides, void* stream) {
  if (rank < 1 || rank > 8) return OA_ERR_ARG;
  StridedDesc d;
  d.rank = rank;
  long long n = 1;
  for (int i = 0; i < rank; ++i) { d.shape[i] = shape[i]; d.stride[i] = src_strides[i]; n *= shape[i]; }
  if (n <= 0) return OA_OK;
  if (dtype == OA_F32) copy_strided_kernel<float><<<grid_for(n, 256), 256, 0, ST>>>((const float*)x, (float*)y, n, d);
  else if (dtype == OA_BF16) copy_strided_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, ST>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, d);
  else if (dtype == 4 /* int32 */) copy_strided_kernel<int><<<grid_for(n, 256), 256, 0, ST>>>((const int*)x, (int*)y, n, d);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}
