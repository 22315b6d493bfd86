// Elementwise / reduction kernels around the batched GEMMs of the chunked (state-space-duality) Mamba-3 scan.
//
// Per (batch b, head h, chunk c) - index g = (b*H + h)*nC + c, Q = 128 tokens per chunk - the scan is
//   G = C~ B~^T,  M = mask(G),  Y = M X + (C~ e^cum) Hin^T,  S = (w.X)^T B~,  h_{c+1} = e^{cumQ} h_c + S
// (ops/mamba3_ssd.py states the algebra and its backward).  The GEMMs run on the tcgen05 batched GEMM; this file holds
// everything in between, each kernel making exactly one pass over its operands:
//   ssd_prep_fwd    per-token scalars (cum, gamma, scale, w), rotated C~ / B~ / C~e^cum in bf16 chunk layout, q.k, X, w.X
//   ssd_mask_fwd    G (fp32) -> M (bf16): decayed strict lower triangle + exact diagonal
//   ssd_state_fwd   recurrence over the chunk states, emits the state entering every chunk
//   ssd_out_fwd     Y (fp32 chunk layout) -> y (token layout) with the silu(z) gate
//   ssd_dy_prep     dy -> dY (bf16 chunk layout) through the gate, dz
//   ssd_state_bwd   reverse recurrence: gradient w.r.t. every chunk's outgoing state and w.r.t. cumQ
//   ssd_mask_bwd    dM, G -> dG (bf16) + row / column sums that carry d cum, d scale, d gamma, d D
//   ssd_prep_bwd    dC~, dB~, d(C~e^cum) -> un-rotate, d theta, dCn / dBn (summed over heads), dCb / dBb
//   ssd_dx_out      dX + w.dXw -> dx in the projection gradient, dw
// All tensors are contiguous; chunk-layout tensors are [G, Q, *].
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr int SQ = 128;           // tokens per chunk

struct SsdDims {
  int B, L, H, P, N, A, nC;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------------------------------------------ forward prep
struct SsdPrepFwd {
  const __nv_bfloat16* x; long long ldx;          // x columns of the projection: x[row*ldx + h*P + p]
  const float *Bn, *Cn, *Bb, *Cb;                 // [B*L, N], [H, N]
  const float *dt, *adt, *trap;                   // [B*L, H]
  const float* theta;                             // [B*L, H, A] (range reduced), null when A == 0
  __nv_bfloat16 *Ct, *Bt, *Ce, *X, *Xw;           // chunk layout outputs
  float *cum, *gamma, *scale, *w, *qk;            // [G, Q]
  SsdDims d;
};

__global__ void __launch_bounds__(256) ssd_prep_fwd_kernel(SsdPrepFwd a) {
  const SsdDims& d = a.d;
  const int g = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = g % d.nC, bh = g / d.nC, h = bh % d.H, b = bh / d.H;
  const long long row0 = (long long)b * d.L + (long long)c * SQ;
  __shared__ float s_adt[SQ], s_cum[SQ], s_w[SQ], s_ecum[SQ];
  if (tid < SQ) s_adt[tid] = a.adt[(row0 + tid) * d.H + h];
  __syncthreads();
  if (warp == 0) {                                 // inclusive scan of 128 values: 4 per lane + warp scan
    float v0 = s_adt[lane * 4], v1 = v0 + s_adt[lane * 4 + 1], v2 = v1 + s_adt[lane * 4 + 2], v3 = v2 + s_adt[lane * 4 + 3];
    float tot = v3;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const float n = __shfl_up_sync(0xffffffffu, tot, o); if (lane >= o) tot += n; }
    const float base = tot - v3;
    s_cum[lane * 4] = base + v0; s_cum[lane * 4 + 1] = base + v1; s_cum[lane * 4 + 2] = base + v2; s_cum[lane * 4 + 3] = base + v3;
  }
  __syncthreads();
  if (tid < SQ) {
    const long long r = row0 + tid;
    const int l = c * SQ + tid;
    const float dtv = a.dt[r * d.H + h], tr = sigmoidf_(a.trap[r * d.H + h]);
    const float gam = dtv * tr;
    float late_next = 0.f;
    if (l + 1 < d.L) late_next = a.dt[(r + 1) * d.H + h] * (1.f - sigmoidf_(a.trap[(r + 1) * d.H + h]));
    const float sc = gam + late_next, cm = s_cum[tid];
    const float wv = __expf(s_cum[SQ - 1] - cm) * sc;
    const long long o = (long long)g * SQ + tid;
    a.cum[o] = cm; a.gamma[o] = gam; a.scale[o] = sc; a.w[o] = wv;
    s_w[tid] = wv; s_ecum[tid] = __expf(cm);
  }
  __syncthreads();
  const int N4 = d.N >> 2, P2 = d.P >> 1;
  for (int t = warp; t < SQ; t += 8) {
    const long long r = row0 + t;
    const long long og = (long long)g * SQ + t;
    float qk = 0.f;
    for (int n4 = lane; n4 < N4; n4 += 32) {
      float4 cv = reinterpret_cast<const float4*>(a.Cn + r * d.N)[n4];
      float4 bv = reinterpret_cast<const float4*>(a.Bn + r * d.N)[n4];
      const float4 cb = reinterpret_cast<const float4*>(a.Cb + (long long)h * d.N)[n4];
      const float4 bb = reinterpret_cast<const float4*>(a.Bb + (long long)h * d.N)[n4];
      cv.x += cb.x; cv.y += cb.y; cv.z += cb.z; cv.w += cb.w;
      bv.x += bb.x; bv.y += bb.y; bv.z += bb.z; bv.w += bb.w;
      const int k0 = n4 * 2;                                   // pair indices k0, k0 + 1
      if (k0 < d.A) {
        const float* th = a.theta + (r * d.H + h) * d.A;
        float sn, cs;
        sincosf(th[k0], &sn, &cs);
        float t0 = cv.x * cs - cv.y * sn, t1 = cv.x * sn + cv.y * cs; cv.x = t0; cv.y = t1;
        t0 = bv.x * cs - bv.y * sn; t1 = bv.x * sn + bv.y * cs; bv.x = t0; bv.y = t1;
        if (k0 + 1 < d.A) {
          sincosf(th[k0 + 1], &sn, &cs);
          t0 = cv.z * cs - cv.w * sn; t1 = cv.z * sn + cv.w * cs; cv.z = t0; cv.w = t1;
          t0 = bv.z * cs - bv.w * sn; t1 = bv.z * sn + bv.w * cs; bv.z = t0; bv.w = t1;
        }
      }
      qk += cv.x * bv.x + cv.y * bv.y + cv.z * bv.z + cv.w * bv.w;
      const float e = s_ecum[t];
      const long long o = og * d.N + n4 * 4;
      *reinterpret_cast<uint2*>(a.Ct + o) = make_uint2(pack_bf16x2(cv.x, cv.y), pack_bf16x2(cv.z, cv.w));
      *reinterpret_cast<uint2*>(a.Bt + o) = make_uint2(pack_bf16x2(bv.x, bv.y), pack_bf16x2(bv.z, bv.w));
      *reinterpret_cast<uint2*>(a.Ce + o) = make_uint2(pack_bf16x2(cv.x * e, cv.y * e), pack_bf16x2(cv.z * e, cv.w * e));
    }
    qk = warp_sum(qk);
    if (lane == 0) a.qk[og] = qk;
    const float wv = s_w[t];
    for (int p2 = lane; p2 < P2; p2 += 32) {
      const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(a.x + r * a.ldx + (long long)h * d.P + p2 * 2);
      const float2 xf = __bfloat1622float2(xv);
      const long long o = og * d.P + p2 * 2;
      *reinterpret_cast<__nv_bfloat162*>(a.X + o) = xv;
      *reinterpret_cast<unsigned*>(a.Xw + o) = pack_bf16x2(xf.x * wv, xf.y * wv);
    }
  }
}

// ------------------------------------------------------------------------------------------------------- mask forward
// M[t,s] = G[t,s] e^{cum_t - cum_s} scale_s (s < t);  M[t,t] = D + gamma_t qk_t;  0 above the diagonal.
__global__ void __launch_bounds__(256) ssd_mask_fwd_kernel(const float* __restrict__ Gm, const float* __restrict__ cum,
                                                           const float* __restrict__ scale, const float* __restrict__ gamma,
                                                           const float* __restrict__ qk, const float* __restrict__ Dh,
                                                           __nv_bfloat16* __restrict__ M, int H, int nC) {
  const int g = blockIdx.x, tid = threadIdx.x;
  const int h = (g / nC) % H;
  __shared__ float s_cum[SQ], s_scale[SQ], s_diag[SQ];
  if (tid < SQ) {
    const long long o = (long long)g * SQ + tid;
    s_cum[tid] = cum[o]; s_scale[tid] = scale[o];
    s_diag[tid] = (Dh ? Dh[h] : 0.f) + gamma[o] * qk[o];
  }
  __syncthreads();
  const float* Gg = Gm + (long long)g * SQ * SQ;
  __nv_bfloat16* Mg = M + (long long)g * SQ * SQ;
  for (int i = tid; i < SQ * SQ / 8; i += 256) {
    const int t = i >> 4, s0 = (i & 15) * 8;
    unsigned out[4];
    if (s0 > t) {
      out[0] = out[1] = out[2] = out[3] = 0u;
    } else {
      const float4 g0 = *reinterpret_cast<const float4*>(Gg + t * SQ + s0);
      const float4 g1 = *reinterpret_cast<const float4*>(Gg + t * SQ + s0 + 4);
      const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      float v[8];
      const float ct = s_cum[t];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int s = s0 + j;
        v[j] = s < t ? gv[j] * __expf(ct - s_cum[s]) * s_scale[s] : (s == t ? s_diag[t] : 0.f);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) out[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    }
    *reinterpret_cast<uint4*>(Mg + t * SQ + s0) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

// ------------------------------------------------------------------------------------------------ chunk-state recurrence
// forward: Hin[c] = h; h = e^{cumQ_c} h + S[c].   One thread per (b*H + h, element of the P x N state).
__global__ void __launch_bounds__(256) ssd_state_fwd_kernel(const float* __restrict__ S, const float* __restrict__ cum,
                                                            __nv_bfloat16* __restrict__ Hin, int nC, int PN) {
  const int bh = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= PN) return;
  float hst = 0.f;
  for (int c = 0; c < nC; ++c) {
    const long long g = (long long)bh * nC + c;
    Hin[g * PN + e] = __float2bfloat16_rn(hst);
    hst = __expf(cum[g * SQ + SQ - 1]) * hst + S[g * PN + e];
  }
}

// backward: dHout[c] = gr; dcumQ[c] += sum_e gr Hin[c] e^{cumQ_c}; gr = e^{cumQ_c} gr + T[c]
__global__ void __launch_bounds__(256) ssd_state_bwd_kernel(const float* __restrict__ T, const float* __restrict__ cum,
                                                            const __nv_bfloat16* __restrict__ Hin, __nv_bfloat16* __restrict__ dHout,
                                                            float* __restrict__ dcumQ, int nC, int PN) {
  const int bh = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = e < PN;
  float gr = 0.f;
  for (int c = nC - 1; c >= 0; --c) {
    const long long g = (long long)bh * nC + c;
    const float dec = __expf(cum[g * SQ + SQ - 1]);
    float part = 0.f;
    if (live) {
      dHout[g * PN + e] = __float2bfloat16_rn(gr);
      part = gr * __bfloat162float(Hin[g * PN + e]) * dec;
      gr = dec * gr + T[g * PN + e];
    }
    part = warp_sum(part);
    if ((threadIdx.x & 31) == 0 && part != 0.f) atomicAdd(dcumQ + g, part);
  }
}

// ------------------------------------------------------------------------------------------------------ output / gate
// Y [G, Q, P] fp32 -> y [rows, ldy] (bf16) = Y * silu(z); yraw (bf16, same layout as y) keeps Y for the backward pass.
__global__ void __launch_bounds__(256) ssd_out_fwd_kernel(const float* __restrict__ Y, const __nv_bfloat16* __restrict__ z, long long ldz,
                                                          __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ yraw, long long ldy,
                                                          SsdDims d) {
  const int P2 = d.P >> 1;
  const long long total = (long long)d.B * d.H * d.nC * SQ * P2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p2 = (int)(i % P2);
    long long r = i / P2;
    const int t = (int)(r % SQ); r /= SQ;
    const int c = (int)(r % d.nC); r /= d.nC;
    const int h = (int)(r % d.H), b = (int)(r / d.H);
    const long long row = (long long)b * d.L + (long long)c * SQ + t;
    const float2 v = *reinterpret_cast<const float2*>(Y + i * 2);
    const long long o = row * ldy + (long long)h * d.P + p2 * 2;
    if (z) {
      const float2 zf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(z + row * ldz + (long long)h * d.P + p2 * 2));
      *reinterpret_cast<unsigned*>(yraw + o) = pack_bf16x2(v.x, v.y);
      *reinterpret_cast<unsigned*>(y + o) = pack_bf16x2(v.x * zf.x * sigmoidf_(zf.x), v.y * zf.y * sigmoidf_(zf.y));
    } else {
      *reinterpret_cast<unsigned*>(y + o) = pack_bf16x2(v.x, v.y);
    }
  }
}

// dy [rows, ldy] -> dY [G, Q, P] bf16 through the gate; dz = dy * Yraw * sigmoid(z) (1 + z (1 - sigmoid(z)))
__global__ void __launch_bounds__(256) ssd_dy_prep_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ yraw,
                                                          long long ldy, const __nv_bfloat16* __restrict__ z, long long ldz,
                                                          __nv_bfloat16* __restrict__ dz, long long lddz, __nv_bfloat16* __restrict__ dY,
                                                          SsdDims d) {
  const int P2 = d.P >> 1;
  const long long total = (long long)d.B * d.H * d.nC * SQ * P2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p2 = (int)(i % P2);
    long long r = i / P2;
    const int t = (int)(r % SQ); r /= SQ;
    const int c = (int)(r % d.nC); r /= d.nC;
    const int h = (int)(r % d.H), b = (int)(r / d.H);
    const long long row = (long long)b * d.L + (long long)c * SQ + t;
    const long long col = (long long)h * d.P + p2 * 2;
    float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dy + row * ldy + col));
    if (z) {
      const float2 zf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(z + row * ldz + col));
      const float2 yr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(yraw + row * ldy + col));
      const float s0 = sigmoidf_(zf.x), s1 = sigmoidf_(zf.y);
      *reinterpret_cast<unsigned*>(dz + row * lddz + col) =
          pack_bf16x2(g.x * yr.x * s0 * (1.f + zf.x * (1.f - s0)), g.y * yr.y * s1 * (1.f + zf.y * (1.f - s1)));
      g.x *= zf.x * s0; g.y *= zf.y * s1;
    }
    *reinterpret_cast<unsigned*>(dY + i * 2) = pack_bf16x2(g.x, g.y);
  }
}

// ------------------------------------------------------------------------------------------------------ mask backward
// Per chunk, with L = strict lower triangle:  dG = dM e^{..} scale (on L);  dMM = dM * M (on L)
//   row_mm[t] = sum_s dMM;  col_mm[s] = sum_t dMM;  col_ge[s] = sum_t dM G e^{..} (on L);  diag[t] = dM[t,t]
// Warp w owns rows w, w+8, ...; lane owns columns 4*lane .. 4*lane+3: row sums are warp reductions, column sums stay in
// registers over the warp's 16 rows and are combined across the 8 warps through 8 KB of shared memory.
__global__ void __launch_bounds__(256) ssd_mask_bwd_kernel(const float* __restrict__ dM, const float* __restrict__ Gm,
                                                           const float* __restrict__ cum, const float* __restrict__ scale,
                                                           __nv_bfloat16* __restrict__ dG, float* __restrict__ row_mm,
                                                           float* __restrict__ col_mm, float* __restrict__ col_ge,
                                                           float* __restrict__ diag) {
  __shared__ float s_cum[SQ], s_scale[SQ];
  __shared__ float s_cm[8][SQ], s_cg[8][SQ];
  const int g = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < SQ) { s_cum[tid] = cum[(long long)g * SQ + tid]; s_scale[tid] = scale[(long long)g * SQ + tid]; }
  __syncthreads();
  const float* dMg = dM + (long long)g * SQ * SQ;
  const float* Gg = Gm + (long long)g * SQ * SQ;
  __nv_bfloat16* dGg = dG + (long long)g * SQ * SQ;
  const int s0 = lane * 4;
  float cs[4], sc[4], cmm[4] = {0.f, 0.f, 0.f, 0.f}, cge[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) { cs[j] = s_cum[s0 + j]; sc[j] = s_scale[s0 + j]; }
  for (int t = warp; t < SQ; t += 8) {
    float o[4] = {0.f, 0.f, 0.f, 0.f}, rsum = 0.f;
    if (s0 <= t) {
      const float4 dm = *reinterpret_cast<const float4*>(dMg + t * SQ + s0);
      const float4 gg = *reinterpret_cast<const float4*>(Gg + t * SQ + s0);
      const float dmv[4] = {dm.x, dm.y, dm.z, dm.w}, gv[4] = {gg.x, gg.y, gg.z, gg.w};
      const float ct = s_cum[t];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int sidx = s0 + j;
        if (sidx < t) {
          const float e = __expf(ct - cs[j]);
          o[j] = dmv[j] * e * sc[j];
          const float ge = dmv[j] * gv[j] * e, mm = ge * sc[j];
          cge[j] += ge; cmm[j] += mm; rsum += mm;
        } else if (sidx == t) {
          diag[(long long)g * SQ + t] = dmv[j];
        }
      }
    }
    *reinterpret_cast<uint2*>(dGg + t * SQ + s0) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
    rsum = warp_sum(rsum);
    if (lane == 0) row_mm[(long long)g * SQ + t] = rsum;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) { s_cm[warp][s0 + j] = cmm[j]; s_cg[warp][s0 + j] = cge[j]; }
  __syncthreads();
  if (tid < SQ) {
    float a = 0.f, b2 = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) { a += s_cm[w8][tid]; b2 += s_cg[w8][tid]; }
    col_mm[(long long)g * SQ + tid] = a; col_ge[(long long)g * SQ + tid] = b2;
  }
}

// ------------------------------------------------------------------------------------------------------ prep backward
struct SsdPrepBwd {
  const float *dCt, *dBt, *dCe;                  // [G, Q, N] fp32 (GEMM outputs)
  const __nv_bfloat16 *Ct, *Bt;                  // saved rotated operands
  const float *cum, *dqk;                        // [G, Q]
  const float* theta;                            // [B*L, H, A]
  float *dCn, *dBn;                              // [B*L, N]  (summed over heads; stored, not accumulated)
  float *dCb, *dBb;                              // [H, N]    (atomic: summed over batch and time)
  float* dtheta;                                 // [B*L, H, A]
  float* dcum_ce;                                // [G, Q]  sum_n dCe C~ e^cum
  SsdDims d;
};

// One CTA owns 32 token rows of a chunk for ALL heads: the sums over heads (dCn, dBn) stay in registers and are stored once,
// without atomics.  Warp w owns rows w, w+8, w+16, w+24 of the 32; lane owns state columns 4*lane .. 4*lane+3 (N <= 128).
__global__ void __launch_bounds__(256) ssd_prep_bwd_kernel(SsdPrepBwd a) {
  const SsdDims& d = a.d;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = blockIdx.x & 3, bc = blockIdx.x >> 2, c = bc % d.nC, b = bc / d.nC;
  const long long row0 = (long long)b * d.L + (long long)c * SQ;
  const int N4 = d.N >> 2;
  const bool live = lane < N4;
  __shared__ float s_cb[8][SQ], s_bb[8][SQ];         // per-warp bias partials of the current head
  float accC[4][4], accB[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { accC[i][j] = 0.f; accB[i][j] = 0.f; }
  for (int h = 0; h < d.H; ++h) {
    const long long g = ((long long)b * d.H + h) * d.nC + c;
    float pc[4] = {0.f, 0.f, 0.f, 0.f}, pb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = q4 * 32 + warp + 8 * i;
      const long long r = row0 + t, og = g * SQ + t;
      const float ecum = __expf(a.cum[og]), dqk = a.dqk[og];
      float dce = 0.f;
      if (live) {
        const long long o = og * d.N + lane * 4;
        const float4 dc = *reinterpret_cast<const float4*>(a.dCt + o), db = *reinterpret_cast<const float4*>(a.dBt + o);
        const float4 de = *reinterpret_cast<const float4*>(a.dCe + o);
        const uint2 cu = *reinterpret_cast<const uint2*>(a.Ct + o), bu = *reinterpret_cast<const uint2*>(a.Bt + o);
        const float2 c01 = unpack_bf16x2(cu.x), c23 = unpack_bf16x2(cu.y), b01 = unpack_bf16x2(bu.x), b23 = unpack_bf16x2(bu.y);
        const float cv[4] = {c01.x, c01.y, c23.x, c23.y}, bv[4] = {b01.x, b01.y, b23.x, b23.y};
        const float dev[4] = {de.x, de.y, de.z, de.w};
        float gc[4] = {dc.x, dc.y, dc.z, dc.w}, gb[4] = {db.x, db.y, db.z, db.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          dce += dev[j] * cv[j];
          gc[j] += dev[j] * ecum + dqk * bv[j];
          gb[j] += dqk * cv[j];
        }
        const int k0 = lane * 2;
        if (k0 < d.A) {
          const float* th = a.theta + (r * d.H + h) * d.A;
          float* dth = a.dtheta + (r * d.H + h) * d.A;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            if (k0 + q < d.A) {
              float sn, cs;
              sincosf(th[k0 + q], &sn, &cs);
              const int j = 2 * q;
              dth[k0 + q] = (-gc[j] * cv[j + 1] + gc[j + 1] * cv[j]) + (-gb[j] * bv[j + 1] + gb[j + 1] * bv[j]);
              float u0 = gc[j] * cs + gc[j + 1] * sn, u1 = -gc[j] * sn + gc[j + 1] * cs; gc[j] = u0; gc[j + 1] = u1;
              u0 = gb[j] * cs + gb[j + 1] * sn; u1 = -gb[j] * sn + gb[j + 1] * cs; gb[j] = u0; gb[j + 1] = u1;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) { accC[i][j] += gc[j]; accB[i][j] += gb[j]; pc[j] += gc[j]; pb[j] += gb[j]; }
      }
      dce = warp_sum(dce);
      if (lane == 0) a.dcum_ce[og] = dce * ecum;
    }
    if (live) {
#pragma unroll
      for (int j = 0; j < 4; ++j) { s_cb[warp][lane * 4 + j] = pc[j]; s_bb[warp][lane * 4 + j] = pb[j]; }
    }
    __syncthreads();
    if (tid < d.N) {
      float sc = 0.f, sb = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) { sc += s_cb[w8][tid]; sb += s_bb[w8][tid]; }
      atomicAdd(a.dCb + (long long)h * d.N + tid, sc);
      atomicAdd(a.dBb + (long long)h * d.N + tid, sb);
    }
    __syncthreads();
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long r = row0 + q4 * 32 + warp + 8 * i;
      *reinterpret_cast<float4*>(a.dCn + r * d.N + lane * 4) = make_float4(accC[i][0], accC[i][1], accC[i][2], accC[i][3]);
      *reinterpret_cast<float4*>(a.dBn + r * d.N + lane * 4) = make_float4(accB[i][0], accB[i][1], accB[i][2], accB[i][3]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------- dx out
// dx[row, h*P + p] = dX + w_t dXw (bf16 into the projection gradient);  dw[g,t] = sum_p dXw X
__global__ void __launch_bounds__(256) ssd_dx_out_kernel(const float* __restrict__ dX, const float* __restrict__ dXw,
                                                         const __nv_bfloat16* __restrict__ X, const float* __restrict__ w,
                                                         __nv_bfloat16* __restrict__ dx, long long lddx, float* __restrict__ dw,
                                                         SsdDims d) {
  const int g = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = g % d.nC, bh = g / d.nC, h = bh % d.H, b = bh / d.H;
  const long long row0 = (long long)b * d.L + (long long)c * SQ;
  const int P2 = d.P >> 1;
  for (int t = warp; t < SQ; t += 8) {
    const long long og = (long long)g * SQ + t;
    const float wv = w[og];
    float acc = 0.f;
    for (int p2 = lane; p2 < P2; p2 += 32) {
      const long long o = og * d.P + p2 * 2;
      const float2 a = *reinterpret_cast<const float2*>(dX + o), bw = *reinterpret_cast<const float2*>(dXw + o);
      const float2 xf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(X + o));
      acc += bw.x * xf.x + bw.y * xf.y;
      *reinterpret_cast<unsigned*>(dx + (row0 + t) * lddx + (long long)h * d.P + p2 * 2) = pack_bf16x2(a.x + bw.x * wv, a.y + bw.y * wv);
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[og] = acc;
  }
}

// ------------------------------------------------------------------------------------------------ rotary phase scans
// theta[b,l,h,a] = sum_{l' <= l} angle[b,l',a] dt[b,l',h], reduced to (-pi, pi].  Two passes over chunks of 128 tokens:
// pass 0 writes the per-chunk totals, pass 1 adds the totals of the earlier chunks and writes the running sum.  One warp
// per (b, chunk, h), lanes over a.  The backward kernel is the mirror image: suffix sums g of dtheta, folded straight into
// d angle[b,l,a] += sum_h g dt and d dt[b,l,h] = sum_a g angle (the suffix sums themselves are never stored).
__global__ void __launch_bounds__(256) ssd_theta_fwd_kernel(const float* __restrict__ angle, int lda, const float* __restrict__ dt,
                                                            float* __restrict__ tot, float* __restrict__ theta, SsdDims d, int pass) {
  const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (wid >= d.B * d.nC * d.H) return;
  const int h = wid % d.H, c = (wid / d.H) % d.nC, b = wid / (d.H * d.nC);
  const long long row0 = (long long)b * d.L + (long long)c * SQ;
  for (int a = lane; a < d.A; a += 32) {
    float run = 0.f;
    if (pass == 1)
      for (int cp = 0; cp < c; ++cp) run += tot[(((long long)b * d.nC + cp) * d.H + h) * d.A + a];
    for (int t = 0; t < SQ; ++t) {
      const long long r = row0 + t;
      run += angle[r * lda + a] * dt[r * d.H + h];
      if (pass == 1) theta[(r * d.H + h) * d.A + a] = run - 6.283185307179586f * rintf(run * 0.15915494309189535f);
    }
    if (pass == 0) tot[(((long long)b * d.nC + c) * d.H + h) * d.A + a] = run;
  }
}

__global__ void __launch_bounds__(256) ssd_theta_bwd_kernel(const float* __restrict__ dtheta, const float* __restrict__ angle, int lda,
                                                            const float* __restrict__ dt, float* __restrict__ tot,
                                                            float* __restrict__ dangle, float* __restrict__ ddt, SsdDims d, int pass) {
  const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (wid >= d.B * d.nC * d.H) return;
  const int h = wid % d.H, c = (wid / d.H) % d.nC, b = wid / (d.H * d.nC);
  const long long row0 = (long long)b * d.L + (long long)c * SQ;
  if (pass == 0) {
    for (int a = lane; a < d.A; a += 32) {
      float run = 0.f;
      for (int t = 0; t < SQ; ++t) run += dtheta[((row0 + t) * d.H + h) * d.A + a];
      tot[(((long long)b * d.nC + c) * d.H + h) * d.A + a] = run;
    }
    return;
  }
  // A <= 32 * 4 supported: each lane carries up to 4 running suffix sums
  float run[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int a = lane + 32 * q;
    if (a < d.A)
      for (int cp = c + 1; cp < d.nC; ++cp) run[q] += tot[(((long long)b * d.nC + cp) * d.H + h) * d.A + a];
  }
  for (int t = SQ - 1; t >= 0; --t) {
    const long long r = row0 + t;
    const float dtv = dt[r * d.H + h];
    float acc = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int a = lane + 32 * q;
      if (a < d.A) {
        run[q] += dtheta[(r * d.H + h) * d.A + a];
        atomicAdd(dangle + r * lda + a, run[q] * dtv);
        acc += run[q] * angle[r * lda + a];
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) ddt[r * d.H + h] = acc;
  }
}

// ---- the per-token scalar tail of the backward pass, three small kernels over [G, Q] / [B, L, H] sized tensors.
// (1) per chunk: gradient of the decay prefix sums (a suffix sum inside the chunk), of gamma and of scale, written in token
//     order [B, L, H]; (2) per token: dt and trap gradients (scale_l looks one token ahead, so token l also receives from
//     token l - 1); (3) per head: the skip gradient, summed over batch and chunks in a fixed order.
__global__ void __launch_bounds__(SQ)
ssd_tail_chunk_kernel(const float* __restrict__ dw, const float* __restrict__ w, const float* __restrict__ col_ge,
                      const float* __restrict__ row_mm, const float* __restrict__ col_mm, const float* __restrict__ dcum_ce,
                      const float* __restrict__ diag, const float* __restrict__ qk, const float* __restrict__ cum,
                      const float* __restrict__ dcumQ, float* __restrict__ dadt, float* __restrict__ dgam, float* __restrict__ dscale_l,
                      float* __restrict__ dpart, int B, int L, int H, int nC) {
  __shared__ float sm[SQ];
  __shared__ float s_tot[2];
  const int g = blockIdx.x, q = threadIdx.x;
  const long long i = (long long)g * SQ + q;
  const float cq = cum[i], cQ = cum[(long long)g * SQ + SQ - 1];
  const float dww = dw[i] * w[i];
  const float dsc = col_ge[i] + dw[i] * __expf(cQ - cq);
  float dc = row_mm[i] - col_mm[i] + dcum_ce[i] - dww;
  const float dg = diag[i];
  // block sums of dww and of diag (fixed tree order)
  float a = warp_sum(dww), b = warp_sum(dg);
  if ((q & 31) == 0) { sm[q >> 5] = a; sm[4 + (q >> 5)] = b; }
  __syncthreads();
  if (q == 0) { s_tot[0] = (sm[0] + sm[1]) + (sm[2] + sm[3]); s_tot[1] = (sm[4] + sm[5]) + (sm[6] + sm[7]); }
  __syncthreads();
  if (q == SQ - 1) dc += dcumQ[g] + s_tot[0];
  // inclusive suffix sum over the chunk: cum is an inclusive prefix sum of a * dt
  __syncthreads();
  sm[q] = dc;
  __syncthreads();
  for (int off = 1; off < SQ; off <<= 1) {
    const float add = (q + off < SQ) ? sm[q + off] : 0.f;
    __syncthreads();
    sm[q] += add;
    __syncthreads();
  }
  const int c = g % nC, h = (g / nC) % H, bb = g / (nC * H);
  const long long o = ((long long)bb * L + c * SQ + q) * H + h;
  dadt[o] = sm[q];
  dgam[o] = dg * qk[i] + dsc;
  dscale_l[o] = dsc;
  if (q == 0 && dpart) dpart[g] = s_tot[1];
}

__global__ void ssd_tail_token_kernel(const float* __restrict__ dgam, const float* __restrict__ dscale_l, const float* __restrict__ dt,
                                      const float* __restrict__ trap, const float* __restrict__ ddt_theta, float* __restrict__ ddt,
                                      float* __restrict__ dtrap, int B, int L, int H) {
  const long long total = (long long)B * L * H;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int l = (int)((i / H) % L);
    const float tr = sigmoid_f(trap[i]), dti = dt[i];
    float a = (ddt_theta ? ddt_theta[i] : 0.f) + dgam[i] * tr;
    float t = dgam[i] * dti;
    if (l > 0) {
      const float prev = dscale_l[i - H];
      a += prev * (1.f - tr);
      t -= prev * dti;
    }
    ddt[i] = a;
    dtrap[i] = t * tr * (1.f - tr);
  }
}

__global__ void ssd_tail_skip_kernel(const float* __restrict__ dpart, float* __restrict__ dD, int B, int H, int nC) {
  const int h = blockIdx.x;
  float s = 0.f;
  for (int k = threadIdx.x; k < B * nC; k += 32) s += dpart[((long long)(k / nC) * H + h) * nC + (k % nC)];
  s = warp_sum(s);
  if (threadIdx.x == 0) dD[h] = s;
}

inline bool ssd_dims_ok(const SsdDims& d) {
  return d.B > 0 && d.L > 0 && d.H > 0 && d.P > 0 && d.N > 0 && d.A >= 0 && d.L % SQ == 0 && d.nC == d.L / SQ && d.N % 4 == 0 && d.P % 2 == 0 &&
         2 * d.A <= d.N;
}
inline int ssd_status() { return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH; }

}  // namespace oa

using namespace oa;

extern "C" {

int oa_ssd_prep_fwd(const void* x, long long ldx, const void* Bn, const void* Cn, const void* Bb, const void* Cb, const void* dt,
                    const void* adt, const void* trap, const void* theta, void* Ct, void* Bt, void* Ce, void* X, void* Xw, void* cum,
                    void* gamma, void* scale, void* w, void* qk, int B, int L, int H, int P, int N, int A, void* stream) {
  SsdDims d{B, L, H, P, N, A, L / SQ};
  if (!ssd_dims_ok(d) || (A > 0 && !theta)) return OA_ERR_ARG;
  SsdPrepFwd a{(const __nv_bfloat16*)x, ldx, (const float*)Bn, (const float*)Cn, (const float*)Bb, (const float*)Cb, (const float*)dt,
               (const float*)adt, (const float*)trap, (const float*)theta, (__nv_bfloat16*)Ct, (__nv_bfloat16*)Bt, (__nv_bfloat16*)Ce,
               (__nv_bfloat16*)X, (__nv_bfloat16*)Xw, (float*)cum, (float*)gamma, (float*)scale, (float*)w, (float*)qk, d};
  ssd_prep_fwd_kernel<<<B * H * d.nC, 256, 0, (cudaStream_t)stream>>>(a);
  return ssd_status();
}

int oa_ssd_mask_fwd(const void* Gm, const void* cum, const void* scale, const void* gamma, const void* qk, const void* Dh, void* M,
                    int G, int H, int nC, void* stream) {
  if (G <= 0) return OA_ERR_ARG;
  ssd_mask_fwd_kernel<<<G, 256, 0, (cudaStream_t)stream>>>((const float*)Gm, (const float*)cum, (const float*)scale, (const float*)gamma,
                                                           (const float*)qk, (const float*)Dh, (__nv_bfloat16*)M, H, nC);
  return ssd_status();
}

int oa_ssd_state_fwd(const void* S, const void* cum, void* Hin, int BH, int nC, int PN, void* stream) {
  if (BH <= 0 || nC <= 0 || PN <= 0) return OA_ERR_ARG;
  ssd_state_fwd_kernel<<<dim3((PN + 255) / 256, BH), 256, 0, (cudaStream_t)stream>>>((const float*)S, (const float*)cum,
                                                                                      (__nv_bfloat16*)Hin, nC, PN);
  return ssd_status();
}

int oa_ssd_state_bwd(const void* T, const void* cum, const void* Hin, void* dHout, void* dcumQ, int BH, int nC, int PN, void* stream) {
  if (BH <= 0 || nC <= 0 || PN <= 0) return OA_ERR_ARG;
  ssd_state_bwd_kernel<<<dim3((PN + 255) / 256, BH), 256, 0, (cudaStream_t)stream>>>((const float*)T, (const float*)cum,
                                                                                      (const __nv_bfloat16*)Hin, (__nv_bfloat16*)dHout,
                                                                                      (float*)dcumQ, nC, PN);
  return ssd_status();
}

int oa_ssd_out_fwd(const void* Y, const void* z, long long ldz, void* y, void* yraw, long long ldy, int B, int L, int H, int P,
                   void* stream) {
  SsdDims d{B, L, H, P, 4, 0, L / SQ};
  if (!ssd_dims_ok(d) || (z && !yraw)) return OA_ERR_ARG;
  const long long total = (long long)B * L * H * (P / 2);
  ssd_out_fwd_kernel<<<(int)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const float*)Y, (const __nv_bfloat16*)z, ldz, (__nv_bfloat16*)y, (__nv_bfloat16*)yraw, ldy, d);
  return ssd_status();
}

int oa_ssd_dy_prep(const void* dy, const void* yraw, long long ldy, const void* z, long long ldz, void* dz, long long lddz, void* dY,
                   int B, int L, int H, int P, void* stream) {
  SsdDims d{B, L, H, P, 4, 0, L / SQ};
  if (!ssd_dims_ok(d) || (z && (!yraw || !dz))) return OA_ERR_ARG;
  const long long total = (long long)B * L * H * (P / 2);
  ssd_dy_prep_kernel<<<(int)((total + 255) / 256 > 148 * 32 ? 148 * 32 : (total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)yraw, ldy, (const __nv_bfloat16*)z, ldz, (__nv_bfloat16*)dz, lddz,
      (__nv_bfloat16*)dY, d);
  return ssd_status();
}

int oa_ssd_mask_bwd(const void* dM, const void* Gm, const void* cum, const void* scale, void* dG, void* row_mm, void* col_mm,
                    void* col_ge, void* diag, int G, void* stream) {
  if (G <= 0) return OA_ERR_ARG;
  ssd_mask_bwd_kernel<<<G, 256, 0, (cudaStream_t)stream>>>((const float*)dM, (const float*)Gm, (const float*)cum, (const float*)scale,
                                                              (__nv_bfloat16*)dG, (float*)row_mm, (float*)col_mm, (float*)col_ge,
                                                              (float*)diag);
  return ssd_status();
}

int oa_ssd_prep_bwd(const void* dCt, const void* dBt, const void* dCe, const void* Ct, const void* Bt, const void* cum, const void* dqk,
                    const void* theta, void* dCn, void* dBn, void* dCb, void* dBb, void* dtheta, void* dcum_ce, int B, int L, int H,
                    int N, int A, void* stream) {
  SsdDims d{B, L, H, 2, N, A, L / SQ};
  if (!ssd_dims_ok(d) || N > 128 || (A > 0 && (!theta || !dtheta))) return OA_ERR_ARG;
  SsdPrepBwd a{(const float*)dCt, (const float*)dBt, (const float*)dCe, (const __nv_bfloat16*)Ct, (const __nv_bfloat16*)Bt,
               (const float*)cum, (const float*)dqk, (const float*)theta, (float*)dCn, (float*)dBn, (float*)dCb, (float*)dBb,
               (float*)dtheta, (float*)dcum_ce, d};
  ssd_prep_bwd_kernel<<<B * d.nC * 4, 256, 0, (cudaStream_t)stream>>>(a);
  return ssd_status();
}

int oa_ssd_dx_out(const void* dX, const void* dXw, const void* X, const void* w, void* dx, long long lddx, void* dw, int B, int L, int H,
                  int P, void* stream) {
  SsdDims d{B, L, H, P, 4, 0, L / SQ};
  if (!ssd_dims_ok(d)) return OA_ERR_ARG;
  ssd_dx_out_kernel<<<B * H * d.nC, 256, 0, (cudaStream_t)stream>>>((const float*)dX, (const float*)dXw, (const __nv_bfloat16*)X,
                                                                    (const float*)w, (__nv_bfloat16*)dx, lddx, (float*)dw, d);
  return ssd_status();
}

// theta [B*L, H, A] from angle [B*L, lda] and dt [B*L, H]; tot is scratch [B, nC, H, A]
int oa_ssd_theta_fwd(const void* angle, int lda, const void* dt, void* tot, void* theta, int B, int L, int H, int A, void* stream) {
  SsdDims d{B, L, H, 2, 2 * A > 4 ? ((2 * A + 3) / 4) * 4 : 4, A, L / SQ};
  if (!ssd_dims_ok(d) || A <= 0 || lda < A) return OA_ERR_ARG;
  const int warps = B * d.nC * H, grid = (warps + 7) / 8;
  ssd_theta_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)angle, lda, (const float*)dt, (float*)tot, (float*)theta, d, 0);
  ssd_theta_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)angle, lda, (const float*)dt, (float*)tot, (float*)theta, d, 1);
  return ssd_status();
}

// dangle [B*L, lda] (+=, zeroed by the caller) and ddt [B*L, H] (=) from dtheta; A <= 128
int oa_ssd_theta_bwd(const void* dtheta, const void* angle, int lda, const void* dt, void* tot, void* dangle, void* ddt, int B, int L,
                     int H, int A, void* stream) {
  SsdDims d{B, L, H, 2, 2 * A > 4 ? ((2 * A + 3) / 4) * 4 : 4, A, L / SQ};
  if (!ssd_dims_ok(d) || A <= 0 || A > 128 || lda < A) return OA_ERR_ARG;
  const int warps = B * d.nC * H, grid = (warps + 7) / 8;
  ssd_theta_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)dtheta, (const float*)angle, lda, (const float*)dt,
                                                              (float*)tot, (float*)dangle, (float*)ddt, d, 0);
  ssd_theta_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)dtheta, (const float*)angle, lda, (const float*)dt,
                                                              (float*)tot, (float*)dangle, (float*)ddt, d, 1);
  return ssd_status();
}

// Scalar tail of the chunked-scan backward: [G, Q] inputs (G = B*H*nC chunks of 128 tokens) -> dadt, dt and trap gradients
// [B*L, H] and the skip gradient dD [H] (null: skipped); ddt_theta [B*L, H] (may be null) is the dt gradient that came through
// the rotary phases; scratch: float[2 * B*L*H + G].
int oa_ssd_tail(const void* dw, const void* w, const void* col_ge, const void* row_mm, const void* col_mm, const void* dcum_ce,
                const void* diag, const void* qk, const void* cum, const void* dcumQ, const void* dt, const void* trap,
                const void* ddt_theta, void* dadt, void* ddt, void* dtrap, void* dD, void* scratch, int B, int L, int H,
                void* stream) {
  if (B <= 0 || L <= 0 || H <= 0 || L % SQ) return OA_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int nC = L / SQ, G = B * H * nC;
  const long long n = (long long)B * L * H;
  float* dgam = (float*)scratch;
  float* dscale_l = dgam + n;
  float* dpart = dscale_l + n;
  ssd_tail_chunk_kernel<<<G, SQ, 0, st>>>((const float*)dw, (const float*)w, (const float*)col_ge, (const float*)row_mm,
                                         (const float*)col_mm, (const float*)dcum_ce, (const float*)diag, (const float*)qk,
                                         (const float*)cum, (const float*)dcumQ, (float*)dadt, dgam, dscale_l, dD ? dpart : nullptr,
                                         B, L, H, nC);
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ssd_tail_token_kernel<<<(int)blocks, 256, 0, st>>>(dgam, dscale_l, (const float*)dt, (const float*)trap, (const float*)ddt_theta,
                                                    (float*)ddt, (float*)dtrap, B, L, H);
  if (dD) ssd_tail_skip_kernel<<<H, 32, 0, st>>>(dpart, (float*)dD, B, H, nC);
  return ssd_status();
}

}  // extern "C"
