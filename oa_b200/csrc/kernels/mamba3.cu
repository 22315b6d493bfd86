// Mamba-3 SISO selective scan (forward, backward, single-token step) with the exact reference recurrence
// (Source/Private/Oa/Ml/Shader/Compute/Nn/Ssm/Mamba3/Mamba3SisoFwd.slang:9-18, CPU statement in
// Test/Ml/Nn/TestMamba3.cpp:107-142), per (batch, head):
//     theta_t += angle_t * dt_t                       (cumulative rotary angle, A angles)
//     C~ = rot(C_t + Cbias, theta_t),  B~ = rot(B_t + Bbias, theta_t)      pairs (2k, 2k+1), k < A
//     a = exp(adt_t); gamma = dt_t * sigmoid(trap_t); scale = gamma + dt_{t+1} * (1 - sigmoid(trap_{t+1}))
//     y_t[p] = sum_n C~[n] * (a * H[p,n]) + (D + gamma * <C~,B~>) * x_t[p]         (* silu(z_t[p]) when gated)
//     H[p,n] = a * H[p,n] + scale * x_t[p] * B~[n]
// The reference runs one work-group per (batch, head), sequential over the sequence, and its backward recomputes
// from states saved every 32 steps.  Here the head dimension is split across CTAs (state rows evolve independently;
// only reductions over p couple them), so a layer runs B*H*P/16 CTAs of 128 threads, the state lives in registers
// (fp32), and checkpoints are chunked: the forward saves the state and the rotary angle at every chunk boundary
// (chunk = 256 tokens by default), the backward walks chunks in reverse, re-runs a chunk from its checkpoint storing
// sub-boundary states every 8 steps in a scratch buffer, then replays 8 steps at a time into shared memory and
// differentiates them in reverse.  Thread (pl, ng) of a CTA owns state row p = pg*PL + pl and columns
// [ng*N/8, (ng+1)*N/8).
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr int M3_NG = 8;        // column groups per state row
constexpr int M3_MAXNT = 16;    // N / 8 <= 16  (N <= 128)
constexpr int M3_SC = 8;        // replay depth of the backward pass
constexpr float M3_TWO_PI = 6.283185307179586f;

template <typename T> __device__ __forceinline__ float m3ld(const T* p);
template <> __device__ __forceinline__ float m3ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float m3ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void m3st(T* p, float v);
template <> __device__ __forceinline__ void m3st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void m3st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

struct M3Params {
  int B, L, H, P, N, A, PL, chunk;
  int has_z, has_d;
  const float* Cn; const float* Bn;            // [B, L, N] normalised, shared by all heads (one group)
  const void* x; const void* z; long long xs;  // [B*L, >= H*P] with row stride xs (elements)
  const float* dt; const float* adt; const float* trap;   // [B, L, H]
  const float* angle;                          // [B, L, A]
  const float* Cb; const float* Bb;            // [H, N]
  const float* D;                              // [H]
  void* y; long long ys;                       // [B*L, H*P] with row stride ys
  float* Hck;                                  // [B, H, nC, P, N] state at the start of every chunk
  float* Tck;                                  // [B, H, nC, A] rotary angle at the start of every chunk
  float* Hfinal; float* Tfinal;                // optional final state [B, H, P, N], [B, H, A]
  float* Kfinal; float* Vfinal;                // optional last rotated B~ [B, H, N] and last x [B, H, P] (decode look-ahead term)
};

// Rotates this thread's column slice in place and returns nothing; cs/sn are per-pair values for the thread's pairs.
template <int NT>
__device__ __forceinline__ void m3_rotate(float* v, const float* cs, const float* sn, int npairs_rot) {
#pragma unroll
  for (int k = 0; k < NT / 2; ++k) {
    if (k < npairs_rot) {
      float v0 = v[2 * k], v1 = v[2 * k + 1];
      v[2 * k] = v0 * cs[k] - v1 * sn[k];
      v[2 * k + 1] = v0 * sn[k] + v1 * cs[k];
    }
  }
}

__device__ __forceinline__ float m3_sum8(float v) {   // sum over the 8 column-group lanes of one state row
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

// One forward step on registers.  Returns yv (before gating) for this thread's row (identical on the 8 lanes of a row).
template <int NT>
__device__ __forceinline__ float m3_step(float* Hs, const float* Ct, const float* Bt, float a, float scale, float coef_d, float gamma,
                                         float xv) {
  float qk = 0.f, yd = 0.f;
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    qk = fmaf(Ct[i], Bt[i], qk);
    float hd = a * Hs[i];
    yd = fmaf(Ct[i], hd, yd);
    Hs[i] = fmaf(scale * xv, Bt[i], hd);
  }
  qk = m3_sum8(qk);
  yd = m3_sum8(yd);
  return yd + (coef_d + gamma * qk) * xv;
}

template <typename T, int NT>
__global__ void __launch_bounds__(128)
mamba3_fwd_kernel(const M3Params p) {
  const int PG = p.P / p.PL;
  const int cta = blockIdx.x;
  const int pg = cta % PG, h = (cta / PG) % p.H, b = cta / (PG * p.H);
  const int pl = threadIdx.x >> 3, ng = threadIdx.x & 7;
  if (pl >= p.PL) return;
  const int pr = pg * p.PL + pl;                 // state row (head-dim index)
  const int n0 = ng * NT;
  const int pair0 = n0 / 2;
  const int nrot = max(0, min(NT / 2, p.A - pair0));   // rotary pairs inside this thread's slice
  const int nC = (p.L + p.chunk - 1) / p.chunk;
  float Hs[NT], th[NT / 2], cb[NT], bb[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) { Hs[i] = 0.f; cb[i] = p.Cb[h * p.N + n0 + i]; bb[i] = p.Bb[h * p.N + n0 + i]; }
#pragma unroll
  for (int k = 0; k < NT / 2; ++k) th[k] = 0.f;
  const float Dh = p.has_d ? p.D[h] : 0.f;
  const T* xp = reinterpret_cast<const T*>(p.x);
  const T* zp = reinterpret_cast<const T*>(p.z);
  T* yp = reinterpret_cast<T*>(p.y);
  for (int t = 0; t < p.L; ++t) {
    if (t % p.chunk == 0) {     // checkpoint: state and angle at the start of the chunk
      const int c = t / p.chunk;
      if (p.Hck) {
        float* hk = p.Hck + ((((long long)b * p.H + h) * nC + c) * p.P + pr) * p.N + n0;
#pragma unroll
        for (int i = 0; i < NT; ++i) hk[i] = Hs[i];
      }
      if (p.Tck && pg == 0 && pl == 0) {
        float* tk = p.Tck + (((long long)b * p.H + h) * nC + c) * p.A + pair0;
#pragma unroll
        for (int k = 0; k < NT / 2; ++k) if (k < nrot) tk[k] = th[k];
      }
    }
    const long long bt = (long long)b * p.L + t;
    const float dt = p.dt[bt * p.H + h], adt = p.adt[bt * p.H + h];
    const float tr = sigmoid_f(p.trap[bt * p.H + h]);
    float sg = 0.f;
    if (t + 1 < p.L) sg = p.dt[(bt + 1) * p.H + h] * (1.f - sigmoid_f(p.trap[(bt + 1) * p.H + h]));
    const float gamma = dt * tr, scale = gamma + sg, a = __expf(adt);
    float Ct[NT], Bt[NT], cs[NT / 2], sn[NT / 2];
#pragma unroll
    for (int i = 0; i < NT; ++i) { Ct[i] = p.Cn[bt * p.N + n0 + i] + cb[i]; Bt[i] = p.Bn[bt * p.N + n0 + i] + bb[i]; }
#pragma unroll
    for (int k = 0; k < NT / 2; ++k) {
      if (k < nrot) {
        float v = th[k] + p.angle[bt * p.A + pair0 + k] * dt;
        v -= M3_TWO_PI * rintf(v * (1.f / M3_TWO_PI));
        th[k] = v;
        __sincosf(v, &sn[k], &cs[k]);
      }
    }
    m3_rotate<NT>(Ct, cs, sn, nrot);
    m3_rotate<NT>(Bt, cs, sn, nrot);
    const float xv = m3ld<T>(xp + bt * p.xs + h * p.P + pr);
    float yv = m3_step<NT>(Hs, Ct, Bt, a, scale, Dh, gamma, xv);
    if (p.has_z) yv *= silu_f(m3ld<T>(zp + bt * p.xs + h * p.P + pr));
    if (ng == 0) m3st<T>(yp + bt * p.ys + h * p.P + pr, yv);
    if (t == p.L - 1) {
      if (p.Kfinal && pg == 0 && pl == 0) {
#pragma unroll
        for (int i = 0; i < NT; ++i) p.Kfinal[((long long)b * p.H + h) * p.N + n0 + i] = Bt[i];
      }
      if (p.Vfinal && ng == 0) p.Vfinal[((long long)b * p.H + h) * p.P + pr] = xv;
    }
  }
  if (p.Hfinal) {
    float* hf = p.Hfinal + (((long long)b * p.H + h) * p.P + pr) * p.N + n0;
#pragma unroll
    for (int i = 0; i < NT; ++i) hf[i] = Hs[i];
  }
  if (p.Tfinal && pg == 0 && pl == 0) {
#pragma unroll
    for (int k = 0; k < NT / 2; ++k) if (k < nrot) p.Tfinal[((long long)b * p.H + h) * p.A + pair0 + k] = th[k];
  }
}

struct M3BwdParams {
  M3Params f;
  const void* dy; long long dys;     // upstream gradient [B*L, H*P]
  void* dx; void* dz; long long dxs; // written (plain stores, one writer per element) with row stride dxs
  float* dCn; float* dBn;            // [B, L, N]  atomically accumulated over heads and row groups (pre-zeroed)
  float* ddt; float* dadt; float* dtrap;   // [B, L, H]   atomics (pre-zeroed)
  float* dangle;                     // [B, L, A]   atomics (pre-zeroed)
  float* dCb; float* dBb;            // [H, N]      atomics (pre-zeroed)
  float* dD;                         // [H]         atomics (pre-zeroed)
  float* scratch;                    // [ctas][chunk / SC][PL * N] sub-boundary states
};

// Shared layout of the backward kernel (floats): replay states [SC][PL*N], partial column sums [2][PL][N],
// scalar partials [4 warps][8].
template <typename T, int NT>
__global__ void __launch_bounds__(128)
mamba3_bwd_kernel(const M3BwdParams q) {
  const M3Params& p = q.f;
  extern __shared__ float sm[];
  const int PG = p.P / p.PL;
  const int cta = blockIdx.x;
  const int pg = cta % PG, h = (cta / PG) % p.H, b = cta / (PG * p.H);
  const int pl = threadIdx.x >> 3, ng = threadIdx.x & 7;
  const bool active = pl < p.PL;
  const int pr = pg * p.PL + min(pl, p.PL - 1);
  const int n0 = ng * NT, pair0 = n0 / 2;
  const int nrot = max(0, min(NT / 2, p.A - pair0));
  const int nC = (p.L + p.chunk - 1) / p.chunk;
  const int rowN = p.PL * p.N;
  float* s_H = sm;                                  // [SC][PL*N]   H_{t-1} of the replayed steps
  float* s_dC = s_H + M3_SC * rowN;                 // [PL][N]
  float* s_dB = s_dC + rowN;                        // [PL][N]
  float* s_red = s_dB + rowN;                       // [4 warps][8] scalar partials
  float* sub = q.scratch + (long long)cta * (p.chunk / M3_SC) * rowN;
  const T* xp = reinterpret_cast<const T*>(p.x);
  const T* zp = reinterpret_cast<const T*>(p.z);
  const T* dyp = reinterpret_cast<const T*>(q.dy);
  T* dxp = reinterpret_cast<T*>(q.dx);
  T* dzp = reinterpret_cast<T*>(q.dz);
  float cb[NT], bb[NT], dH[NT], gth[NT / 2], dcb[NT], dbb[NT];
#pragma unroll
  for (int i = 0; i < NT; ++i) { cb[i] = p.Cb[h * p.N + n0 + i]; bb[i] = p.Bb[h * p.N + n0 + i]; dH[i] = 0.f; dcb[i] = 0.f; dbb[i] = 0.f; }
#pragma unroll
  for (int k = 0; k < NT / 2; ++k) gth[k] = 0.f;     // running sum of d(theta_s) for s >= t
  const float Dh = p.has_d ? p.D[h] : 0.f;
  float dD_acc = 0.f;

  auto load_step = [&](long long bt, int t, float* Ct, float* Bt, float* cs, float* sn, const float* thv, float& a, float& gamma,
                       float& scale, float& dt, float& tr, float& dtn, float& trn) {
    dt = p.dt[bt * p.H + h];
    tr = sigmoid_f(p.trap[bt * p.H + h]);
    dtn = 0.f; trn = 0.f;
    if (t + 1 < p.L) { dtn = p.dt[(bt + 1) * p.H + h]; trn = sigmoid_f(p.trap[(bt + 1) * p.H + h]); }
    gamma = dt * tr; scale = gamma + dtn * (1.f - trn); a = __expf(p.adt[bt * p.H + h]);
#pragma unroll
    for (int i = 0; i < NT; ++i) { Ct[i] = p.Cn[bt * p.N + n0 + i] + cb[i]; Bt[i] = p.Bn[bt * p.N + n0 + i] + bb[i]; }
#pragma unroll
    for (int k = 0; k < NT / 2; ++k) if (k < nrot) __sincosf(thv[k], &sn[k], &cs[k]);
    m3_rotate<NT>(Ct, cs, sn, nrot);
    m3_rotate<NT>(Bt, cs, sn, nrot);
  };

  for (int c = nC - 1; c >= 0; --c) {
    const int t0 = c * p.chunk, t1 = min(p.L, t0 + p.chunk);
    // ---- pass A: re-run the chunk from its checkpoint, storing the state every SC steps
    float Hs[NT], th[NT / 2];
    {
      const float* hk = p.Hck + ((((long long)b * p.H + h) * nC + c) * p.P + pr) * p.N + n0;
      const float* tk = p.Tck + (((long long)b * p.H + h) * nC + c) * p.A + pair0;
#pragma unroll
      for (int i = 0; i < NT; ++i) Hs[i] = hk[i];
#pragma unroll
      for (int k = 0; k < NT / 2; ++k) th[k] = k < nrot ? tk[k] : 0.f;
    }
    for (int t = t0; t < t1; ++t) {
      if ((t - t0) % M3_SC == 0 && active) {
        float* d = sub + (long long)((t - t0) / M3_SC) * rowN + pl * p.N + n0;
#pragma unroll
        for (int i = 0; i < NT; ++i) d[i] = Hs[i];
        // theta at the sub-boundary is recomputed in pass B from the chunk checkpoint, see below
      }
      const long long bt = (long long)b * p.L + t;
      float Ct[NT], Bt[NT], cs[NT / 2], sn[NT / 2], a, gamma, scale, dt, tr, dtn, trn;
#pragma unroll
      for (int k = 0; k < NT / 2; ++k) if (k < nrot) {
        float v = th[k] + p.angle[bt * p.A + pair0 + k] * p.dt[bt * p.H + h];
        th[k] = v - M3_TWO_PI * rintf(v * (1.f / M3_TWO_PI));
      }
      load_step(bt, t, Ct, Bt, cs, sn, th, a, gamma, scale, dt, tr, dtn, trn);
      const float xv = m3ld<T>(xp + bt * p.xs + h * p.P + pr);
      (void)m3_step<NT>(Hs, Ct, Bt, a, scale, Dh, gamma, xv);
    }
    // theta at the END of the chunk is now in th[]; walking back we subtract angle*dt step by step.
    // ---- pass B: sub-chunks in reverse
    const int nsub = (t1 - t0 + M3_SC - 1) / M3_SC;
    for (int sidx = nsub - 1; sidx >= 0; --sidx) {
      const int u0 = t0 + sidx * M3_SC, u1 = min(t1, u0 + M3_SC);
      // replay: store H_{t-1} for every step of the sub-chunk; thetas of the steps are derived backwards from th[]
      __syncthreads();
      if (active) {
        const float* s = sub + (long long)sidx * rowN + pl * p.N + n0;
#pragma unroll
        for (int i = 0; i < NT; ++i) Hs[i] = s[i];
      }
      // theta_t for t in [u0, u1): th currently holds theta_{u1-1}
      float thr[M3_SC][NT / 2];
      {
        float cur[NT / 2];
#pragma unroll
        for (int k = 0; k < NT / 2; ++k) cur[k] = th[k];
#pragma unroll
        for (int j = M3_SC - 1; j >= 0; --j) {
          const int t = u0 + j;
          if (t < u1) {
            const long long bt = (long long)b * p.L + t;
#pragma unroll
            for (int k = 0; k < NT / 2; ++k) {
              thr[j][k] = cur[k];
              if (k < nrot) cur[k] -= p.angle[bt * p.A + pair0 + k] * p.dt[bt * p.H + h];
            }
          }
        }
#pragma unroll
        for (int k = 0; k < NT / 2; ++k) th[k] = cur[k];     // theta_{u0-1}, the value needed by the previous sub-chunk
      }
#pragma unroll 1
      for (int j = 0; j < M3_SC; ++j) {
        const int t = u0 + j;
        if (t >= u1) break;
        if (active) {
          float* d = s_H + (long long)j * rowN + pl * p.N + n0;
#pragma unroll
          for (int i = 0; i < NT; ++i) d[i] = Hs[i];
        }
        const long long bt = (long long)b * p.L + t;
        float Ct[NT], Bt[NT], cs[NT / 2], sn[NT / 2], a, gamma, scale, dt, tr, dtn, trn;
        load_step(bt, t, Ct, Bt, cs, sn, thr[j], a, gamma, scale, dt, tr, dtn, trn);
        const float xv = m3ld<T>(xp + bt * p.xs + h * p.P + pr);
        (void)m3_step<NT>(Hs, Ct, Bt, a, scale, Dh, gamma, xv);
      }
      // reverse differentiation of the sub-chunk
#pragma unroll 1
      for (int j = M3_SC - 1; j >= 0; --j) {
        const int t = u0 + j;
        if (t >= u1) continue;
        const long long bt = (long long)b * p.L + t;
        float Ct[NT], Bt[NT], cs[NT / 2], sn[NT / 2], a, gamma, scale, dt, tr, dtn, trn;
        load_step(bt, t, Ct, Bt, cs, sn, thr[j], a, gamma, scale, dt, tr, dtn, trn);
        const float xv = m3ld<T>(xp + bt * p.xs + h * p.P + pr);
        float Hp[NT];
        {
          const float* s = s_H + (long long)j * rowN + min(pl, p.PL - 1) * p.N + n0;
#pragma unroll
          for (int i = 0; i < NT; ++i) Hp[i] = s[i];
        }
        // recompute the forward scalars of this step
        float qk = 0.f, yd = 0.f;
#pragma unroll
        for (int i = 0; i < NT; ++i) { qk = fmaf(Ct[i], Bt[i], qk); yd = fmaf(Ct[i], a * Hp[i], yd); }
        qk = m3_sum8(qk); yd = m3_sum8(yd);
        const float coef = Dh + gamma * qk;
        const float yv = yd + coef * xv;
        float dyv = active ? m3ld<T>(dyp + bt * q.dys + h * p.P + pr) : 0.f;
        if (p.has_z) {
          const float zv = m3ld<T>(zp + bt * p.xs + h * p.P + pr);
          const float sg_ = sigmoid_f(zv);
          if (active && ng == 0) m3st<T>(dzp + bt * q.dxs + h * p.P + pr, dyv * yv * sg_ * (1.f + zv * (1.f - sg_)));
          dyv *= zv * sg_;
        }
        // state update H_t = a H_{t-1} + scale x B~ ; output y = C~ . (a H_{t-1}) + coef x
        float dxs_ = 0.f, dsc = 0.f, da = 0.f;
        float dCt[NT], dBt[NT];
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          const float g = dH[i];                      // dL/dH_t
          dxs_ = fmaf(g, Bt[i], dxs_);
          dsc = fmaf(g * xv, Bt[i], dsc);
          dBt[i] = scale * g * xv;
          const float dhd = g + dyv * Ct[i];          // dL/d(a H_{t-1})
          dCt[i] = dyv * a * Hp[i];
          da = fmaf(dhd, Hp[i], da);
          dH[i] = a * dhd;                            // dL/dH_{t-1}
        }
        dxs_ = m3_sum8(dxs_);
        const float dcoef_row = dyv * xv;             // per state row; summed over rows below
        float dx_total = scale * dxs_ + dyv * coef;
        if (active && ng == 0) m3st<T>(dxp + bt * q.dxs + h * p.P + pr, dx_total);
        // sums over the rows of this CTA: scalars via shuffles + shared, vectors via shared
        float sc_dsc = active ? dsc : 0.f, sc_da = active ? da : 0.f, sc_dcoef = (active && ng == 0) ? dcoef_row : 0.f;
        sc_dsc = warp_sum(sc_dsc); sc_da = warp_sum(sc_da); sc_dcoef = warp_sum(sc_dcoef);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) { float* r = s_red + (threadIdx.x >> 5) * 8; r[0] = sc_dsc; r[1] = sc_da; r[2] = sc_dcoef; }
        if (active) {
#pragma unroll
          for (int i = 0; i < NT; ++i) { s_dC[pl * p.N + n0 + i] = dCt[i]; s_dB[pl * p.N + n0 + i] = dBt[i]; }
        }
        __syncthreads();
        float t_dsc = 0.f, t_da = 0.f, t_dcoef = 0.f;
        for (int w = 0; w < 4; ++w) { t_dsc += s_red[w * 8]; t_da += s_red[w * 8 + 1]; t_dcoef += s_red[w * 8 + 2]; }
        // column sums over the rows of this CTA; row 0's threads then own column slice n0.. of the totals
        if (pl == 0) {
          float dCs[NT], dBs[NT];
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            float sc_ = 0.f, sb_ = 0.f;
            for (int r = 0; r < p.PL; ++r) { sc_ += s_dC[r * p.N + n0 + i]; sb_ += s_dB[r * p.N + n0 + i]; }
            // coefficient path: coef = D + gamma * qk, qk = <C~, B~>
            dCs[i] = sc_ + t_dcoef * gamma * Bt[i];
            dBs[i] = sb_ + t_dcoef * gamma * Ct[i];
          }
          // rotation backward: d(theta_k) += g0 * (-r1) + g1 * r0 for C~ and B~; un-rotate the gradients
#pragma unroll
          for (int k = 0; k < NT / 2; ++k) {
            if (k < nrot) {
              float dth = -dCs[2 * k] * Ct[2 * k + 1] + dCs[2 * k + 1] * Ct[2 * k] - dBs[2 * k] * Bt[2 * k + 1] + dBs[2 * k + 1] * Bt[2 * k];
              gth[k] += dth;
              float g0 = dCs[2 * k], g1 = dCs[2 * k + 1];
              dCs[2 * k] = g0 * cs[k] + g1 * sn[k]; dCs[2 * k + 1] = -g0 * sn[k] + g1 * cs[k];
              g0 = dBs[2 * k]; g1 = dBs[2 * k + 1];
              dBs[2 * k] = g0 * cs[k] + g1 * sn[k]; dBs[2 * k + 1] = -g0 * sn[k] + g1 * cs[k];
            }
          }
          float ddt_th = 0.f;
#pragma unroll
          for (int k = 0; k < NT / 2; ++k) {
            if (k < nrot) {
              const float ang = p.angle[bt * p.A + pair0 + k];
              atomicAdd(q.dangle + bt * p.A + pair0 + k, gth[k] * dt);
              ddt_th = fmaf(gth[k], ang, ddt_th);
            }
          }
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            atomicAdd(q.dCn + bt * p.N + n0 + i, dCs[i]);
            atomicAdd(q.dBn + bt * p.N + n0 + i, dBs[i]);
            dcb[i] += dCs[i]; dbb[i] += dBs[i];
          }
          // only lanes 0..7 of warp 0 are here
          ddt_th += __shfl_xor_sync(0xffu, ddt_th, 1);
          ddt_th += __shfl_xor_sync(0xffu, ddt_th, 2);
          ddt_th += __shfl_xor_sync(0xffu, ddt_th, 4);
          if (ng == 0) {
            // scale = gamma_t + dt_{t+1} (1 - tr_{t+1});  gamma_t = dt_t * tr_t;  coef = D + gamma * qk
            const float dgamma = t_dcoef * qk + t_dsc;
            atomicAdd(q.ddt + bt * p.H + h, dgamma * tr + ddt_th);
            atomicAdd(q.dtrap + bt * p.H + h, dgamma * dt * tr * (1.f - tr));
            if (t + 1 < p.L) {
              atomicAdd(q.ddt + (bt + 1) * p.H + h, t_dsc * (1.f - trn));
              atomicAdd(q.dtrap + (bt + 1) * p.H + h, -t_dsc * dtn * trn * (1.f - trn));
            }
            atomicAdd(q.dadt + bt * p.H + h, t_da * a);
            dD_acc += t_dcoef;
          }
        }
      }
    }
  }
  if (pl == 0) {
#pragma unroll
    for (int i = 0; i < NT; ++i) { atomicAdd(q.dCb + h * p.N + n0 + i, dcb[i]); atomicAdd(q.dBb + h * p.N + n0 + i, dbb[i]); }
    if (ng == 0 && p.has_d) atomicAdd(q.dD + h, dD_acc);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Single-token step (decode).  scale_t needs dt_{t+1} and trap_{t+1}, which a decoder does not have yet, so the state
// kept between steps is the partial one, H_t - dt_{t+1}(1 - sigmoid(trap_{t+1})) x_t (x) B~_t, together with x_t and B~_t;
// the missing term is added when token t+1 arrives (Nn/Ssm/Mamba3/Mamba3.cpp Step: StepSsm / StepAngle / StepK / StepV).
struct M3StepParams {
  int B, H, P, N, A, PL, has_z, has_d, first;
  const float* Cn; const float* Bn;     // [B, N]
  const void* x; const void* z; long long xs;
  const float* dt; const float* adt; const float* trap;   // [B, H]
  const float* angle;                   // [B, A]
  const float* Cb; const float* Bb; const float* D;
  void* y; long long ys;
  float* Hst; float* Vst;                           // [B,H,P,N] [B,H,P]   updated in place (one owner per element)
  const float* Tin; const float* Kin;               // [B,H,A] [B,H,N]     read by every row group of a head ...
  float* Tout; float* Kout;                         //                     ... so the new values go to a second buffer
};

template <typename T, int NT>
__global__ void __launch_bounds__(128)
mamba3_step_kernel(const M3StepParams p) {
  const int PG = p.P / p.PL;
  const int cta = blockIdx.x;
  const int pg = cta % PG, h = (cta / PG) % p.H, b = cta / (PG * p.H);
  const int pl = threadIdx.x >> 3, ng = threadIdx.x & 7;
  if (pl >= p.PL) return;
  const int pr = pg * p.PL + pl, n0 = ng * NT, pair0 = n0 / 2;
  const int nrot = max(0, min(NT / 2, p.A - pair0));
  const long long bh = (long long)b * p.H + h;
  float* Hp = p.Hst + (bh * p.P + pr) * p.N + n0;
  const float dt = p.dt[bh], tr = sigmoid_f(p.trap[bh]), a = __expf(p.adt[bh]);
  const float gamma = dt * tr, late = p.first ? 0.f : dt * (1.f - tr);
  const float xprev = p.first ? 0.f : p.Vst[bh * p.P + pr];
  float Hs[NT], Ct[NT], Bt[NT], cs[NT / 2], sn[NT / 2];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    const float kprev = p.first ? 0.f : p.Kin[bh * p.N + n0 + i];
    Hs[i] = (p.first ? 0.f : Hp[i]) + late * xprev * kprev;
    Ct[i] = p.Cn[(long long)b * p.N + n0 + i] + p.Cb[h * p.N + n0 + i];
    Bt[i] = p.Bn[(long long)b * p.N + n0 + i] + p.Bb[h * p.N + n0 + i];
  }
  float thv[NT / 2];
#pragma unroll
  for (int k = 0; k < NT / 2; ++k) {
    thv[k] = 0.f;
    if (k < nrot) {
      float v = (p.first ? 0.f : p.Tin[bh * p.A + pair0 + k]) + p.angle[(long long)b * p.A + pair0 + k] * dt;
      v -= M3_TWO_PI * rintf(v * (1.f / M3_TWO_PI));
      thv[k] = v;
      __sincosf(v, &sn[k], &cs[k]);
    }
  }
  m3_rotate<NT>(Ct, cs, sn, nrot);
  m3_rotate<NT>(Bt, cs, sn, nrot);
  const T* xp = reinterpret_cast<const T*>(p.x);
  const float xv = m3ld<T>(xp + (long long)b * p.xs + h * p.P + pr);
  float yv = m3_step<NT>(Hs, Ct, Bt, a, gamma, p.has_d ? p.D[h] : 0.f, gamma, xv);
  if (p.has_z) yv *= silu_f(m3ld<T>(reinterpret_cast<const T*>(p.z) + (long long)b * p.xs + h * p.P + pr));
#pragma unroll
  for (int i = 0; i < NT; ++i) Hp[i] = Hs[i];
  if (ng == 0) {
    m3st<T>(reinterpret_cast<T*>(p.y) + (long long)b * p.ys + h * p.P + pr, yv);
    p.Vst[bh * p.P + pr] = xv;
  }
  if (pg == 0 && pl == 0) {
#pragma unroll
    for (int i = 0; i < NT; ++i) p.Kout[bh * p.N + n0 + i] = Bt[i];
#pragma unroll
    for (int k = 0; k < NT / 2; ++k) if (k < nrot) p.Tout[bh * p.A + pair0 + k] = thv[k];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Preprocess: one CTA per projected row [z | x | B | C | dd_dt | dd_A | trap | angle]
// (Shader/Compute/Nn/Ssm/Mamba3/Mamba3Preprocess.slang:1-14).  z and x stay in the projection and are read strided.
struct M3PreParams {
  int rows, H, N, A;
  long long stride;                  // row stride of proj / dproj (elements)
  int b_off, c_off, dt_off, a_off, trap_off, angle_off;
  float eps, dt_min, dt_max, afloor;
  const void* proj; const float* dt_bias;
  float* Bn; float* Cn; float* rstd;          // [rows, N], [rows, N], [rows, 2]
  float* dt; float* adt; float* trap; float* angle;
  // backward
  const float* dBn; const float* dCn; const float* ddt; const float* dadt; const float* dtrap; const float* dangle;
  void* dproj; float* ddt_bias;
};

__device__ __forceinline__ float m3_block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
  return t;
}

template <typename T>
__global__ void __launch_bounds__(128)
mamba3_pre_fwd_kernel(const M3PreParams p) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const T* pr = reinterpret_cast<const T*>(p.proj) + row * p.stride;
  const int i = threadIdx.x;
  const float bv = i < p.N ? m3ld<T>(pr + p.b_off + i) : 0.f;
  const float cv = i < p.N ? m3ld<T>(pr + p.c_off + i) : 0.f;
  const float rb = rsqrtf(m3_block_sum(bv * bv, red) / p.N + p.eps);
  const float rc = rsqrtf(m3_block_sum(cv * cv, red) / p.N + p.eps);
  if (i < p.N) { p.Bn[row * p.N + i] = bv * rb; p.Cn[row * p.N + i] = cv * rc; }
  if (i == 0) { p.rstd[row * 2] = rb; p.rstd[row * 2 + 1] = rc; }
  for (int h = i; h < p.H; h += blockDim.x) {
    const float u = m3ld<T>(pr + p.dt_off + h) + p.dt_bias[h];
    const float sp = u > 20.f ? u : log1pf(__expf(u));
    const float dt = fminf(fmaxf(sp, p.dt_min), p.dt_max);
    const float da = m3ld<T>(pr + p.a_off + h);
    const float ht = da >= 0.f ? 1.f + da : 1.f / (1.f - da);
    p.dt[row * p.H + h] = dt;
    p.adt[row * p.H + h] = fminf(-ht, -p.afloor) * dt;
    p.trap[row * p.H + h] = m3ld<T>(pr + p.trap_off + h);
  }
  for (int k = i; k < p.A; k += blockDim.x) p.angle[row * p.A + k] = m3ld<T>(pr + p.angle_off + k);
}

template <typename T>
__global__ void __launch_bounds__(128)
mamba3_pre_bwd_kernel(const M3PreParams p) {
  __shared__ float red[4];
  const long long row = blockIdx.x;
  const T* pr = reinterpret_cast<const T*>(p.proj) + row * p.stride;
  T* dp = reinterpret_cast<T*>(p.dproj) + row * p.stride;
  const int i = threadIdx.x;
  const float rb = p.rstd[row * 2], rc = p.rstd[row * 2 + 1];
  const float bn = i < p.N ? p.Bn[row * p.N + i] : 0.f, cn = i < p.N ? p.Cn[row * p.N + i] : 0.f;
  const float gb = i < p.N ? p.dBn[row * p.N + i] : 0.f, gc = i < p.N ? p.dCn[row * p.N + i] : 0.f;
  const float mb = m3_block_sum(gb * bn, red) / p.N;
  const float mc = m3_block_sum(gc * cn, red) / p.N;
  if (i < p.N) {
    m3st<T>(dp + p.b_off + i, rb * (gb - bn * mb));
    m3st<T>(dp + p.c_off + i, rc * (gc - cn * mc));
  }
  for (int h = i; h < p.H; h += blockDim.x) {
    const float u = m3ld<T>(pr + p.dt_off + h) + p.dt_bias[h];
    const float sp = u > 20.f ? u : log1pf(__expf(u));
    const float dt = fminf(fmaxf(sp, p.dt_min), p.dt_max);
    const float da = m3ld<T>(pr + p.a_off + h);
    const float ht = da >= 0.f ? 1.f + da : 1.f / (1.f - da);
    const float atok = fminf(-ht, -p.afloor);
    const float g_adt = p.dadt[row * p.H + h];
    const float g_dt = p.ddt[row * p.H + h] + g_adt * atok;
    const float pass = (sp > p.dt_min && sp < p.dt_max) ? 1.f : 0.f;
    const float g_u = g_dt * pass * sigmoid_f(u);
    m3st<T>(dp + p.dt_off + h, g_u);
    atomicAdd(p.ddt_bias + h, g_u);
    const float dht = da >= 0.f ? 1.f : ht * ht;
    m3st<T>(dp + p.a_off + h, (ht > p.afloor) ? -g_adt * dt * dht : 0.f);
    m3st<T>(dp + p.trap_off + h, p.dtrap[row * p.H + h]);
  }
  for (int k = i; k < p.A; k += blockDim.x) m3st<T>(dp + p.angle_off + k, p.dangle[row * p.A + k]);
}

}  // namespace oa

using namespace oa;

namespace {

int m3_check(int P, int N, int A, int* PL, int* NT) {
  if (N % 8 != 0 || N > 128 || N < 16) return OA_ERR_ARG;
  const int nt = N / 8;
  if (nt != 2 && nt != 4 && nt != 8 && nt != 16) return OA_ERR_ARG;
  if (A * 2 > N) return OA_ERR_ARG;
  int pl = P < 16 ? P : 16;
  if (P % pl != 0) return OA_ERR_ARG;
  *PL = pl; *NT = nt;
  return OA_OK;
}

#define M3_DISPATCH(KERNEL, NTV, DTYPE, ...)                                               \
  do {                                                                                     \
    if ((DTYPE) == OA_BF16) {                                                              \
      switch (NTV) {                                                                       \
        case 2: KERNEL<__nv_bfloat16, 2> __VA_ARGS__; break;                               \
        case 4: KERNEL<__nv_bfloat16, 4> __VA_ARGS__; break;                               \
        case 8: KERNEL<__nv_bfloat16, 8> __VA_ARGS__; break;                               \
        default: KERNEL<__nv_bfloat16, 16> __VA_ARGS__; break;                             \
      }                                                                                    \
    } else {                                                                               \
      switch (NTV) {                                                                       \
        case 2: KERNEL<float, 2> __VA_ARGS__; break;                                       \
        case 4: KERNEL<float, 4> __VA_ARGS__; break;                                       \
        case 8: KERNEL<float, 8> __VA_ARGS__; break;                                       \
        default: KERNEL<float, 16> __VA_ARGS__; break;                                     \
      }                                                                                    \
    }                                                                                      \
  } while (0)

}  // namespace

static void m3_fill(M3Params& f, const void* x, const void* z, long long xs, const float* Cn, const float* Bn, const float* dt,
                    const float* adt, const float* trap, const float* angle, const float* Cb, const float* Bb, const float* D, int B,
                    int L, int H, int P, int N, int A, int PL, int chunk) {
  f.B = B; f.L = L; f.H = H; f.P = P; f.N = N; f.A = A; f.PL = PL; f.chunk = chunk;
  f.has_z = z != nullptr; f.has_d = D != nullptr;
  f.Cn = Cn; f.Bn = Bn; f.x = x; f.z = z; f.xs = xs; f.dt = dt; f.adt = adt; f.trap = trap; f.angle = angle;
  f.Cb = Cb; f.Bb = Bb; f.D = D;
  f.y = nullptr; f.ys = 0; f.Hck = nullptr; f.Tck = nullptr; f.Hfinal = nullptr; f.Tfinal = nullptr; f.Kfinal = nullptr; f.Vfinal = nullptr;
}

extern "C" int oa_mamba3_scan_fwd(int dtype, const void* x, const void* z, long long xs, const float* Cn, const float* Bn, const float* dt,
                                  const float* adt, const float* trap, const float* angle, const float* Cb, const float* Bb,
                                  const float* D, void* y, long long ys, float* Hck, float* Tck, float* Hfinal, float* Tfinal,
                                  float* Kfinal, float* Vfinal, int B, int L, int H, int P, int N, int A, int chunk, void* stream) {
  int PL, NT;
  if (int rc = m3_check(P, N, A, &PL, &NT)) return rc;
  if (chunk <= 0 || chunk % M3_SC != 0) return OA_ERR_ARG;
  if (B <= 0 || L <= 0) return OA_OK;
  M3Params f;
  m3_fill(f, x, z, xs, Cn, Bn, dt, adt, trap, angle, Cb, Bb, D, B, L, H, P, N, A, PL, chunk);
  f.y = y; f.ys = ys; f.Hck = Hck; f.Tck = Tck; f.Hfinal = Hfinal; f.Tfinal = Tfinal; f.Kfinal = Kfinal; f.Vfinal = Vfinal;
  const int grid = B * H * (P / PL);
  M3_DISPATCH(mamba3_fwd_kernel, NT, dtype, <<<grid, PL * M3_NG, 0, (cudaStream_t)stream>>>(f));
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" size_t oa_mamba3_scratch_floats(int B, int H, int P, int N, int chunk) {
  const int PL = P < 16 ? P : 16;
  return (size_t)B * H * (P / PL) * (chunk / M3_SC) * PL * N;
}

template <typename T, int NT>
static int m3_launch_bwd(const M3BwdParams& q, int grid, size_t smem, cudaStream_t st) {
  static bool set = false;     // per instantiation
  if (!set) {
    if (cudaFuncSetAttribute(mamba3_bwd_kernel<T, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
      return OA_ERR_DRIVER;
    set = true;
  }
  mamba3_bwd_kernel<T, NT><<<grid, 128, smem, st>>>(q);
  return OA_OK;
}

extern "C" int oa_mamba3_scan_bwd(int dtype, const void* x, const void* z, long long xs, const float* Cn, const float* Bn, const float* dt,
                                  const float* adt, const float* trap, const float* angle, const float* Cb, const float* Bb,
                                  const float* D, const void* dy, long long dys, void* dx, void* dz, long long dxs, float* dCn,
                                  float* dBn, float* ddt, float* dadt, float* dtrap, float* dangle, float* dCb, float* dBb, float* dD,
                                  const float* Hck, const float* Tck, float* scratch, int B, int L, int H, int P, int N, int A,
                                  int chunk, void* stream) {
  int PL, NT;
  if (int rc = m3_check(P, N, A, &PL, &NT)) return rc;
  if (chunk <= 0 || chunk % M3_SC != 0) return OA_ERR_ARG;
  if (B <= 0 || L <= 0) return OA_OK;
  M3BwdParams q;
  m3_fill(q.f, x, z, xs, Cn, Bn, dt, adt, trap, angle, Cb, Bb, D, B, L, H, P, N, A, PL, chunk);
  q.f.Hck = const_cast<float*>(Hck); q.f.Tck = const_cast<float*>(Tck);
  q.dy = dy; q.dys = dys; q.dx = dx; q.dz = dz; q.dxs = dxs; q.dCn = dCn; q.dBn = dBn; q.ddt = ddt; q.dadt = dadt; q.dtrap = dtrap;
  q.dangle = dangle; q.dCb = dCb; q.dBb = dBb; q.dD = dD; q.scratch = scratch;
  const int grid = B * H * (P / PL);
  const size_t smem = ((size_t)(M3_SC + 2) * PL * N + 32) * sizeof(float);
  if (smem > 100 * 1024) return OA_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = OA_OK;
#define M3_BWD(TT)                                                    \
  switch (NT) {                                                       \
    case 2: rc = m3_launch_bwd<TT, 2>(q, grid, smem, st); break;      \
    case 4: rc = m3_launch_bwd<TT, 4>(q, grid, smem, st); break;      \
    case 8: rc = m3_launch_bwd<TT, 8>(q, grid, smem, st); break;      \
    default: rc = m3_launch_bwd<TT, 16>(q, grid, smem, st); break;    \
  }
  if (dtype == OA_BF16) { M3_BWD(__nv_bfloat16) } else { M3_BWD(float) }
#undef M3_BWD
  if (rc) return rc;
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_mamba3_step(int dtype, const void* x, const void* z, long long xs, const float* Cn, const float* Bn, const float* dt,
                              const float* adt, const float* trap, const float* angle, const float* Cb, const float* Bb, const float* D,
                              void* y, long long ys, float* Hst, float* Vst, const float* Tin, const float* Kin, float* Tout,
                              float* Kout, int B, int H, int P, int N, int A, int first, void* stream) {
  int PL, NT;
  if (int rc = m3_check(P, N, A, &PL, &NT)) return rc;
  if (B <= 0) return OA_OK;
  M3StepParams s;
  s.B = B; s.H = H; s.P = P; s.N = N; s.A = A; s.PL = PL; s.has_z = z != nullptr; s.has_d = D != nullptr; s.first = first;
  s.Cn = Cn; s.Bn = Bn; s.x = x; s.z = z; s.xs = xs; s.dt = dt; s.adt = adt; s.trap = trap; s.angle = angle; s.Cb = Cb; s.Bb = Bb;
  s.D = D; s.y = y; s.ys = ys; s.Hst = Hst; s.Vst = Vst; s.Tin = Tin; s.Kin = Kin; s.Tout = Tout; s.Kout = Kout;
  const int grid = B * H * (P / PL);
  M3_DISPATCH(mamba3_step_kernel, NT, dtype, <<<grid, PL * M3_NG, 0, (cudaStream_t)stream>>>(s));
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

static int m3_pre_fill(M3PreParams& p, int rows, int H, int N, int A, int d_inner, long long stride, float eps, float dt_min,
                       float dt_max, float afloor) {
  if (N > 128 || N <= 0) return OA_ERR_ARG;
  p.rows = rows; p.H = H; p.N = N; p.A = A; p.stride = stride;
  p.b_off = 2 * d_inner; p.c_off = p.b_off + N; p.dt_off = p.c_off + N; p.a_off = p.dt_off + H; p.trap_off = p.a_off + H;
  p.angle_off = p.trap_off + H;
  p.eps = eps; p.dt_min = dt_min; p.dt_max = dt_max; p.afloor = afloor;
  p.dBn = p.dCn = p.ddt = p.dadt = p.dtrap = p.dangle = nullptr; p.dproj = nullptr; p.ddt_bias = nullptr;
  return OA_OK;
}

extern "C" int oa_mamba3_pre_fwd(int dtype, const void* proj, long long stride, const float* dt_bias, int rows, int H, int N, int A,
                                 int d_inner, float eps, float dt_min, float dt_max, float afloor, float* Bn, float* Cn, float* rstd,
                                 float* dt, float* adt, float* trap, float* angle, void* stream) {
  M3PreParams p;
  if (int rc = m3_pre_fill(p, rows, H, N, A, d_inner, stride, eps, dt_min, dt_max, afloor)) return rc;
  if (rows <= 0) return OA_OK;
  p.proj = proj; p.dt_bias = dt_bias; p.Bn = Bn; p.Cn = Cn; p.rstd = rstd; p.dt = dt; p.adt = adt; p.trap = trap; p.angle = angle;
  if (dtype == OA_BF16) mamba3_pre_fwd_kernel<__nv_bfloat16><<<rows, 128, 0, (cudaStream_t)stream>>>(p);
  else mamba3_pre_fwd_kernel<float><<<rows, 128, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_mamba3_pre_bwd(int dtype, const void* proj, void* dproj, long long stride, const float* dt_bias, int rows, int H, int N,
                                 int A, int d_inner, float eps, float dt_min, float dt_max, float afloor, const float* Bn,
                                 const float* Cn, const float* rstd, const float* dBn, const float* dCn, const float* ddt,
                                 const float* dadt, const float* dtrap, const float* dangle, float* ddt_bias, void* stream) {
  M3PreParams p;
  if (int rc = m3_pre_fill(p, rows, H, N, A, d_inner, stride, eps, dt_min, dt_max, afloor)) return rc;
  if (rows <= 0) return OA_OK;
  p.proj = proj; p.dproj = dproj; p.dt_bias = dt_bias; p.Bn = const_cast<float*>(Bn); p.Cn = const_cast<float*>(Cn);
  p.rstd = const_cast<float*>(rstd); p.dBn = dBn; p.dCn = dCn; p.ddt = ddt; p.dadt = dadt; p.dtrap = dtrap; p.dangle = dangle;
  p.ddt_bias = ddt_bias; p.dt = p.adt = p.trap = p.angle = nullptr;
  if (dtype == OA_BF16) mamba3_pre_bwd_kernel<__nv_bfloat16><<<rows, 128, 0, (cudaStream_t)stream>>>(p);
  else mamba3_pre_bwd_kernel<float><<<rows, 128, 0, (cudaStream_t)stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------------------------------------------------
// Gated per-head RMSNorm of the scan output: out = y * rstd(y over the head) * w[h, p] * silu(z)
// (Nn/Mamba3/Mamba3.cpp:230-244 composes RmsNormGated(y, 1, 0, z, 1e-5, norm_before_gate) with the weight product).
// One warp per (token, head); z is read, and dz written, at its place inside the projected row.
namespace oa {

template <typename T>
__global__ void __launch_bounds__(256)
gated_norm_fwd_kernel(const T* __restrict__ y, const T* __restrict__ z, long long zs, const float* __restrict__ w, T* __restrict__ out,
                      float* __restrict__ rstd, long long rows, int H, int P, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  for (long long r = warp0; r < rows * H; r += (long long)gridDim.x * 8) {
    const long long tok = r / H;
    const int h = (int)(r % H);
    const T* yr = y + r * P;
    float v[4], ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { const int pp = lane + 32 * j; v[j] = pp < P ? m3ld<T>(yr + pp) : 0.f; ss = fmaf(v[j], v[j], ss); }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / P + eps);
    if (lane == 0 && rstd) rstd[r] = rs;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int pp = lane + 32 * j;
      if (pp < P) m3st<T>(out + r * P + pp, v[j] * rs * w[h * P + pp] * silu_f(m3ld<T>(z + tok * zs + h * P + pp)));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gated_norm_bwd_kernel(const T* __restrict__ y, const T* __restrict__ z, long long zs, const float* __restrict__ w,
                      const float* __restrict__ rstd, const T* __restrict__ dout, T* __restrict__ dy, T* __restrict__ dz, long long dzs,
                      float* __restrict__ dw, long long rows, int H, int P) {
  extern __shared__ float s_dw[];     // [H * P]; a head is always handled by the same warp of a CTA (H % 8 == 0) or by atomics
  for (int i = threadIdx.x; i < H * P; i += blockDim.x) s_dw[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  for (long long r = warp0; r < rows * H; r += (long long)gridDim.x * 8) {
    const long long tok = r / H;
    const int h = (int)(r % H);
    const float rs = rstd[r];
    float n[4], dn[4], g[4], zv[4], dot = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int pp = lane + 32 * j;
      n[j] = dn[j] = g[j] = zv[j] = 0.f;
      if (pp < P) {
        n[j] = m3ld<T>(y + r * P + pp) * rs;
        g[j] = m3ld<T>(dout + r * P + pp);
        zv[j] = m3ld<T>(z + tok * zs + h * P + pp);
        dn[j] = g[j] * w[h * P + pp] * silu_f(zv[j]);
        dot = fmaf(dn[j], n[j], dot);
      }
    }
    dot = warp_sum(dot) / P;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int pp = lane + 32 * j;
      if (pp < P) {
        const float sg = sigmoid_f(zv[j]);
        m3st<T>(dy + r * P + pp, rs * (dn[j] - n[j] * dot));
        m3st<T>(dz + tok * dzs + h * P + pp, g[j] * n[j] * w[h * P + pp] * sg * (1.f + zv[j] * (1.f - sg)));
        atomicAdd(&s_dw[h * P + pp], g[j] * n[j] * zv[j] * sg);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H * P; i += blockDim.x) if (s_dw[i] != 0.f) atomicAdd(dw + i, s_dw[i]);
}

}  // namespace oa

extern "C" int oa_gated_norm_fwd(int dtype, const void* y, const void* z, long long zs, const float* w, void* out, float* rstd,
                                 long long rows, int H, int P, float eps, void* stream) {
  if (P > 128 || P <= 0) return OA_ERR_ARG;
  if (rows <= 0) return OA_OK;
  long long warps = rows * H;
  int grid = (int)((warps + 7) / 8 < 148 * 8 ? (warps + 7) / 8 : 148 * 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == OA_BF16)
    gated_norm_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)z, zs, w, (__nv_bfloat16*)out,
                                                                 rstd, rows, H, P, eps);
  else
    gated_norm_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)y, (const float*)z, zs, w, (float*)out, rstd, rows, H, P, eps);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_gated_norm_bwd(int dtype, const void* y, const void* z, long long zs, const float* w, const float* rstd, const void* dout,
                                 void* dy, void* dz, long long dzs, float* dw, long long rows, int H, int P, void* stream) {
  if (P > 128 || P <= 0) return OA_ERR_ARG;
  if ((size_t)H * P * 4 > 48 * 1024) return OA_ERR_TOO_LARGE;
  if (rows <= 0) return OA_OK;
  long long warps = rows * H;
  int grid = (int)((warps + 7) / 8 < 148 * 4 ? (warps + 7) / 8 : 148 * 4);
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)H * P * 4;
  if (dtype == OA_BF16)
    gated_norm_bwd_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)z, zs, w, rstd,
                                                                    (const __nv_bfloat16*)dout, (__nv_bfloat16*)dy, (__nv_bfloat16*)dz,
                                                                    dzs, dw, rows, H, P);
  else
    gated_norm_bwd_kernel<float><<<grid, 256, smem, st>>>((const float*)y, (const float*)z, zs, w, rstd, (const float*)dout, (float*)dy,
                                                           (float*)dz, dzs, dw, rows, H, P);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
