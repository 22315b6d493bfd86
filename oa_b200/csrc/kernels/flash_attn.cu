// Causal / full scaled-dot-product attention for sm_100a, forward and backward, bf16 in / fp32 accumulate.
//
// The reference's FlashCausal kernels (Source/Private/Oa/Ml/Shader/Compute/Nn/Attention/FlashCausal*.slang)
// run one work-group per query row with all scores of the row in shared memory (S <= 1024, fp32 only, no
// tensor cores).  Here the work is tiled 128 queries x 128 keys, every matrix product of a tile runs on
// tcgen05 with accumulators in TMEM, tiles arrive through TMA, and the probabilities (and their gradients) are
// written back to TMEM as bf16 and read from there as the A operand of the next product: nothing but Q, K, V, dO
// passes through shared memory.  Q, K, V are read in place from a packed projection output ([B*S, row_stride] with
// head h at column h*head_dim), and O is written merged ([B*S, H*head_dim]), so there are no SplitHeads / MergeHeads
// passes.
//
// Measured facts that shape the kernels: one tcgen05.mma costs about 50 cycles to issue from a thread (the N = 64
// products are issue bound), an MUFU exponential occupies its pipe for 8 cycles per warp (1024 cycles per 128 x 128
// tile), and a warp that waits for the tensor pipe between key blocks idles the SFU.  Hence: score tiles are copied
// to registers and released at once so the next score product is issued under this block's exponentials, products are
// issued by two or three warps, and every kernel but the head_dim 128 forward is persistent (one CTA per SM walks its
// work items in snake order, heaviest causal items first), so TMEM, barriers and the operand rings live across items.
//
// Backward is two kernels, both deterministic (single writer per output element, like the reference's
// FlashCausalBwdQ / FlashCausalBwdKV): one accumulates dK, dV in TMEM over the query blocks of a key block, the other dQ
// over the key blocks of a query block.  Probabilities are recomputed from the saved log-sum-exp.
// Every wait is bounded and reports to a status word.
#include "common.cuh"
#include "api.h"

namespace oa {

constexpr int FA_BM = 128;   // queries per tile
constexpr int FA_BN = 128;   // keys per tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr int FA_THREADS = 320;   // head_dim 128 forward: 8 softmax warps + MMA warp + TMA warp

// 64-thread named barrier shared by the two warps that own the same 32 query rows.
__device__ __forceinline__ void pair_sync(int quad) {
  asm volatile("bar.sync %0, 64;" ::"r"(quad + 1) : "memory");
}

struct FlashParams {
  int batch, heads, seq, head_dim;
  float scale;
  int causal;
  __nv_bfloat16* o;
  long long o_stride;
  float* lse;            // [B, H, S]
  int* status;
};

// ===================================================================================== forward, S double-buffered in TMEM
// One CTA owns one 128-query tile of one (batch, head).  S = Q K_j^T alternates between two TMEM buffers, and the MMA warp
// always runs two key blocks ahead of the softmax (Q K_{j+2}^T is issued right after P_j V_j), so the softmax warps never
// wait for the tensor pipe: they go from block j straight to block j+1 and the SFU stays busy.
//   warps 0-7  softmax: two threads per query row (warp w: TMEM lane quadrant w % 4, key columns [64 * (w / 4), +64)), the
//              64 scores of a thread are read from TMEM once, the row maximum is exchanged with the partner thread through
//              a parity-double-buffered slot, probabilities go back to TMEM as packed bf16 over the columns of S_j;
//   warp 8     MMA issuer: P is the A operand straight from TMEM, V the B operand from shared memory, O accumulates in
//              TMEM over all key blocks and is read once at the end;
//   warp 9     TMA producer (Q once, K / V rings).
// The running maximum is updated lazily: while the new row maximum exceeds the one in use by less than 2^8 the old one is
// kept (probabilities then stay below 256), so O in TMEM is rescaled only in the rare iterations where some row of a warp
// jumps by more than that; the final 1/l uses the same maxima, so the result is the exact softmax.
// TMEM: S0 | S1 | O = 128 + 128 + head_dim columns.
template <int HD>
struct Fwd2Cfg {
  static constexpr int NSK = 3;                            // K ring depth (K runs two blocks ahead of V)
  static constexpr int NSV = (HD == 64) ? 3 : 2;           // V ring depth
  static constexpr int Q_BYTES = FA_BM * HD * 2;
  static constexpr int KV_BYTES = FA_BN * HD * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + NSK * KV_BYTES;
  static constexpr int OFF_X = OFF_V + NSV * KV_BYTES;     // float[2 parities][2 halves][128 rows]: row-maximum exchange
  static constexpr int OFF_BAR = OFF_X + 2 * 2 * FA_BM * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0;                           // + 128 * (j & 1)
  static constexpr int TM_O = 256;
};

constexpr float FA_RESCALE_THRESHOLD = 8.f;                // log2 units


template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  using Cfg = Fwd2Cfg<HD>;
  constexpr int NSK = Cfg::NSK, NSV = Cfg::NSV;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;                 // [NSK]
  uint64_t* k_empty = k_full + NSK;            // [NSK]
  uint64_t* v_full = k_empty + NSK;            // [NSV]
  uint64_t* v_empty = v_full + NSV;            // [NSV]
  uint64_t* s_full = v_empty + NSV;            // [2]  S buffer holds Q K_j^T
  uint64_t* p_full = s_full + 2;               // [2]  P_j written over S buffer (and O rescaled if needed)
  uint64_t* o_done = s_full + 4;               //      O += P_j V_j finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
  float* xch = reinterpret_cast<float*>(smem + Cfg::OFF_X);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.seq + FA_BM - 1) / FA_BM;
  const int qb = nblk - 1 - blockIdx.x;        // heaviest causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int n_kv = p.causal ? (qb + 1) : nblk;
  const int row0 = b * p.seq;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_error(p.status, OA_KERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    for (int s = 0; s < NSK; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < NSV; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 8); }
    mbar_init(o_done, 1);
    mbar_fence_init();
  }
  if (warp == 8) { tmem_alloc<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                            // the prologue above ran under the previous kernel's tail; global memory from here on

  if (warp == 9) {
    // ------------- producer: the whole warp walks the loop and waits together; one lane issues the copies.  K block i is
    // loaded two iterations before V block i - 2... both rings are simply filled in order, K first.
    if (lane == 0) {
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int x = 0; x < HD / 64; ++x)
        tma_load_2d(smem + Cfg::OFF_Q + x * (FA_BM * 128), &tmQ, q_full, h * HD + x * 64, row0 + qb * FA_BM);
    }
    for (int i = 0; i < n_kv + 2; ++i) {
      if (i < n_kv) {
        const int st = i % NSK;
        if (!warp_wait(&k_empty[st], ((i / NSK) & 1) ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
        if (lane == 0) {
          mbar_expect_tx(&k_full[st], Cfg::KV_BYTES);
#pragma unroll
          for (int x = 0; x < HD / 64; ++x)
            tma_load_2d(smem + Cfg::OFF_K + st * Cfg::KV_BYTES + x * (FA_BN * 128), &tmK, &k_full[st], h * HD + x * 64, row0 + i * FA_BN);
        }
      }
      const int jv = i - 2;                    // V lags K by two blocks, like its consumer
      if (jv >= 0) {
        const int st = jv % NSV;
        if (!warp_wait(&v_empty[st], ((jv / NSV) & 1) ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
        if (lane == 0) {
          mbar_expect_tx(&v_full[st], Cfg::KV_BYTES);
#pragma unroll
          for (int x = 0; x < HD / 64; ++x)
            tma_load_2d(smem + Cfg::OFF_V + st * Cfg::KV_BYTES + x * (FA_BN * 128), &tmV, &v_full[st], h * HD + x * 64, row0 + jv * FA_BN);
        }
      }
      __syncwarp();
    }
  } else if (warp == 8) {
    // ------------- MMA issuer (warp-uniform waits, lane 0 issues)
    constexpr uint32_t idesc_qk = umma_idesc_bf16(FA_BM, FA_BN, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(FA_BM, HD, 0, 1);
    const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q);
    auto issue_qk = [&](int i) -> bool {       // S[i & 1] = Q K_i^T
      const int st = i % NSK;
      if (!warp_wait(&k_full[st], (i / NSK) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); return false; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K + st * Cfg::KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_S + (i & 1) * FA_BN, umma_smem_desc_sw128(q_addr + off, 16, 1024),
                   umma_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[i & 1]);
      }
      __syncwarp();
      return true;
    };
    bool ok = warp_wait(q_full, 0);
    if (!ok && lane == 0) report_error(p.status, OA_KERR_WAIT_FULL);
    if (ok) ok = issue_qk(0);
    if (ok && n_kv > 1) ok = issue_qk(1);
    for (int j = 0; j < n_kv && ok; ++j) {
      const int st = j % NSV;
      if (!warp_wait(&v_full[st], (j / NSV) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); break; }
      if (!warp_wait(&p_full[j & 1], (j >> 1) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_SOFTMAX); break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = smem_u32(smem + Cfg::OFF_V + st * Cfg::KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks)
          umma_f16_ts(tmem_base + Cfg::TM_O, tmem_base + Cfg::TM_S + (j & 1) * FA_BN + ks * 8,
                      umma_smem_desc_sw128(v_addr + ks * 2048, FA_BN * 128, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&v_empty[st]);
        umma_commit(o_done);
      }
      __syncwarp();
      if (j + 2 < n_kv) ok = issue_qk(j + 2);  // overwrites S[j & 1] = P_j: ordered after P_j V_j by the pipe
    }
  } else {
    // ------------- softmax + output: two threads per query row (key columns split in halves)
    constexpr int OC = HD / 2;                   // output columns owned by this thread
    const int quad = warp & 3;
    const int half = warp >> 2;
    const int r = quad * 32 + lane;
    const int qi = qb * FA_BM + r;               // query index inside the sequence
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const uint32_t o_addr = tmem_base + t_lane + Cfg::TM_O + half * OC;
    const float sl2 = p.scale * LOG2E;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      ok = warp_wait(&s_full[j & 1], (j >> 1) & 1);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + t_lane + Cfg::TM_S + (j & 1) * FA_BN;
      uint32_t sv[64];
      tmem_ld32(s_addr + half * 64, sv);
      tmem_ld32(s_addr + half * 64 + 32, sv + 32);
      tmem_ld_wait();
      const bool need_mask = (p.causal && j == qb) || (j * FA_BN + FA_BN > p.seq);
      if (need_mask) {
        const int lim = min(p.causal ? qi : 0x7fffffff, p.seq - 1) - j * FA_BN - half * 64;   // columns i <= lim are alive
#pragma unroll
        for (int i = 0; i < 64; ++i) sv[i] = (i <= lim) ? sv[i] : 0xff800000u;                 // -inf
      }
      float m0 = __uint_as_float(sv[0]), m1 = __uint_as_float(sv[1]), m2 = __uint_as_float(sv[2]), m3 = __uint_as_float(sv[3]);
#pragma unroll
      for (int i = 4; i < 64; i += 4) {
        m0 = fmaxf(m0, __uint_as_float(sv[i])); m1 = fmaxf(m1, __uint_as_float(sv[i + 1]));
        m2 = fmaxf(m2, __uint_as_float(sv[i + 2])); m3 = fmaxf(m3, __uint_as_float(sv[i + 3]));
      }
      float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      // Exchange with the partner thread of this row.  Both threads now hold their scores in registers, so after this
      // barrier the S buffer may be overwritten by either of them.
      float* slots = xch + (j & 1) * (2 * FA_BM);
      slots[(half ^ 1) * FA_BM + r] = mx;
      pair_sync(quad);
      mx = fmaxf(mx, slots[half * FA_BM + r]) * sl2;
      const float m_new = fmaxf(m_run, mx);
      const bool grow = (m_new - m_run) > FA_RESCALE_THRESHOLD;           // first block: m_run = -inf -> true
      const float m_cand = grow ? m_new : m_run;
      const float m_use = (m_cand == -INFINITY) ? 0.f : m_cand;           // row fully masked so far
      const float alpha = grow ? fast_exp2(m_run - m_use) : 1.f;           // m_run = -inf -> 0
      const float neg_m = -m_use;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        const float e0 = fast_exp2(fmaf(__uint_as_float(sv[i]), sl2, neg_m));
        const float e1 = fast_exp2(fmaf(__uint_as_float(sv[i + 1]), sl2, neg_m));
        const float e2 = fast_exp2(fmaf(__uint_as_float(sv[i + 2]), sl2, neg_m));
        const float e3 = fast_exp2(fmaf(__uint_as_float(sv[i + 3]), sl2, neg_m));
        l0 += e0; l1 += e1; l2 += e2; l3 += e3;
        pk[i >> 1] = pack_bf16x2(e0, e1);
        pk[(i >> 1) + 1] = pack_bf16x2(e2, e3);
      }
      tmem_st32(s_addr + half * 32, pk);          // P over the first 64 columns of S (two keys per column)
      l_run = l_run * alpha + ((l0 + l1) + (l2 + l3));
      m_run = m_cand;
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // some row of this warp moved its maximum: rescale O (needs the previous P*V finished)
        ok = warp_wait(o_done, (j - 1) & 1);
        if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(o_addr + c * 32, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[j & 1]);
    }
    // combine the two partial row sums (parity slot of an iteration that is two behind any reader)
    {
      float* slots = xch + (n_kv & 1) * (2 * FA_BM);
      slots[(half ^ 1) * FA_BM + r] = l_run;
      pair_sync(quad);
      l_run += slots[half * FA_BM + r];
    }
    if (ok) {
      ok = warp_wait(o_done, (n_kv - 1) & 1);
      if (!ok && lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL);
    }
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* op = p.o + (long long)(row0 + qi) * p.o_stride + h * HD + half * OC;
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (qi < p.seq) {
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(op + c * 32 + g * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(o[g * 8]) * inv, __uint_as_float(o[g * 8 + 1]) * inv),
                pack_bf16x2(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv),
                pack_bf16x2(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv),
                pack_bf16x2(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv));
        }
      }
      if (p.lse && half == 0 && qi < p.seq) p.lse[((long long)b * p.heads + h) * p.seq + qi] = (m_run + log2f(l_run)) / LOG2E;
    }
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) { tc_fence_after(); tmem_dealloc<Cfg::TMEM_COLS>(tmem_base); }
}

// ===================================================================================== forward, head_dim 64: two tiles per CTA
// Two adjacent 128-query tiles of one (batch, head) share a CTA and the K / V rings but are otherwise independent pipelines
// (softmax warps 0-3 + MMA warp 8 for tile 0, warps 4-7 + MMA warp 9 for tile 1), so their phases drift apart and the
// exponentials of one tile cover the TMEM traffic, row maxima and barrier hand-offs of the other.  One thread owns one query
// row (all 128 key columns: no partner exchange).  The score tile is copied to registers and RELEASED at once, so
// Q K_{j+1}^T is issued while the exponentials of block j run; probabilities have their own TMEM columns:
// S0 | S1 | P0 | P1 | O0 | O1 = 128 + 128 + 64 + 64 + 64 + 64.
struct FwdPairCfg {
  static constexpr int HD = 64;
  static constexpr int NS = 3;
  static constexpr int Q_BYTES = FA_BM * HD * 2;
  static constexpr int KV_BYTES = FA_BN * HD * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + NS * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + NS * KV_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0, TM_P = 256, TM_O = 384;   // + 128 / 64 / 64 * tile
  static constexpr int THREADS = 352;                        // 8 softmax warps, 2 MMA warps, 1 TMA warp
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Persistent: one CTA per SM walks the work items (tile pair, head, batch) it owns, heaviest causal pairs first and items
// dealt in snake order (round r: CTA c takes item r G + c, or r G + G-1-c when r is odd; within 3 % of the greedy optimum), so TMEM, barriers and the K / V rings live across items, the producer and the MMA warps run ahead
// into the next item while the softmax warps write the previous output, and no SM pays a CTA launch per item.  Every
// barrier phase is derived from a running count kept identically by its producers and consumers.
__global__ void __launch_bounds__(FwdPairCfg::THREADS, 1)
flash_fwd_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  using Cfg = FwdPairCfg;
  constexpr int NS = Cfg::NS, HD = Cfg::HD;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;            // both MMA warps are done with the Q tiles of the item
  uint64_t* k_full = bars + 2;             // [NS]
  uint64_t* k_empty = k_full + NS;         // [NS]  one arrival per MMA warp
  uint64_t* v_full = k_empty + NS;         // [NS]
  uint64_t* v_empty = v_full + NS;         // [NS]  one arrival per MMA warp
  uint64_t* s_full = v_empty + NS;         // [2]   S_t holds Q_t K_j^T
  uint64_t* s_empty = s_full + 2;          // [2]   ... and is in registers (4 warps)
  uint64_t* p_full = s_full + 4;           // [2]   P_t written (and O_t rescaled if needed) (4 warps)
  uint64_t* o_done = s_full + 6;           // [2]   O_t += P_t V_j finished: P_t may be overwritten, O_t may be rescaled
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.seq + FA_BM - 1) / FA_BM;
  const int npair = (nblk + 1) >> 1;
  const int hb = p.heads * p.batch;
  const int n_items = npair * hb;
  const int n_rounds = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  auto item_of = [&](int round) -> int {     // snake order; >= n_items: this CTA sits the round out
    return round * (int)gridDim.x + ((round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  };

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_error(p.status, OA_KERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    mbar_init(q_empty, 2);
    for (int s = 0; s < NS; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 2); mbar_init(&v_empty[s], 2); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&s_empty[t], 4); mbar_init(&p_full[t], 4); mbar_init(&o_done[t], 1); }
    mbar_fence_init();
  }
  if (warp == 8) { tmem_alloc<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                            // the prologue above ran under the previous kernel's tail; global memory from here on

  // item -> (pair, head, batch) and the block counts of its two tiles (tile 1 absent: 0)
  auto decode = [&](int item, int& pr, int& h, int& b, int& nkv0, int& nkv1) {
    pr = npair - 1 - item / hb;
    const int rem = item % hb;
    h = rem % p.heads;
    b = rem / p.heads;
    nkv0 = p.causal ? (2 * pr + 1) : nblk;
    nkv1 = (2 * pr + 1 < nblk) ? (p.causal ? (2 * pr + 2) : nblk) : 0;
  };

  if (warp == 10) {
    // ------------- producer
    uint32_t blk = 0, itc = 0;   // K / V blocks and items loaded so far
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int pr, h, b, nkv0, nkv1;
      decode(item, pr, h, b, nkv0, nkv1);
      const int n_it = max(nkv0, nkv1), row0 = b * p.seq;
      if (!warp_wait(q_empty, (itc & 1) ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
      if (lane == 0) {
        const int tiles = nkv1 > 0 ? 2 : 1;
        mbar_expect_tx(q_full, tiles * Cfg::Q_BYTES);
        for (int t = 0; t < tiles; ++t)
          tma_load_2d(smem + Cfg::OFF_Q + t * Cfg::Q_BYTES, &tmQ, q_full, h * HD, row0 + (2 * pr + t) * FA_BM);
      }
      for (int j = 0; j < n_it; ++j, ++blk) {
        const int st = blk % NS;
        const uint32_t ph = (blk / NS) & 1;
        if (!warp_wait(&k_empty[st], ph ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(&k_full[st], Cfg::KV_BYTES);
          tma_load_2d(smem + Cfg::OFF_K + st * Cfg::KV_BYTES, &tmK, &k_full[st], h * HD, row0 + j * FA_BN);
        }
        if (!warp_wait(&v_empty[st], ph ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(&v_full[st], Cfg::KV_BYTES);
          tma_load_2d(smem + Cfg::OFF_V + st * Cfg::KV_BYTES, &tmV, &v_full[st], h * HD, row0 + j * FA_BN);
        }
        __syncwarp();
      }
      ++itc;
    }
  } else if (warp == 8 || warp == 9) {
    // ------------- MMA issuer of tile t (warp-uniform waits, lane 0 issues)
    const int t = warp - 8;
    constexpr uint32_t idesc_qk = umma_idesc_bf16(FA_BM, FA_BN, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(FA_BM, HD, 0, 1);
    const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q + t * Cfg::Q_BYTES);
    const uint32_t s_tm = tmem_base + Cfg::TM_S + t * FA_BN, p_tm = tmem_base + Cfg::TM_P + t * 64, o_tm = tmem_base + Cfg::TM_O + t * HD;
    uint32_t base = 0, itc = 0, sc = 0, pc = 0;   // K / V blocks before this item, items, S products and P V products of this tile so far
    bool ok = true;
    auto issue_qk = [&](uint32_t blk, bool last) -> bool {       // S_t = Q_t K^T of ring block `blk`
      const int st = blk % NS;
      if (!warp_wait(&k_full[st], (blk / NS) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); return false; }
      if (sc > 0 && !warp_wait(&s_empty[t], (sc - 1) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_EMPTY); return false; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K + st * Cfg::KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma_f16(s_tm, umma_smem_desc_sw128(q_addr + ks * 32, 16, 1024), umma_smem_desc_sw128(k_addr + ks * 32, 16, 1024),
                   idesc_qk, ks > 0 ? 1u : 0u);
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[t]);
        if (last) umma_commit(q_empty);
      }
      __syncwarp();
      ++sc;
      return true;
    };
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int pr, h, b, nkv0, nkv1;
      decode(item, pr, h, b, nkv0, nkv1);
      const int n_it = max(nkv0, nkv1);
      const int n = t == 0 ? nkv0 : nkv1;
      if (!warp_wait(q_full, itc & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); break; }
      if (n > 0) ok = issue_qk(base, n == 1);
      for (int j = 0; j < n && ok; ++j) {
        if (j + 1 < n) { ok = issue_qk(base + j + 1, j + 2 == n); if (!ok) break; }
        const int st = (base + j) % NS;
        if (!warp_wait(&v_full[st], ((base + j) / NS) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        if (!warp_wait(&p_full[t], pc & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_SOFTMAX); ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t v_addr = smem_u32(smem + Cfg::OFF_V + st * Cfg::KV_BYTES);
#pragma unroll
          for (int ks = 0; ks < FA_BN / 16; ++ks)
            umma_f16_ts(o_tm, p_tm + ks * 8, umma_smem_desc_sw128(v_addr + ks * 2048, FA_BN * 128, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&v_empty[st]);
          umma_commit(&o_done[t]);
        }
        __syncwarp();
        ++pc;
      }
      // blocks of this item that this tile does not use (the last one of the pair's shorter tile, or all of an absent tile):
      // the rings still expect one arrival per MMA warp, given once the block has landed
      for (int j = n; j < n_it && ok; ++j) {
        const int st = (base + j) % NS;
        const uint32_t ph = ((base + j) / NS) & 1;
        if (!warp_wait(&k_full[st], ph)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        if (lane == 0) mbar_arrive(&k_empty[st]);
        if (!warp_wait(&v_full[st], ph)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        if (lane == 0) mbar_arrive(&v_empty[st]);
        __syncwarp();
      }
      if (n == 0 && ok && lane == 0) mbar_arrive(q_empty);
      __syncwarp();
      base += n_it;
      ++itc;
    }
  } else {
    // ------------- softmax + output of tile t: one thread per query row
    const int t = warp >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + t_lane + Cfg::TM_S + t * FA_BN;
    const uint32_t p_addr = tmem_base + t_lane + Cfg::TM_P + t * 64;
    const uint32_t o_addr = tmem_base + t_lane + Cfg::TM_O + t * HD;
    const float sl2 = p.scale * LOG2E;
    uint32_t sc = 0, pc = 0;     // score tiles consumed and P V completions awaited so far
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int pr, h, b, nkv0, nkv1;
      decode(item, pr, h, b, nkv0, nkv1);
      const int n = t == 0 ? nkv0 : nkv1;
      if (n == 0) continue;
      const int row0 = b * p.seq;
      const int qbt = 2 * pr + t;
      const int qi = qbt * FA_BM + r;               // query index inside the sequence
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < n; ++j, ++sc) {
        ok = warp_wait(&s_full[t], sc & 1);
        if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
        tc_fence_after();
        uint32_t sv[FA_BN];
#pragma unroll
        for (int c = 0; c < FA_BN / 32; ++c) tmem_ld32(s_addr + c * 32, sv + c * 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[t]);   // the next block's scores may overwrite S_t now
        const bool need_mask = (p.causal && j == qbt) || (j * FA_BN + FA_BN > p.seq);
        if (need_mask) {
          const int lim = min(p.causal ? qi : 0x7fffffff, p.seq - 1) - j * FA_BN;   // columns i <= lim are alive
#pragma unroll
          for (int i = 0; i < FA_BN; ++i) sv[i] = (i <= lim) ? sv[i] : 0xff800000u;  // -inf
        }
        float m0 = __uint_as_float(sv[0]), m1 = __uint_as_float(sv[1]);
#pragma unroll
        for (int i = 2; i < FA_BN - 2; i += 4) {
          m0 = fmax3(m0, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
          m1 = fmax3(m1, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
        }
        const float mx = fmax3(m0, m1, fmaxf(__uint_as_float(sv[FA_BN - 2]), __uint_as_float(sv[FA_BN - 1]))) * sl2;
        const float m_new = fmaxf(m_run, mx);
        const bool grow = (m_new - m_run) > FA_RESCALE_THRESHOLD;           // first block: m_run = -inf -> true
        const float m_cand = grow ? m_new : m_run;
        const float m_use = (m_cand == -INFINITY) ? 0.f : m_cand;           // row fully masked so far
        const float alpha = grow ? fast_exp2(m_run - m_use) : 1.f;           // m_run = -inf -> 0
        const float neg_m = -m_use;
        if (j > 0) {                               // P_t is free and O_t is complete once the previous P V has finished
          ok = warp_wait(&o_done[t], pc & 1);
          if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
          ++pc;
          tc_fence_after();
        }
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
        for (int c = 0; c < FA_BN / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float e0 = fast_exp2(fmaf(__uint_as_float(sv[c * 32 + i]), sl2, neg_m));
            const float e1 = fast_exp2(fmaf(__uint_as_float(sv[c * 32 + i + 1]), sl2, neg_m));
            const float e2 = fast_exp2(fmaf(__uint_as_float(sv[c * 32 + i + 2]), sl2, neg_m));
            const float e3 = fast_exp2(fmaf(__uint_as_float(sv[c * 32 + i + 3]), sl2, neg_m));
            l0 += e0; l1 += e1; l2 += e2; l3 += e3;
            pk[i >> 1] = pack_bf16x2(e0, e1);
            pk[(i >> 1) + 1] = pack_bf16x2(e2, e3);
          }
          tmem_st16(p_addr + c * 16, pk);
        }
        l_run = l_run * alpha + ((l0 + l1) + (l2 + l3));
        m_run = m_cand;
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          // some row of this warp moved its maximum: rescale O
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_addr + c * 32, o);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t]);
      }
      if (!ok) break;
      ok = warp_wait(&o_done[t], pc & 1);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      ++pc;
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* op = p.o + (long long)(row0 + qi) * p.o_stride + h * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (qi < p.seq) {
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(op + c * 32 + g * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(o[g * 8]) * inv, __uint_as_float(o[g * 8 + 1]) * inv),
                pack_bf16x2(__uint_as_float(o[g * 8 + 2]) * inv, __uint_as_float(o[g * 8 + 3]) * inv),
                pack_bf16x2(__uint_as_float(o[g * 8 + 4]) * inv, __uint_as_float(o[g * 8 + 5]) * inv),
                pack_bf16x2(__uint_as_float(o[g * 8 + 6]) * inv, __uint_as_float(o[g * 8 + 7]) * inv));
        }
      }
      if (p.lse && qi < p.seq) p.lse[((long long)b * p.heads + h) * p.seq + qi] = (m_run + log2f(l_run)) / LOG2E;
      tc_fence_before();   // the O reads above complete before this warp's next p_full arrival lets the next item's first P V overwrite O
    }
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) { tc_fence_after(); tmem_dealloc<Cfg::TMEM_COLS>(tmem_base); }
}

template <int HD>
static int launch_fwd2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashParams& p, dim3 grid, cudaStream_t st) {
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(flash_fwd2_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Cfg<HD>::SMEM_BYTES) != cudaSuccess) return OA_ERR_LAUNCH;
    set = true;
  }
  launch_pdl(flash_fwd2_kernel<HD>, grid, dim3(FA_THREADS), Fwd2Cfg<HD>::SMEM_BYTES, st, tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

// ===================================================================================== backward
struct FlashBwdParams {
  int batch, heads, seq, head_dim;
  float scale;
  int causal;
  const float* lse;      // [B, H, S]
  const float* delta;    // [B, H, S]  sum_d dO * O
  __nv_bfloat16* dq; long long dq_stride;
  __nv_bfloat16* dk; __nv_bfloat16* dv; long long dkv_stride;
  int* status;
};

// delta[b,h,i] = sum_d dO[i, h*hd + d] * O[i, h*hd + d]; hd / 8 lanes per (row, head), 16-byte loads.
__global__ void __launch_bounds__(256)
flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta, int batch,
                   int heads, int seq, int hd, long long o_stride, long long do_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int lpi = hd >> 3;                                   // lanes per item: 8 (hd 64) or 16 (hd 128)
  const long long total = (long long)batch * seq * heads;
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long item = t / lpi;
  const int sub = (int)(t % lpi);
  float s = 0.f;
  int h = 0;
  long long row = 0;
  if (item < total) {
    h = (int)(item % heads);
    row = item / heads;
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * o_stride + h * hd + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(dout + row * do_stride + h * hd + sub * 8);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
    s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
  }
  for (int off = lpi >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (item < total && sub == 0) {
    const int bi = (int)(row / seq), si = (int)(row % seq);
    delta[((long long)bi * heads + h) * seq + si] = s;
  }
}

constexpr int FA_BWD_THREADS = 384;   // 8 softmax warps + 3 MMA issuer warps (the dQ kernel uses 2) + 1 TMA warp

// Backward pipeline (both kernels).  The score products of a tile land in TMEM; the eight softmax warps (two threads
// per TMEM lane) copy them to registers and release the buffers at once, so the first MMA warp issues the score products
// of the NEXT tile while this tile's exponentials run.  The bf16 results (P^T and dS^T in the dK/dV kernel, dS in the dQ
// kernel) are written back to TMEM and are the A operands of the gradient products, which the second MMA warp issues:
// nothing passes through shared memory.  One tcgen05.mma costs about 50 cycles to issue from a thread and the
// N = head_dim products are issue bound, hence two issuing warps.
//
// The dK/dV kernel works on the TRANSPOSED tile, S^T = K Q^T with keys on the TMEM lanes, because dV = P^T dO and
// dK = dS^T Q need P^T / dS^T with keys as the M dimension.  Per-query statistics (log-sum-exp, delta) are then per
// COLUMN: the softmax warps stage them in shared memory (double buffered by iteration parity) and read them as broadcasts.
template <int HD>
struct BwdKvCfg {
  static constexpr int NST = (HD == 64) ? 3 : 2;       // Q / dO ring: a stage is held from the score products to the end of dK
  static constexpr bool ALIAS = HD != 64;               // head_dim 128: P^T / dS^T overwrite S^T / dP^T (no spare TMEM columns)
  static constexpr int T_BYTES = FA_BM * HD * 2;        // one [128 x HD] tile
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + T_BYTES;
  static constexpr int OFF_Q = OFF_V + T_BYTES;
  static constexpr int OFF_DO = OFF_Q + NST * T_BYTES;
  static constexpr int OFF_STAT = OFF_DO + NST * T_BYTES;   // float[NST][256]: -lse*log2e | -delta*scale of the query block
  static constexpr int OFF_BAR = OFF_STAT + NST * 256 * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 128;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0, TM_DP = 128;
  static constexpr int TM_P = ALIAS ? 0 : 256, TM_DS = ALIAS ? 128 : 320;
  static constexpr int TM_DV = ALIAS ? 256 : 384, TM_DK = TM_DV + HD;
};

// Persistent: one CTA per SM walks the work items (key block, head, batch) it owns, heaviest causal key blocks first, items
// dealt in snake order; dK, dV of an item accumulate in TMEM over its query blocks.  Barrier phases come from running counts.
template <int HD>
__global__ void __launch_bounds__(FA_BWD_THREADS, 1)
flash_bwd_kv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const FlashBwdParams p) {
  using Cfg = BwdKvCfg<HD>;
  constexpr int NST = Cfg::NST;
  constexpr bool ALIAS = Cfg::ALIAS;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* kv_empty = bars + 1;   // the item's last score products have read K, V
  uint64_t* qdo_full = bars + 2;   // [3]
  uint64_t* qdo_empty = bars + 5;  // [3]  (dV and dK issuers both arrive)
  uint64_t* s_full = bars + 8;     // S^T, dP^T of this tile are in TMEM
  uint64_t* s_empty = bars + 9;    // ... and have been copied to registers (8 warps)
  uint64_t* pds_full = bars + 10;  // P^T, dS^T of this tile are in TMEM (8 warps)
  uint64_t* pds_empty = bars + 11; // ... and have been consumed by the gradient products (dV and dK issuers both arrive)
  uint64_t* fin_full = bars + 12;  // dV, dK of the item are complete (both issuers arrive)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  float* stat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.seq + FA_BM - 1) / FA_BM;
  const int hb = p.heads * p.batch;
  const int n_items = nblk * hb;
  const int n_rounds = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  auto item_of = [&](int round) -> int {     // snake order; >= n_items: this CTA sits the round out
    return round * (int)gridDim.x + ((round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  };
  auto decode = [&](int item, int& jb, int& h, int& b) {   // key block 0 has the most query blocks under the causal mask
    jb = item / hb;
    const int rem = item % hb;
    h = rem % p.heads;
    b = rem / p.heads;
  };

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_error(p.status, OA_KERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    for (int s = 0; s < NST; ++s) { mbar_init(&qdo_full[s], 2); mbar_init(&qdo_empty[s], 2); }   // full: TMA bytes + the statistics
    mbar_init(s_full, 1);
    mbar_init(s_empty, 8);
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 2);
    mbar_init(fin_full, 2);
    mbar_fence_init();
  }
  if (warp == 8) { tmem_alloc<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                            // the prologue above ran under the previous kernel's tail; global memory from here on

  if (warp == 11) {
    // ------------- TMA producer (also stages the per-query statistics of each block)
    uint32_t itc = 0, qc = 0;       // items and Q / dO blocks loaded so far
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int jb, h, b;
      decode(item, jb, h, b);
      const int i0 = p.causal ? jb : 0, n_it = nblk - i0, row0 = b * p.seq;
      const long long stat_base = ((long long)b * p.heads + h) * p.seq;
      if (!warp_wait(kv_empty, (itc & 1) ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
      if (lane == 0) {
        mbar_expect_tx(kv_full, 2 * Cfg::T_BYTES);
#pragma unroll
        for (int x = 0; x < HD / 64; ++x) {
          tma_load_2d(smem + Cfg::OFF_K + x * (FA_BN * 128), &tmK, kv_full, h * HD + x * 64, row0 + jb * FA_BN);
          tma_load_2d(smem + Cfg::OFF_V + x * (FA_BN * 128), &tmV, kv_full, h * HD + x * 64, row0 + jb * FA_BN);
        }
      }
      for (int it = 0; it < n_it; ++it, ++qc) {
        const int st = qc % NST;
        const uint32_t ph = (qc / NST) & 1;
        if (!warp_wait(&qdo_empty[st], ph ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(&qdo_full[st], 2 * Cfg::T_BYTES);
          const int qrow = row0 + (i0 + it) * FA_BM;
#pragma unroll
          for (int x = 0; x < HD / 64; ++x) {
            tma_load_2d(smem + Cfg::OFF_Q + st * Cfg::T_BYTES + x * (FA_BM * 128), &tmQ, &qdo_full[st], h * HD + x * 64, qrow);
            tma_load_2d(smem + Cfg::OFF_DO + st * Cfg::T_BYTES + x * (FA_BM * 128), &tmDO, &qdo_full[st], h * HD + x * 64, qrow);
          }
        }
        // per-query statistics of this block, negated and pre-scaled: lane l stages queries 4l .. 4l+3
        {
          float4 nl, nd;
          float* nlp = reinterpret_cast<float*>(&nl);
          float* ndp = reinterpret_cast<float*>(&nd);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int qi = (i0 + it) * FA_BM + lane * 4 + u;
            const bool okq = qi < p.seq;
            nlp[u] = okq ? -p.lse[stat_base + qi] * LOG2E : -INFINITY;
            ndp[u] = okq ? -p.delta[stat_base + qi] * p.scale : 0.f;
          }
          float* dst = stat + st * 256;
          reinterpret_cast<float4*>(dst)[lane] = nl;
          reinterpret_cast<float4*>(dst + 128)[lane] = nd;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&qdo_full[st]);
        __syncwarp();
      }
      ++itc;
    }
  } else if (warp == 8) {
    // ------------- MMA issuer A: transposed score products S^T = K Q^T, dP^T = V dO^T
    constexpr uint32_t idesc_s = umma_idesc_bf16(FA_BN, FA_BM, 0, 0);
    const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K), v_addr = smem_u32(smem + Cfg::OFF_V);
    uint32_t itc = 0, qc = 0;
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int jb, h, b;
      decode(item, jb, h, b);
      const int n_it = nblk - (p.causal ? jb : 0);
      if (!warp_wait(kv_full, itc & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); break; }
      for (int it = 0; it < n_it; ++it, ++qc) {
        const int st = qc % NST;
        if (!warp_wait(&qdo_full[st], (qc / NST) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        // S^T / dP^T may be overwritten once the softmax warps hold the previous tile in registers; when P^T / dS^T share
        // those columns, only once the previous gradient products have consumed them
        if (qc > 0 && !warp_wait(ALIAS ? pds_empty : s_empty, (qc - 1) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_EMPTY); ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q + st * Cfg::T_BYTES);
          const uint32_t do_addr = smem_u32(smem + Cfg::OFF_DO + st * Cfg::T_BYTES);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
            umma_f16(tmem_base + Cfg::TM_S, umma_smem_desc_sw128(k_addr + off, 16, 1024),
                     umma_smem_desc_sw128(q_addr + off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
            umma_f16(tmem_base + Cfg::TM_DP, umma_smem_desc_sw128(v_addr + off, 16, 1024),
                     umma_smem_desc_sw128(do_addr + off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
          }
          umma_commit(s_full);
          if (it + 1 == n_it) umma_commit(kv_empty);
        }
        __syncwarp();
      }
      ++itc;
    }
  } else if (warp == 9 || warp == 10) {
    // ------------- MMA issuers B (warp 9: dV += P^T dO) and C (warp 10: dK += dS^T Q), A operands from TMEM
    constexpr uint32_t idesc_g = umma_idesc_bf16(FA_BN, HD, 0, 1);   // [keys x HD] += X^T[keys x q] (TMEM) * Y[q x HD]
    const bool is_dv = warp == 9;
    const uint32_t acc_addr = tmem_base + (is_dv ? Cfg::TM_DV : Cfg::TM_DK);
    const uint32_t a_addr = tmem_base + (is_dv ? Cfg::TM_P : Cfg::TM_DS);
    uint32_t qc = 0;
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int jb, h, b;
      decode(item, jb, h, b);
      const int n_it = nblk - (p.causal ? jb : 0);
      // the previous item's dV / dK were read by the softmax warps before they produced this item's first P^T, dS^T
      for (int it = 0; it < n_it; ++it, ++qc) {
        const int st = qc % NST;
        if (!warp_wait(&qdo_full[st], (qc / NST) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        if (!warp_wait(pds_full, qc & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_SOFTMAX); ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t b_addr = smem_u32(smem + (is_dv ? Cfg::OFF_DO : Cfg::OFF_Q) + st * Cfg::T_BYTES);
#pragma unroll
          for (int ks = 0; ks < FA_BM / 16; ++ks)    // reduction over the 128 queries of this block
            umma_f16_ts(acc_addr, a_addr + ks * 8, umma_smem_desc_sw128(b_addr + ks * 2048, FA_BM * 128, 1024), idesc_g,
                        (it > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&qdo_empty[st]);
          umma_commit(pds_empty);
          if (it + 1 == n_it) umma_commit(fin_full);
        }
        __syncwarp();
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = warp >> 2;                  // this thread owns query columns [64*half, 64*half+64) of the tile
    const int r = quad * 32 + lane;              // key row inside the block = TMEM lane
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    uint32_t itc = 0, qc = 0;
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int jb, h, b;
      decode(item, jb, h, b);
      const int i0 = p.causal ? jb : 0, n_it = nblk - i0, row0 = b * p.seq;
      for (int it = 0; it < n_it; ++it, ++qc) {
        const int ib = i0 + it;
        const int st = qc % NST;
        const float* st_cur = stat + st * 256;
        ok = warp_wait(&qdo_full[st], (qc / NST) & 1);   // statistics of this block are staged
        if (ok) ok = warp_wait(s_full, qc & 1);
        if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
        tc_fence_after();
        uint32_t s[64], dp[64];
        tmem_ld32(tmem_base + t_lane + Cfg::TM_S + half * 64, s);
        tmem_ld32(tmem_base + t_lane + Cfg::TM_S + half * 64 + 32, s + 32);
        tmem_ld32(tmem_base + t_lane + Cfg::TM_DP + half * 64, dp);
        tmem_ld32(tmem_base + t_lane + Cfg::TM_DP + half * 64 + 32, dp + 32);
        tmem_ld_wait();
        if (ALIAS) {
          pair_sync(quad);                         // both threads of the lane hold their columns before either overwrites them
        } else {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_empty);     // the next tile's score products may overwrite S^T, dP^T now
        }
        const float4* nl4 = reinterpret_cast<const float4*>(st_cur + half * 64);
        const float4* nd4 = reinterpret_cast<const float4*>(st_cur + 128 + half * 64);
        const bool diag = p.causal && ib == jb;    // alive iff key <= query: column >= row
        const int first = r - half * 64;           // first alive column of this thread on the diagonal tile
        uint32_t pw[32], dw[32];
        if (diag) {
#pragma unroll
          for (int i = 0; i < 64; i += 4) {
            const float4 nl = nl4[i >> 2], nd = nd4[i >> 2];
            const float p0 = (i >= first) ? fast_exp2(fmaf(__uint_as_float(s[i]), sl2, nl.x)) : 0.f;
            const float p1 = (i + 1 >= first) ? fast_exp2(fmaf(__uint_as_float(s[i + 1]), sl2, nl.y)) : 0.f;
            const float p2 = (i + 2 >= first) ? fast_exp2(fmaf(__uint_as_float(s[i + 2]), sl2, nl.z)) : 0.f;
            const float p3 = (i + 3 >= first) ? fast_exp2(fmaf(__uint_as_float(s[i + 3]), sl2, nl.w)) : 0.f;
            pw[i >> 1] = pack_bf16x2(p0, p1);
            pw[(i >> 1) + 1] = pack_bf16x2(p2, p3);
            dw[i >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(dp[i]), p.scale, nd.x), p1 * fmaf(__uint_as_float(dp[i + 1]), p.scale, nd.y));
            dw[(i >> 1) + 1] = pack_bf16x2(p2 * fmaf(__uint_as_float(dp[i + 2]), p.scale, nd.z), p3 * fmaf(__uint_as_float(dp[i + 3]), p.scale, nd.w));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 64; i += 4) {
            const float4 nl = nl4[i >> 2], nd = nd4[i >> 2];
            const float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), sl2, nl.x));
            const float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), sl2, nl.y));
            const float p2 = fast_exp2(fmaf(__uint_as_float(s[i + 2]), sl2, nl.z));
            const float p3 = fast_exp2(fmaf(__uint_as_float(s[i + 3]), sl2, nl.w));
            pw[i >> 1] = pack_bf16x2(p0, p1);
            pw[(i >> 1) + 1] = pack_bf16x2(p2, p3);
            dw[i >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(dp[i]), p.scale, nd.x), p1 * fmaf(__uint_as_float(dp[i + 1]), p.scale, nd.y));
            dw[(i >> 1) + 1] = pack_bf16x2(p2 * fmaf(__uint_as_float(dp[i + 2]), p.scale, nd.z), p3 * fmaf(__uint_as_float(dp[i + 3]), p.scale, nd.w));
          }
        }
        if (!ALIAS && qc > 0) {                     // the previous tile's gradient products still read P^T, dS^T
          ok = warp_wait(pds_empty, (qc - 1) & 1);
          if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
          tc_fence_after();
        }
        tmem_st32(tmem_base + t_lane + Cfg::TM_P + half * 32, pw);
        tmem_st32(tmem_base + t_lane + Cfg::TM_DS + half * 32, dw);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pds_full);
      }
      if (!ok) break;
      ok = warp_wait(fin_full, itc & 1);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      ++itc;
      tc_fence_after();
      const int kj = jb * FA_BN + r;   // accumulator rows are keys
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* base = (which == 0 ? p.dv : p.dk) + (long long)(row0 + kj) * p.dkv_stride + h * HD;
        const uint32_t tcol = which == 0 ? Cfg::TM_DV : Cfg::TM_DK;
#pragma unroll 1
        for (int cc = 0; cc < HD / 64; ++cc) {
          const int c = half * (HD / 64) + cc;
          uint32_t a[32];
          tmem_ld32(tmem_base + t_lane + tcol + c * 32, a);
          tmem_ld_wait();
          if (kj < p.seq) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
              *reinterpret_cast<uint4*>(base + c * 32 + g * 8) = make_uint4(
                  pack_bf16x2(__uint_as_float(a[g * 8]), __uint_as_float(a[g * 8 + 1])),
                  pack_bf16x2(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3])),
                  pack_bf16x2(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5])),
                  pack_bf16x2(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7])));
          }
        }
      }
      tc_fence_before();   // dV / dK are read before this warp's next pds_full arrival lets the next item's products overwrite them
    }
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) { tc_fence_after(); tmem_dealloc<Cfg::TMEM_COLS>(tmem_base); }
}

template <int HD>
struct BwdQCfg {
  static constexpr int NST = (HD == 64) ? 3 : 2;       // K / V ring
  static constexpr int T_BYTES = FA_BM * HD * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + T_BYTES;
  static constexpr int OFF_K = OFF_DO + T_BYTES;
  static constexpr int OFF_V = OFF_K + NST * T_BYTES;
  static constexpr int OFF_BAR = OFF_V + NST * T_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0, TM_DP = 128, TM_DS = 256, TM_DQ = 320;
};

// Persistent, like the dK / dV kernel: items are (query block, head, batch), heaviest causal query blocks first; dQ of an item
// accumulates in TMEM over its key blocks.
template <int HD>
__global__ void __launch_bounds__(FA_BWD_THREADS, 1)
flash_bwd_q_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const FlashBwdParams p) {
  using Cfg = BwdQCfg<HD>;
  constexpr int NST = Cfg::NST;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* q_empty = bars + 1;    // the item's last score products have read Q, dO
  uint64_t* kv_full = bars + 2;    // [3]
  uint64_t* kv_empty = bars + 5;   // [3]
  uint64_t* s_full = bars + 8;
  uint64_t* s_empty = bars + 9;
  uint64_t* ds_full = bars + 10;
  uint64_t* ds_empty = bars + 11;
  uint64_t* fin_full = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.seq + FA_BM - 1) / FA_BM;
  const int hb = p.heads * p.batch;
  const int n_items = nblk * hb;
  const int n_rounds = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
  auto item_of = [&](int round) -> int {
    return round * (int)gridDim.x + ((round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
  };
  auto decode = [&](int item, int& ib, int& h, int& b) {   // the last query block has the most key blocks under the causal mask
    ib = nblk - 1 - item / hb;
    const int rem = item % hb;
    h = rem % p.heads;
    b = rem / p.heads;
  };

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_error(p.status, OA_KERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < NST; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 8);
    mbar_init(ds_full, 8);
    mbar_init(ds_empty, 1);
    mbar_init(fin_full, 1);
    mbar_fence_init();
  }
  if (warp == 8) { tmem_alloc<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                            // the prologue above ran under the previous kernel's tail; global memory from here on

  if (warp == 10) {
    uint32_t itc = 0, kc = 0;
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int ib, h, b;
      decode(item, ib, h, b);
      const int n_kv = p.causal ? (ib + 1) : nblk, row0 = b * p.seq;
      if (!warp_wait(q_empty, (itc & 1) ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
      if (lane == 0) {
        mbar_expect_tx(q_full, 2 * Cfg::T_BYTES);
#pragma unroll
        for (int x = 0; x < HD / 64; ++x) {
          tma_load_2d(smem + Cfg::OFF_Q + x * (FA_BM * 128), &tmQ, q_full, h * HD + x * 64, row0 + ib * FA_BM);
          tma_load_2d(smem + Cfg::OFF_DO + x * (FA_BM * 128), &tmDO, q_full, h * HD + x * 64, row0 + ib * FA_BM);
        }
      }
      for (int j = 0; j < n_kv; ++j, ++kc) {
        const int st = kc % NST;
        const uint32_t ph = (kc / NST) & 1;
        if (!warp_wait(&kv_empty[st], ph ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(&kv_full[st], 2 * Cfg::T_BYTES);
#pragma unroll
          for (int x = 0; x < HD / 64; ++x) {
            tma_load_2d(smem + Cfg::OFF_K + st * Cfg::T_BYTES + x * (FA_BN * 128), &tmK, &kv_full[st], h * HD + x * 64, row0 + j * FA_BN);
            tma_load_2d(smem + Cfg::OFF_V + st * Cfg::T_BYTES + x * (FA_BN * 128), &tmV, &kv_full[st], h * HD + x * 64, row0 + j * FA_BN);
          }
        }
        __syncwarp();
      }
      ++itc;
    }
  } else if (warp == 8) {
    // ------------- MMA issuer A: S = Q K_j^T, dP = dO V_j^T
    constexpr uint32_t idesc_s = umma_idesc_bf16(FA_BM, FA_BN, 0, 0);
    const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q), do_addr = smem_u32(smem + Cfg::OFF_DO);
    uint32_t itc = 0, kc = 0;
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int ib, h, b;
      decode(item, ib, h, b);
      const int n_kv = p.causal ? (ib + 1) : nblk;
      if (!warp_wait(q_full, itc & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); break; }
      for (int j = 0; j < n_kv; ++j, ++kc) {
        const int st = kc % NST;
        if (!warp_wait(&kv_full[st], (kc / NST) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        if (kc > 0 && !warp_wait(s_empty, (kc - 1) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_EMPTY); ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K + st * Cfg::T_BYTES);
          const uint32_t v_addr = smem_u32(smem + Cfg::OFF_V + st * Cfg::T_BYTES);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
            umma_f16(tmem_base + Cfg::TM_S, umma_smem_desc_sw128(q_addr + off, 16, 1024),
                     umma_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
            umma_f16(tmem_base + Cfg::TM_DP, umma_smem_desc_sw128(do_addr + off, 16, 1024),
                     umma_smem_desc_sw128(v_addr + off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
          }
          umma_commit(s_full);
          if (j + 1 == n_kv) umma_commit(q_empty);
        }
        __syncwarp();
      }
      ++itc;
    }
  } else if (warp == 9) {
    // ------------- MMA issuer B: dQ += dS K_j (dS from TMEM)
    constexpr uint32_t idesc_q = umma_idesc_bf16(FA_BM, HD, 0, 1);   // dQ[q x HD] += dS[q x keys] * K[keys x HD]
    uint32_t kc = 0;
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int ib, h, b;
      decode(item, ib, h, b);
      const int n_kv = p.causal ? (ib + 1) : nblk;
      for (int j = 0; j < n_kv; ++j, ++kc) {
        const int st = kc % NST;
        if (!warp_wait(&kv_full[st], (kc / NST) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        if (!warp_wait(ds_full, kc & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_SOFTMAX); ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K + st * Cfg::T_BYTES);
#pragma unroll
          for (int ks = 0; ks < FA_BN / 16; ++ks)
            umma_f16_ts(tmem_base + Cfg::TM_DQ, tmem_base + Cfg::TM_DS + ks * 8,
                        umma_smem_desc_sw128(k_addr + ks * 2048, FA_BN * 128, 1024), idesc_q, (j > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&kv_empty[st]);
          umma_commit(ds_empty);
          if (j + 1 == n_kv) umma_commit(fin_full);
        }
        __syncwarp();
      }
    }
  } else if (warp < 8) {
    const int quad = warp & 3;
    const int half = warp >> 2;
    const int r = quad * 32 + lane;
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    uint32_t itc = 0, kc = 0;
    bool ok = true;
    for (int round = 0; round < n_rounds && ok; ++round) {
      const int item = item_of(round);
      if (item >= n_items) continue;
      int ib, h, b;
      decode(item, ib, h, b);
      const int n_kv = p.causal ? (ib + 1) : nblk, row0 = b * p.seq;
      const long long stat_base = ((long long)b * p.heads + h) * p.seq;
      const int qi = ib * FA_BM + r;
      const bool q_ok = qi < p.seq;
      const float lse2 = q_ok ? p.lse[stat_base + qi] * LOG2E : INFINITY;
      const float dlt = q_ok ? p.delta[stat_base + qi] : 0.f;
      const float nlse = -lse2, ndlt = -dlt * p.scale;
      for (int j = 0; j < n_kv; ++j, ++kc) {
        ok = warp_wait(s_full, kc & 1);
        if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
        tc_fence_after();
        uint32_t s[64], dp[64];
        tmem_ld32(tmem_base + t_lane + Cfg::TM_S + half * 64, s);
        tmem_ld32(tmem_base + t_lane + Cfg::TM_S + half * 64 + 32, s + 32);
        tmem_ld32(tmem_base + t_lane + Cfg::TM_DP + half * 64, dp);
        tmem_ld32(tmem_base + t_lane + Cfg::TM_DP + half * 64 + 32, dp + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty);
        const int k0 = j * FA_BN;
        const bool need_mask = (p.causal && j == ib) || (k0 + FA_BN > p.seq) || !q_ok;
        uint32_t dw[32];
        if (need_mask) {
          const int lim = q_ok ? (min(p.causal ? qi : 0x7fffffff, p.seq - 1) - (k0 + half * 64)) : -1;
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            const float p0 = (i <= lim) ? fast_exp2(fmaf(__uint_as_float(s[i]), sl2, nlse)) : 0.f;
            const float p1 = (i + 1 <= lim) ? fast_exp2(fmaf(__uint_as_float(s[i + 1]), sl2, nlse)) : 0.f;
            dw[i >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(dp[i]), p.scale, ndlt), p1 * fmaf(__uint_as_float(dp[i + 1]), p.scale, ndlt));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), sl2, nlse));
            const float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), sl2, nlse));
            dw[i >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(dp[i]), p.scale, ndlt), p1 * fmaf(__uint_as_float(dp[i + 1]), p.scale, ndlt));
          }
        }
        if (kc > 0) {
          ok = warp_wait(ds_empty, (kc - 1) & 1);
          if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
          tc_fence_after();
        }
        tmem_st32(tmem_base + t_lane + Cfg::TM_DS + half * 32, dw);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_full);
      }
      if (!ok) break;
      ok = warp_wait(fin_full, itc & 1);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      ++itc;
      tc_fence_after();
      __nv_bfloat16* base = p.dq + (long long)(row0 + qi) * p.dq_stride + h * HD;
#pragma unroll 1
      for (int cc = 0; cc < HD / 64; ++cc) {
        const int c = half * (HD / 64) + cc;
        uint32_t a[32];
        tmem_ld32(tmem_base + t_lane + Cfg::TM_DQ + c * 32, a);
        tmem_ld_wait();
        if (q_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(base + c * 32 + g * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(a[g * 8]), __uint_as_float(a[g * 8 + 1])),
                pack_bf16x2(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3])),
                pack_bf16x2(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5])),
                pack_bf16x2(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7])));
        }
      }
      tc_fence_before();   // dQ is read before this warp's next ds_full arrival lets the next item's products overwrite it
    }
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) { tc_fence_after(); tmem_dealloc<Cfg::TMEM_COLS>(tmem_base); }
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer);

}  // namespace oa

using namespace oa;

extern "C" int oa_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int heads,
                            int seq, int head_dim, long long q_row_stride, long long kv_row_stride,
                            long long o_row_stride, float scale, int causal, int* status, void* stream) {
  if (head_dim != 64 && head_dim != 128) return OA_ERR_UNSUPPORTED;
  if (batch <= 0 || heads <= 0 || seq <= 0) return OA_ERR_ARG;
  if ((o_row_stride & 7) || (reinterpret_cast<uintptr_t>(o) & 15)) return OA_ERR_ALIGN;
  CUtensorMap tq, tk, tv;
  int rc;
  uint64_t rows = (uint64_t)batch * seq, width = (uint64_t)heads * head_dim;
  if ((rc = make_tmap_2d_bf16(&tq, q, width, rows, (uint64_t)q_row_stride, 64, FA_BM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tk, k, width, rows, (uint64_t)kv_row_stride, 64, FA_BN))) return rc;
  if ((rc = make_tmap_2d_bf16(&tv, v, width, rows, (uint64_t)kv_row_stride, 64, FA_BN))) return rc;
  FlashParams p;
  p.batch = batch; p.heads = heads; p.seq = seq; p.head_dim = head_dim; p.scale = scale; p.causal = causal;
  p.o = (__nv_bfloat16*)o; p.o_stride = o_row_stride; p.lse = lse; p.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  if (head_dim == 64) {
    // persistent kernel, two query tiles per work item
    static int sms = 0;
    if (sms == 0) {
      int dev = 0;
      if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return OA_ERR_DRIVER;
      if (cudaFuncSetAttribute(flash_fwd_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdPairCfg::SMEM_BYTES) != cudaSuccess) return OA_ERR_LAUNCH;
    }
    const int nblk = (seq + FA_BM - 1) / FA_BM;
    const long long items = (long long)((nblk + 1) / 2) * heads * batch;
    const int ctas = (int)(items < sms ? items : sms);
    launch_pdl(flash_fwd_pair_kernel, dim3(ctas), dim3(FwdPairCfg::THREADS), FwdPairCfg::SMEM_BYTES, st, tq, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
  }
  return launch_fwd2<128>(tq, tk, tv, p, dim3((seq + FA_BM - 1) / FA_BM, heads, batch), st);
}

// scratch: float[B*H*S] for delta
extern "C" size_t oa_flash_bwd_scratch_bytes(int batch, int heads, int seq, int head_dim) {
  (void)head_dim;
  return (size_t)batch * heads * seq * sizeof(float);
}

template <typename K>
static int set_max_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

extern "C" int oa_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                            const float* lse, void* dq, void* dk, void* dv, int batch, int heads, int seq, int head_dim,
                            long long q_row_stride, long long kv_row_stride, long long o_row_stride,
                            long long dq_row_stride, long long dkv_row_stride, float scale, int causal, float* scratch,
                            int* status, void* stream) {
  if (head_dim != 64 && head_dim != 128) return OA_ERR_UNSUPPORTED;
  if (batch <= 0 || heads <= 0 || seq <= 0) return OA_ERR_ARG;
  if ((dq_row_stride & 7) || (dkv_row_stride & 7) || (reinterpret_cast<uintptr_t>(dq) & 15) ||
      (reinterpret_cast<uintptr_t>(dk) & 15) || (reinterpret_cast<uintptr_t>(dv) & 15))
    return OA_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  uint64_t rows = (uint64_t)batch * seq, width = (uint64_t)heads * head_dim;
  if ((rc = make_tmap_2d_bf16(&tq, q, width, rows, (uint64_t)q_row_stride, 64, FA_BM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tk, k, width, rows, (uint64_t)kv_row_stride, 64, FA_BN))) return rc;
  if ((rc = make_tmap_2d_bf16(&tv, v, width, rows, (uint64_t)kv_row_stride, 64, FA_BN))) return rc;
  if ((rc = make_tmap_2d_bf16(&tdo, dout, width, rows, (uint64_t)o_row_stride, 64, FA_BM))) return rc;
  {
    long long threads = (long long)batch * seq * heads * (head_dim / 8);
    unsigned blocks = (unsigned)((threads + 255) / 256);
    launch_pdl(flash_delta_kernel, dim3(blocks), dim3(256), 0, st, (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, scratch, batch, heads,
               seq, head_dim, o_row_stride, o_row_stride);
  }
  FlashBwdParams p;
  p.batch = batch; p.heads = heads; p.seq = seq; p.head_dim = head_dim; p.scale = scale; p.causal = causal;
  p.lse = lse; p.delta = scratch;
  p.dq = (__nv_bfloat16*)dq; p.dq_stride = dq_row_stride;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.dkv_stride = dkv_row_stride;
  p.status = status;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return OA_ERR_DRIVER;
  }
  const long long items = (long long)((seq + FA_BM - 1) / FA_BM) * heads * batch;
  const dim3 grid((unsigned)(items < sms ? items : sms));     // persistent: one CTA per SM walks its items
  if (head_dim == 64) {
    static bool set = false;
    if (!set) {
      if ((rc = set_max_smem(flash_bwd_kv_kernel<64>, BwdKvCfg<64>::SMEM_BYTES))) return rc;
      if ((rc = set_max_smem(flash_bwd_q_kernel<64>, BwdQCfg<64>::SMEM_BYTES))) return rc;
      set = true;
    }
    launch_pdl(flash_bwd_kv_kernel<64>, dim3(grid), dim3(FA_BWD_THREADS), BwdKvCfg<64>::SMEM_BYTES, st, tq, tk, tv, tdo, p);
    launch_pdl(flash_bwd_q_kernel<64>, dim3(grid), dim3(FA_BWD_THREADS), BwdQCfg<64>::SMEM_BYTES, st, tq, tk, tv, tdo, p);
  } else {
    static bool set = false;
    if (!set) {
      if ((rc = set_max_smem(flash_bwd_kv_kernel<128>, BwdKvCfg<128>::SMEM_BYTES))) return rc;
      if ((rc = set_max_smem(flash_bwd_q_kernel<128>, BwdQCfg<128>::SMEM_BYTES))) return rc;
      set = true;
    }
    launch_pdl(flash_bwd_kv_kernel<128>, dim3(grid), dim3(FA_BWD_THREADS), BwdKvCfg<128>::SMEM_BYTES, st, tq, tk, tv, tdo, p);
    launch_pdl(flash_bwd_q_kernel<128>, dim3(grid), dim3(FA_BWD_THREADS), BwdQCfg<128>::SMEM_BYTES, st, tq, tk, tv, tdo, p);
  }
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}
