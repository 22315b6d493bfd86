// Causal / full scaled-dot-product attention for sm_100a, forward and backward, bf16 in / fp32 accumulate.
//
// The reference's FlashCausal kernels (Source/Private/Oa/Ml/Shader/Compute/Nn/Attention/FlashCausal*.slang)
// run one work-group per query row with all scores of the row in shared memory (S <= 1024, fp32 only, no
// tensor cores).  Here the work is tiled 128 queries x 128 keys, both matrix products of a tile run on
// tcgen05 with accumulators in TMEM, tiles arrive through TMA, and softmax runs one thread per query row on
// values read straight from TMEM (no shuffles).  Q, K, V are read in place from a packed projection output
// ([B*S, row_stride] with head h at column h*head_dim), and O is written merged ([B*S, H*head_dim]), so there
// are no SplitHeads / MergeHeads passes.
//
// Backward is two kernels, both deterministic (single writer per output element, like the reference's
// FlashCausalBwdQ / FlashCausalBwdKV): one CTA per key block accumulates dK, dV in TMEM over the query blocks,
// one CTA per query block accumulates dQ in TMEM over the key blocks.  Probabilities are recomputed from the
// saved log-sum-exp.
//
// CTA = 320 threads: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM owner), warps 2..9 = softmax /
// epilogue.  Two threads share a query row: warp w works on TMEM lane quadrant w % 4 and on key columns
// [64*half, 64*half+64) with half = (w-2)/4, which doubles the warps available to hide TMEM-load and
// exp latency.  Every wait is bounded and reports to a status word.
#include "common.cuh"
#include "api.h"
#include <stdlib.h>

namespace oa {

constexpr int FA_BM = 128;   // queries per tile
constexpr int FA_BN = 128;   // keys per tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr int FA_THREADS = 320;   // 2 service warps + 8 softmax warps

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

// Byte offset of element (row, col) in a [rows x 64] bf16 box stored with the 128-byte swizzle
// (16-byte chunk index XOR (row % 8)); boxes of 64 columns are `box_bytes` apart.
__device__ __forceinline__ uint32_t sw128_offset(int row, int col, int box_bytes) {
  int box = col >> 6, c = col & 63;
  return box * box_bytes + row * 128 + ((((c >> 3) ^ (row & 7)) << 4) | ((c & 7) << 1));
}

template <int HD>
struct FwdCfg {
  static constexpr int Q_BYTES = FA_BM * HD * 2;
  static constexpr int KV_BYTES = FA_BN * HD * 2;
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;
  static constexpr int STAGES = 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128;
  static constexpr int TMEM_COLS = 256;
  static constexpr int TM_S = 0;
  static constexpr int TM_O = 128;
};

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, HD == 64 ? 2 : 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  using Cfg = FwdCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* v_full = bars + 3;   // [2]
  uint64_t* kv_empty = bars + 5; // [2]  V stage free (P*V done)
  uint64_t* k_empty = bars + 11; // [2]  K stage free (Q*K^T done): lets the next K load start one iteration earlier
  uint64_t* s_full = bars + 7;
  uint64_t* p_full = bars + 8;
  uint64_t* o_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.seq + FA_BM - 1) / FA_BM;
  const int qb = nblk - 1 - blockIdx.x;  // heaviest causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int n_kv = p.causal ? (qb + 1) : nblk;
  const int row0 = b * p.seq;            // first row of this batch element in the [B*S, .] matrices

  if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) report_error(p.status, OA_KERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&kv_empty[s], 1); mbar_init(&k_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);
    mbar_init(o_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------- producer.  The whole warp walks the loop and waits together; one lane issues the copies.
    // (A warp split between a spinning lane and 31 lanes parked at the final barrier hands off very slowly.)
    if (lane == 0) {
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int x = 0; x < HD / 64; ++x)
        tma_load_2d(smem + Cfg::OFF_Q + x * (FA_BM * 128), &tmQ, q_full, h * HD + x * 64, row0 + qb * FA_BM);
    }
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!warp_wait(&k_empty[st], ph ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
      if (lane == 0) {
        mbar_expect_tx(&k_full[st], Cfg::KV_BYTES);
#pragma unroll
        for (int x = 0; x < HD / 64; ++x)
          tma_load_2d(smem + Cfg::OFF_K + st * Cfg::KV_BYTES + x * (FA_BN * 128), &tmK, &k_full[st], h * HD + x * 64, row0 + j * FA_BN);
      }
      if (!warp_wait(&kv_empty[st], ph ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
      if (lane == 0) {
        mbar_expect_tx(&v_full[st], Cfg::KV_BYTES);
#pragma unroll
        for (int x = 0; x < HD / 64; ++x)
          tma_load_2d(smem + Cfg::OFF_V + st * Cfg::KV_BYTES + x * (FA_BN * 128), &tmV, &v_full[st], h * HD + x * 64, row0 + j * FA_BN);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------- MMA issuer (warp-uniform waits, lane 0 issues)
    constexpr uint32_t idesc_qk = umma_idesc_bf16(FA_BM, FA_BN, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(FA_BM, HD, 0, 1);
    const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q);
    const uint32_t p_addr = smem_u32(smem + Cfg::OFF_P);
    bool ok = warp_wait(q_full, 0);
    if (!ok && lane == 0) report_error(p.status, OA_KERR_WAIT_FULL);
    auto issue_qk = [&](int j) -> bool {
      const int st = j & 1;
      if (!warp_wait(&k_full[st], (j >> 1) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); return false; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K + st * Cfg::KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_S, umma_smem_desc_sw128(q_addr + off, 16, 1024),
                   umma_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(s_full);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < n_kv && ok; ++j) {
      const int st = j & 1;
      if (!warp_wait(p_full, j & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_SOFTMAX); break; }
      if (!warp_wait(&v_full[st], (j >> 1) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = smem_u32(smem + Cfg::OFF_V + st * Cfg::KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          uint32_t a_off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_O, umma_smem_desc_sw128(p_addr + a_off, 16, 1024),
                   umma_smem_desc_sw128(v_addr + ks * 2048, FA_BN * 128, 1024), idesc_pv, ks > 0 ? 1u : 0u);
        }
        umma_commit(&kv_empty[st]);
        umma_commit(o_full);
      }
      __syncwarp();
      if (j + 1 < n_kv) ok = issue_qk(j + 1);
    }
  } else {
    // ------------- softmax + output: two threads per query row (key columns split in halves)
    constexpr int OC = HD / 2;                   // output columns owned by this thread
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int qi = qb * FA_BM + r;               // query index inside the sequence
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[OC];
#pragma unroll
    for (int d = 0; d < OC; ++d) acc[d] = 0.f;
    uint8_t* sP = smem + Cfg::OFF_P;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      ok = warp_wait(s_full, j & 1);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      const int k0 = j * FA_BN + half * 64;
      const bool need_mask = (p.causal && j == qb) || (j * FA_BN + FA_BN > p.seq);
      const uint32_t s_addr = tmem_base + t_lane + Cfg::TM_S + half * 64;
      // pass 1: maximum over this thread's 64 key columns.  Masked tiles (the diagonal one and the sequence tail)
      // take a separate loop so that the common loop carries no per-element predicate.
      float mx = -INFINITY;
      if (need_mask) {
        const int lim = min(p.causal ? qi : 0x7fffffff, p.seq - 1) - k0;   // columns i <= lim are alive
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t sv[32];
          tmem_ld32(s_addr + c * 32, sv);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, (c * 32 + i <= lim) ? __uint_as_float(sv[i]) : -INFINITY);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t sv[32];
          tmem_ld32(s_addr + c * 32, sv);
          tmem_ld_wait();
          float m0 = __uint_as_float(sv[0]), m1 = __uint_as_float(sv[1]), m2 = __uint_as_float(sv[2]), m3 = __uint_as_float(sv[3]);
#pragma unroll
          for (int i = 4; i < 32; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(sv[i])); m1 = fmaxf(m1, __uint_as_float(sv[i + 1]));
            m2 = fmaxf(m2, __uint_as_float(sv[i + 2])); m3 = fmaxf(m3, __uint_as_float(sv[i + 3]));
          }
          mx = fmaxf(mx, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
        }
      }
      // Exchange with the partner thread.  The slot is the first word of the PARTNER's own row of the P tile: the
      // P tile is idle here (the previous P*V has completed before s_full fires) and only the slot's reader
      // overwrites it later.
      float* slot_mine = reinterpret_cast<float*>(sP + half * (FA_BM * 128) + r * 128);
      float* slot_partner = reinterpret_cast<float*>(sP + (half ^ 1) * (FA_BM * 128) + r * 128);
      *slot_partner = mx;
      pair_sync(quad);
      mx = fmaxf(mx, *slot_mine);
      const float m_new = fmaxf(m_run, mx * sl2);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;   // fully masked row so far
      const float alpha = fast_exp2(m_run - m_use);             // m_run = -inf -> 0
      const float neg_m = -m_use;
      float l0 = 0.f, l1 = 0.f;
      uint8_t* prow = sP + half * (FA_BM * 128) + r * 128;       // this thread's 128-byte row of box `half`
      const int rx = r & 7;
      // pass 2: probabilities -> bf16 -> swizzled smem tile (A operand of P*V)
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32];
        tmem_ld32(s_addr + c * 32, sv);
        tmem_ld_wait();
        uint32_t pk[16];
        if (need_mask) {
          const int lim = min(p.causal ? qi : 0x7fffffff, p.seq - 1) - k0 - c * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float e0 = (i <= lim) ? fast_exp2(fmaf(__uint_as_float(sv[i]), sl2, neg_m)) : 0.f;
            float e1 = (i + 1 <= lim) ? fast_exp2(fmaf(__uint_as_float(sv[i + 1]), sl2, neg_m)) : 0.f;
            l0 += e0; l1 += e1;
            pk[i >> 1] = pack_bf16x2(e0, e1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float e0 = fast_exp2(fmaf(__uint_as_float(sv[i]), sl2, neg_m));
            float e1 = fast_exp2(fmaf(__uint_as_float(sv[i + 1]), sl2, neg_m));
            l0 += e0; l1 += e1;
            pk[i >> 1] = pack_bf16x2(e0, e1);
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4*>(prow + (((c * 4 + g) ^ rx) << 4)) = make_uint4(pk[g * 4], pk[g * 4 + 1], pk[g * 4 + 2], pk[g * 4 + 3]);
      }
      l_run = l_run * alpha + (l0 + l1);
      m_run = m_new;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // accumulate the partial output of this key block (this thread's half of the head dimension)
      ok = warp_wait(o_full, j & 1);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_base + t_lane + Cfg::TM_O + half * OC + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(acc[c * 32 + i], alpha, __uint_as_float(o[i]));
      }
      tc_fence_before();
    }
    // combine the two partial row sums (same exchange slots; the last P*V has completed)
    {
      float* slot_mine = reinterpret_cast<float*>(sP + half * (FA_BM * 128) + r * 128);
      float* slot_partner = reinterpret_cast<float*>(sP + (half ^ 1) * (FA_BM * 128) + r * 128);
      *slot_partner = l_run;
      pair_sync(quad);
      l_run += *slot_mine;
    }
    if (ok && qi < p.seq) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* op = p.o + (long long)(row0 + qi) * p.o_stride + h * HD + half * OC;
#pragma unroll
      for (int g = 0; g < OC / 8; ++g)
        *reinterpret_cast<uint4*>(op + g * 8) =
            make_uint4(pack_bf16x2(acc[g * 8] * inv, acc[g * 8 + 1] * inv), pack_bf16x2(acc[g * 8 + 2] * inv, acc[g * 8 + 3] * inv),
                       pack_bf16x2(acc[g * 8 + 4] * inv, acc[g * 8 + 5] * inv), pack_bf16x2(acc[g * 8 + 6] * inv, acc[g * 8 + 7] * inv));
      if (p.lse && half == 0) p.lse[((long long)b * p.heads + h) * p.seq + qi] = (m_run + log2f(l_run)) / LOG2E;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc<Cfg::TMEM_COLS>(tmem_base); }
}

// ===================================================================================== forward, two query tiles per CTA
// One CTA owns two adjacent 128-query tiles of one (batch, head) and walks the key blocks once for both.  The tensor pipe
// alternates between the tiles (S_t = Q_t K^T, O_t += P_t V), so the products of one tile run while the other tile's
// softmax occupies the SFU / FMA pipes:
//   warps 0-3  softmax of tile 0, warps 4-7 softmax of tile 1: ONE thread per query row (TMEM lane = row), the whole
//              128-column score row is read from TMEM once, the row maximum and sum stay in registers (no shuffles, no
//              exchange through shared memory), probabilities go back to TMEM as packed bf16 over the columns of S;
//   warp 8     MMA issuer: P is the A operand straight from TMEM, V the B operand from shared memory, O accumulates in
//              TMEM over all key blocks and is read once at the end;
//   warp 9     TMA producer (Q tiles once, K / V rings).
// The running maximum is updated lazily: while the new row maximum exceeds the one in use by less than 2^8 the old one
// is kept (probabilities then stay below 256, exact in fp32 / safe in bf16), so O in TMEM is rescaled only in the
// rare iterations where some row of a warp jumps by more than that; the final 1/l uses the same maxima, so the result is
// the exact softmax.  TMEM: S0 | S1 | O0 | O1 = 128 + 128 + 2 * head_dim columns.
template <int HD>
struct Fwd2Cfg {
  static constexpr int NS = (HD == 64) ? 3 : 2;           // K / V ring depth
  static constexpr int Q_BYTES = FA_BM * HD * 2;          // one query tile
  static constexpr int KV_BYTES = FA_BN * HD * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + NS * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + NS * KV_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0;                           // + 128 * tile
  static constexpr int TM_O = 256;                         // + HD * tile
};

constexpr float FA_RESCALE_THRESHOLD = 8.f;                // log2 units

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FlashParams p) {
  using Cfg = Fwd2Cfg<HD>;
  constexpr int NS = Cfg::NS;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;             // [NS]
  uint64_t* v_full = bars + 1 + NS;        // [NS]
  uint64_t* k_empty = bars + 1 + 2 * NS;   // [NS]
  uint64_t* v_empty = bars + 1 + 3 * NS;   // [NS]
  uint64_t* s_full = bars + 1 + 4 * NS;    // [2]  S_t holds Q_t K_j^T
  uint64_t* p_full = s_full + 2;           // [2]  P_t written (and O_t rescaled if needed)
  uint64_t* o_done = s_full + 4;           // [2]  O_t += P_t V_j finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 6);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.seq + FA_BM - 1) / FA_BM;
  const int npair = (nblk + 1) >> 1;
  const int pr = npair - 1 - blockIdx.x;   // heaviest causal pairs first
  const int h = blockIdx.y, b = blockIdx.z;
  const int row0 = b * p.seq;
  const int nkv0 = p.causal ? (2 * pr + 1) : nblk;                                  // key blocks of tile 0 (query block 2 pr)
  const int nkv1 = (2 * pr + 1 < nblk) ? (p.causal ? (2 * pr + 2) : nblk) : 0;      // tile 1 (query block 2 pr + 1), 0 = absent
  const int n_it = max(nkv0, nkv1);

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_error(p.status, OA_KERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    mbar_init(q_full, 1);
    for (int s = 0; s < NS; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 4); mbar_init(&o_done[t], 1); }
    mbar_fence_init();
  }
  if (warp == 8) { tmem_alloc<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 9) {
    // ------------- producer: the whole warp walks the loop and waits together; one lane issues the copies
    if (lane == 0) {
      mbar_expect_tx(q_full, (nkv1 > 0 ? 2 : 1) * Cfg::Q_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (t == 0 || nkv1 > 0)
#pragma unroll
          for (int x = 0; x < HD / 64; ++x)
            tma_load_2d(smem + Cfg::OFF_Q + t * Cfg::Q_BYTES + x * (FA_BM * 128), &tmQ, q_full, h * HD + x * 64, row0 + (2 * pr + t) * FA_BM);
    }
    for (int j = 0; j < n_it; ++j) {
      const int st = j % NS;
      const uint32_t ph = (j / NS) & 1;
      if (!warp_wait(&k_empty[st], ph ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
      if (lane == 0) {
        mbar_expect_tx(&k_full[st], Cfg::KV_BYTES);
#pragma unroll
        for (int x = 0; x < HD / 64; ++x)
          tma_load_2d(smem + Cfg::OFF_K + st * Cfg::KV_BYTES + x * (FA_BN * 128), &tmK, &k_full[st], h * HD + x * 64, row0 + j * FA_BN);
      }
      if (!warp_wait(&v_empty[st], ph ^ 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
      if (lane == 0) {
        mbar_expect_tx(&v_full[st], Cfg::KV_BYTES);
#pragma unroll
        for (int x = 0; x < HD / 64; ++x)
          tma_load_2d(smem + Cfg::OFF_V + st * Cfg::KV_BYTES + x * (FA_BN * 128), &tmV, &v_full[st], h * HD + x * 64, row0 + j * FA_BN);
      }
      __syncwarp();
    }
  } else if (warp == 8) {
    // ------------- MMA issuer (warp-uniform waits, lane 0 issues)
    constexpr uint32_t idesc_qk = umma_idesc_bf16(FA_BM, FA_BN, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(FA_BM, HD, 0, 1);
    const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q);
    auto issue_qk = [&](int t, int st) {
      if (lane == 0) {
        const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K + st * Cfg::KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_S + t * FA_BN, umma_smem_desc_sw128(q_addr + t * Cfg::Q_BYTES + off, 16, 1024),
                   umma_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      }
      __syncwarp();
    };
    bool ok = warp_wait(q_full, 0);
    if (ok) ok = warp_wait(&k_full[0], 0);
    if (!ok && lane == 0) report_error(p.status, OA_KERR_WAIT_FULL);
    if (ok) {
      tc_fence_after();
      issue_qk(0, 0);
      if (nkv1 > 0) issue_qk(1, 0);
      if (lane == 0) umma_commit(&k_empty[0]);
      __syncwarp();
    }
    for (int j = 0; j < n_it && ok; ++j) {
      const int st = j % NS;
      const int stn = (j + 1) % NS;
      const bool has_next = j + 1 < n_it;
      if (!warp_wait(&v_full[st], (j / NS) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); break; }
      if (has_next && !warp_wait(&k_full[stn], ((j + 1) / NS) & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_FULL); break; }
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const int n_t = t == 0 ? nkv0 : nkv1;
        if (j >= n_t) continue;
        if (!warp_wait(&p_full[t], j & 1)) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_SOFTMAX); ok = false; break; }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t v_addr = smem_u32(smem + Cfg::OFF_V + st * Cfg::KV_BYTES);
#pragma unroll
          for (int ks = 0; ks < FA_BN / 16; ++ks)
            umma_f16_ts(tmem_base + Cfg::TM_O + t * HD, tmem_base + Cfg::TM_S + t * FA_BN + ks * 8,
                        umma_smem_desc_sw128(v_addr + ks * 2048, FA_BN * 128, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&o_done[t]);
        }
        __syncwarp();
        if (j + 1 < n_t) issue_qk(t, stn);
      }
      if (!ok) break;
      if (lane == 0) {
        umma_commit(&v_empty[st]);
        if (has_next) umma_commit(&k_empty[stn]);
      }
      __syncwarp();
    }
  } else {
    // ------------- softmax + output: one thread per query row
    const int t = warp >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int qbt = 2 * pr + t;                   // this tile's query block
    const int qi = qbt * FA_BM + r;               // query index inside the sequence
    const int n = t == 0 ? nkv0 : nkv1;
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const uint32_t s_addr = tmem_base + t_lane + Cfg::TM_S + t * FA_BN;
    const uint32_t o_addr = tmem_base + t_lane + Cfg::TM_O + t * HD;
    const float sl2 = p.scale * LOG2E;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      ok = warp_wait(&s_full[t], j & 1);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      uint32_t sv[FA_BN];
#pragma unroll
      for (int c = 0; c < FA_BN / 32; ++c) tmem_ld32(s_addr + c * 32, sv + c * 32);
      tmem_ld_wait();
      const bool need_mask = (p.causal && j == qbt) || (j * FA_BN + FA_BN > p.seq);
      if (need_mask) {
        const int lim = min(p.causal ? qi : 0x7fffffff, p.seq - 1) - j * FA_BN;   // columns i <= lim are alive
#pragma unroll
        for (int i = 0; i < FA_BN; ++i) sv[i] = (i <= lim) ? sv[i] : 0xff800000u;  // -inf
      }
      float m0 = __uint_as_float(sv[0]), m1 = __uint_as_float(sv[1]), m2 = __uint_as_float(sv[2]), m3 = __uint_as_float(sv[3]);
#pragma unroll
      for (int i = 4; i < FA_BN; i += 4) {
        m0 = fmaxf(m0, __uint_as_float(sv[i])); m1 = fmaxf(m1, __uint_as_float(sv[i + 1]));
        m2 = fmaxf(m2, __uint_as_float(sv[i + 2])); m3 = fmaxf(m3, __uint_as_float(sv[i + 3]));
      }
      const float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * sl2;
      const float m_new = fmaxf(m_run, mx);
      const bool grow = (m_new - m_run) > FA_RESCALE_THRESHOLD;           // first block: m_run = -inf -> true
      const float m_cand = grow ? m_new : m_run;
      const float m_use = (m_cand == -INFINITY) ? 0.f : m_cand;           // row fully masked so far
      const float alpha = grow ? fast_exp2(m_run - m_use) : 1.f;           // m_run = -inf -> 0
      const float neg_m = -m_use;
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
        tmem_st16(s_addr + c * 16, pk);          // P over the first 64 columns of S (two keys per column)
      }
      l_run = l_run * alpha + ((l0 + l1) + (l2 + l3));
      m_run = m_cand;
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // some row of this warp moved its maximum: rescale O (needs the previous P*V finished)
        ok = warp_wait(&o_done[t], (j - 1) & 1);
        if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
        tc_fence_after();
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
    if (ok && n > 0) {
      ok = warp_wait(&o_done[t], (n - 1) & 1);
      if (!ok && lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL);
    }
    if (ok && n > 0) {
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
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) { tc_fence_after(); tmem_dealloc<Cfg::TMEM_COLS>(tmem_base); }
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

template <int HD>
struct BwdKvCfg {
  static constexpr int NST = (HD == 64) ? 2 : 1;
  static constexpr int T_BYTES = FA_BM * HD * 2;        // one [128 x HD] tile
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + T_BYTES;
  static constexpr int OFF_Q = OFF_V + T_BYTES;
  static constexpr int OFF_DO = OFF_Q + NST * T_BYTES;
  static constexpr int OFF_P = OFF_DO + NST * T_BYTES;
  static constexpr int OFF_DS = OFF_P + P_BYTES;
  static constexpr int OFF_BAR = OFF_DS + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 256 + HD;
};

// One CTA per (key block, head, batch): dK, dV accumulate in TMEM over the query blocks.
template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_bwd_kv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const FlashBwdParams p) {
  using Cfg = BwdKvCfg<HD>;
  constexpr int NST = Cfg::NST;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;   // [2]
  uint64_t* qdo_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* pds_full = bars + 6;
  uint64_t* fin_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.seq + FA_BM - 1) / FA_BM;
  const int jb = blockIdx.x;                     // key block (light causal tiles are the high jb: launched last)
  const int h = blockIdx.y, b = blockIdx.z;
  const int i0 = p.causal ? jb : 0;
  const int n_it = nblk - i0;
  const int row0 = b * p.seq;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_error(p.status, OA_KERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&qdo_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(fin_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * Cfg::T_BYTES);
#pragma unroll
      for (int x = 0; x < HD / 64; ++x) {
        tma_load_2d(smem + Cfg::OFF_K + x * (FA_BN * 128), &tmK, kv_full, h * HD + x * 64, row0 + jb * FA_BN);
        tma_load_2d(smem + Cfg::OFF_V + x * (FA_BN * 128), &tmV, kv_full, h * HD + x * 64, row0 + jb * FA_BN);
      }
      for (int it = 0; it < n_it; ++it) {
        int st = it % NST;
        uint32_t ph = (it / NST) & 1;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1)) { report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
        mbar_expect_tx(&qdo_full[st], 2 * Cfg::T_BYTES);
        int qrow = row0 + (i0 + it) * FA_BM;
#pragma unroll
        for (int x = 0; x < HD / 64; ++x) {
          tma_load_2d(smem + Cfg::OFF_Q + st * Cfg::T_BYTES + x * (FA_BM * 128), &tmQ, &qdo_full[st], h * HD + x * 64, qrow);
          tma_load_2d(smem + Cfg::OFF_DO + st * Cfg::T_BYTES + x * (FA_BM * 128), &tmDO, &qdo_full[st], h * HD + x * 64, qrow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(FA_BM, FA_BN, 0, 0);
      constexpr uint32_t idesc_g = umma_idesc_bf16(FA_BN, HD, 1, 1);   // [keys x HD] += X^T[keys x q] * Y[q x HD]
      const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K), v_addr = smem_u32(smem + Cfg::OFF_V);
      const uint32_t p_addr = smem_u32(smem + Cfg::OFF_P), ds_addr = smem_u32(smem + Cfg::OFF_DS);
      bool ok = mbar_wait(kv_full, 0);
      if (!ok) report_error(p.status, OA_KERR_WAIT_FULL);
      for (int it = 0; it < n_it && ok; ++it) {
        int st = it % NST;
        if (!mbar_wait(&qdo_full[st], (it / NST) & 1)) { report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        tc_fence_after();
        const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q + st * Cfg::T_BYTES);
        const uint32_t do_addr = smem_u32(smem + Cfg::OFF_DO + st * Cfg::T_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_S, umma_smem_desc_sw128(q_addr + off, 16, 1024),
                   umma_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_DP, umma_smem_desc_sw128(do_addr + off, 16, 1024),
                   umma_smem_desc_sw128(v_addr + off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait(pds_full, it & 1)) { report_error(p.status, OA_KERR_WAIT_SOFTMAX); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < FA_BM / 16; ++ks) {   // reduction over the 128 queries of this block
          umma_f16(tmem_base + Cfg::TM_DV, umma_smem_desc_sw128(p_addr + ks * 2048, FA_BM * 128, 1024),
                   umma_smem_desc_sw128(do_addr + ks * 2048, FA_BM * 128, 1024), idesc_g, (it > 0 || ks > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < FA_BM / 16; ++ks) {
          umma_f16(tmem_base + Cfg::TM_DK, umma_smem_desc_sw128(ds_addr + ks * 2048, FA_BM * 128, 1024),
                   umma_smem_desc_sw128(q_addr + ks * 2048, FA_BM * 128, 1024), idesc_g, (it > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&qdo_empty[st]);
      }
      if (ok) umma_commit(fin_full);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;            // this thread owns key columns [64*half, 64*half+64)
    const int r = quad * 32 + lane;
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    uint8_t* sP = smem + Cfg::OFF_P;
    uint8_t* sDS = smem + Cfg::OFF_DS;
    const long long stat_base = ((long long)b * p.heads + h) * p.seq;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int ib = i0 + it;
      const int qi = ib * FA_BM + r;
      const bool q_ok = qi < p.seq;
      const float lse2 = q_ok ? p.lse[stat_base + qi] * LOG2E : INFINITY;
      const float dlt = q_ok ? p.delta[stat_base + qi] : 0.f;
      ok = mbar_wait(s_full, it & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      const int k0 = jb * FA_BN;
      const bool need_mask = (p.causal && ib == jb) || (k0 + FA_BN > p.seq) || !q_ok;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t s[32], dp[32];
        tmem_ld32(tmem_base + t_lane + Cfg::TM_S + c * 32, s);
        tmem_ld32(tmem_base + t_lane + Cfg::TM_DP + c * 32, dp);
        tmem_ld_wait();
        uint32_t pw[16], dw[16];
        const float nlse = -lse2, ndlt = -dlt * p.scale;
        if (need_mask) {
          const int lim = q_ok ? (min(p.causal ? qi : 0x7fffffff, p.seq - 1) - (k0 + c * 32)) : -1;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = (i <= lim) ? fast_exp2(fmaf(__uint_as_float(s[i]), sl2, nlse)) : 0.f;
            float p1 = (i + 1 <= lim) ? fast_exp2(fmaf(__uint_as_float(s[i + 1]), sl2, nlse)) : 0.f;
            pw[i >> 1] = pack_bf16x2(p0, p1);
            dw[i >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(dp[i]), p.scale, ndlt), p1 * fmaf(__uint_as_float(dp[i + 1]), p.scale, ndlt));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), sl2, nlse));
            float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), sl2, nlse));
            pw[i >> 1] = pack_bf16x2(p0, p1);
            dw[i >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(dp[i]), p.scale, ndlt), p1 * fmaf(__uint_as_float(dp[i + 1]), p.scale, ndlt));
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t off = half * (FA_BM * 128) + r * 128 + ((((cc * 4 + g) ^ (r & 7))) << 4);
          *reinterpret_cast<uint4*>(sP + off) = make_uint4(pw[g * 4], pw[g * 4 + 1], pw[g * 4 + 2], pw[g * 4 + 3]);
          *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dw[g * 4], dw[g * 4 + 1], dw[g * 4 + 2], dw[g * 4 + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    if (ok) {
      ok = mbar_wait(fin_full, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL);
    }
    if (ok) {
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
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc<Cfg::TMEM_COLS>(tmem_base); }
}

template <int HD>
struct BwdQCfg {
  static constexpr int NST = (HD == 64) ? 2 : 1;
  static constexpr int T_BYTES = FA_BM * HD * 2;
  static constexpr int P_BYTES = FA_BM * FA_BN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = OFF_Q + T_BYTES;
  static constexpr int OFF_K = OFF_DO + T_BYTES;
  static constexpr int OFF_V = OFF_K + NST * T_BYTES;
  static constexpr int OFF_DS = OFF_V + NST * T_BYTES;
  static constexpr int OFF_BAR = OFF_DS + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128;
  static constexpr int TMEM_COLS = 512;
  static constexpr int TM_S = 0, TM_DP = 128, TM_DQ = 256;
};

// One CTA per (query block, head, batch): dQ accumulates in TMEM over the key blocks.
template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
flash_bwd_q_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const FlashBwdParams p) {
  using Cfg = BwdQCfg<HD>;
  constexpr int NST = Cfg::NST;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* ds_full = bars + 6;
  uint64_t* fin_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = (p.seq + FA_BM - 1) / FA_BM;
  const int ib = nblk - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int n_kv = p.causal ? (ib + 1) : nblk;
  const int row0 = b * p.seq;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_error(p.status, OA_KERR_BAD_ARG);
    return;
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(ds_full, 8);
    mbar_init(fin_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * Cfg::T_BYTES);
#pragma unroll
      for (int x = 0; x < HD / 64; ++x) {
        tma_load_2d(smem + Cfg::OFF_Q + x * (FA_BM * 128), &tmQ, q_full, h * HD + x * 64, row0 + ib * FA_BM);
        tma_load_2d(smem + Cfg::OFF_DO + x * (FA_BM * 128), &tmDO, q_full, h * HD + x * 64, row0 + ib * FA_BM);
      }
      for (int j = 0; j < n_kv; ++j) {
        int st = j % NST;
        uint32_t ph = (j / NST) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1)) { report_error(p.status, OA_KERR_WAIT_EMPTY); break; }
        mbar_expect_tx(&kv_full[st], 2 * Cfg::T_BYTES);
#pragma unroll
        for (int x = 0; x < HD / 64; ++x) {
          tma_load_2d(smem + Cfg::OFF_K + st * Cfg::T_BYTES + x * (FA_BN * 128), &tmK, &kv_full[st], h * HD + x * 64, row0 + j * FA_BN);
          tma_load_2d(smem + Cfg::OFF_V + st * Cfg::T_BYTES + x * (FA_BN * 128), &tmV, &kv_full[st], h * HD + x * 64, row0 + j * FA_BN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(FA_BM, FA_BN, 0, 0);
      constexpr uint32_t idesc_q = umma_idesc_bf16(FA_BM, HD, 0, 1);   // dQ[q x HD] += dS[q x keys] * K[keys x HD]
      const uint32_t q_addr = smem_u32(smem + Cfg::OFF_Q), do_addr = smem_u32(smem + Cfg::OFF_DO);
      const uint32_t ds_addr = smem_u32(smem + Cfg::OFF_DS);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) report_error(p.status, OA_KERR_WAIT_FULL);
      for (int j = 0; j < n_kv && ok; ++j) {
        int st = j % NST;
        if (!mbar_wait(&kv_full[st], (j / NST) & 1)) { report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + Cfg::OFF_K + st * Cfg::T_BYTES);
        const uint32_t v_addr = smem_u32(smem + Cfg::OFF_V + st * Cfg::T_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_S, umma_smem_desc_sw128(q_addr + off, 16, 1024),
                   umma_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          uint32_t off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_DP, umma_smem_desc_sw128(do_addr + off, 16, 1024),
                   umma_smem_desc_sw128(v_addr + off, 16, 1024), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait(ds_full, j & 1)) { report_error(p.status, OA_KERR_WAIT_SOFTMAX); ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          uint32_t a_off = (ks >> 2) * (FA_BM * 128) + (ks & 3) * 32;
          umma_f16(tmem_base + Cfg::TM_DQ, umma_smem_desc_sw128(ds_addr + a_off, 16, 1024),
                   umma_smem_desc_sw128(k_addr + ks * 2048, FA_BN * 128, 1024), idesc_q, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[st]);
      }
      if (ok) umma_commit(fin_full);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    uint8_t* sDS = smem + Cfg::OFF_DS;
    const long long stat_base = ((long long)b * p.heads + h) * p.seq;
    const int qi = ib * FA_BM + r;
    const bool q_ok = qi < p.seq;
    const float lse2 = q_ok ? p.lse[stat_base + qi] * LOG2E : INFINITY;
    const float dlt = q_ok ? p.delta[stat_base + qi] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      ok = mbar_wait(s_full, j & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      const int k0 = j * FA_BN;
      const bool need_mask = (p.causal && j == ib) || (k0 + FA_BN > p.seq) || !q_ok;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t s[32], dp[32];
        tmem_ld32(tmem_base + t_lane + Cfg::TM_S + c * 32, s);
        tmem_ld32(tmem_base + t_lane + Cfg::TM_DP + c * 32, dp);
        tmem_ld_wait();
        uint32_t dw[16];
        const float nlse = -lse2, ndlt = -dlt * p.scale;
        if (need_mask) {
          const int lim = q_ok ? (min(p.causal ? qi : 0x7fffffff, p.seq - 1) - (k0 + c * 32)) : -1;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = (i <= lim) ? fast_exp2(fmaf(__uint_as_float(s[i]), sl2, nlse)) : 0.f;
            float p1 = (i + 1 <= lim) ? fast_exp2(fmaf(__uint_as_float(s[i + 1]), sl2, nlse)) : 0.f;
            dw[i >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(dp[i]), p.scale, ndlt), p1 * fmaf(__uint_as_float(dp[i + 1]), p.scale, ndlt));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = fast_exp2(fmaf(__uint_as_float(s[i]), sl2, nlse));
            float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), sl2, nlse));
            dw[i >> 1] = pack_bf16x2(p0 * fmaf(__uint_as_float(dp[i]), p.scale, ndlt), p1 * fmaf(__uint_as_float(dp[i + 1]), p.scale, ndlt));
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4*>(sDS + half * (FA_BM * 128) + r * 128 + ((((cc * 4 + g) ^ (r & 7))) << 4)) =
              make_uint4(dw[g * 4], dw[g * 4 + 1], dw[g * 4 + 2], dw[g * 4 + 3]);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok) {
      ok = mbar_wait(fin_full, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL);
    }
    if (ok) {
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
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc<Cfg::TMEM_COLS>(tmem_base); }
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
  static const int version = [] { const char* e = getenv("OA_FLASH_FWD"); return (e && e[0] == '1') ? 1 : 2; }();
  if (version == 2) {
    const int nblk = (seq + FA_BM - 1) / FA_BM;
    dim3 grid2((nblk + 1) / 2, heads, batch);
    if (head_dim == 64) {
      static bool set = false;
      if (!set) { if (cudaFuncSetAttribute(flash_fwd2_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Cfg<64>::SMEM_BYTES) != cudaSuccess) return OA_ERR_LAUNCH; set = true; }
      flash_fwd2_kernel<64><<<grid2, FA_THREADS, Fwd2Cfg<64>::SMEM_BYTES, st>>>(tq, tk, tv, p);
    } else {
      static bool set = false;
      if (!set) { if (cudaFuncSetAttribute(flash_fwd2_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd2Cfg<128>::SMEM_BYTES) != cudaSuccess) return OA_ERR_LAUNCH; set = true; }
      flash_fwd2_kernel<128><<<grid2, FA_THREADS, Fwd2Cfg<128>::SMEM_BYTES, st>>>(tq, tk, tv, p);
    }
    return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
  }
  dim3 grid((seq + FA_BM - 1) / FA_BM, heads, batch);
  if (head_dim == 64) {
    static bool set = false;
    if (!set) { if (cudaFuncSetAttribute(flash_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<64>::SMEM_BYTES) != cudaSuccess) return OA_ERR_LAUNCH; set = true; }
    flash_fwd_kernel<64><<<grid, FA_THREADS, FwdCfg<64>::SMEM_BYTES, st>>>(tq, tk, tv, p);
  } else {
    static bool set = false;
    if (!set) { if (cudaFuncSetAttribute(flash_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<128>::SMEM_BYTES) != cudaSuccess) return OA_ERR_LAUNCH; set = true; }
    flash_fwd_kernel<128><<<grid, FA_THREADS, FwdCfg<128>::SMEM_BYTES, st>>>(tq, tk, tv, p);
  }
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
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
    flash_delta_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, scratch, batch, heads, seq,
                                               head_dim, o_row_stride, o_row_stride);
  }
  FlashBwdParams p;
  p.batch = batch; p.heads = heads; p.seq = seq; p.head_dim = head_dim; p.scale = scale; p.causal = causal;
  p.lse = lse; p.delta = scratch;
  p.dq = (__nv_bfloat16*)dq; p.dq_stride = dq_row_stride;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.dkv_stride = dkv_row_stride;
  p.status = status;
  dim3 grid((seq + FA_BM - 1) / FA_BM, heads, batch);
  if (head_dim == 64) {
    static bool set = false;
    if (!set) {
      if ((rc = set_max_smem(flash_bwd_kv_kernel<64>, BwdKvCfg<64>::SMEM_BYTES))) return rc;
      if ((rc = set_max_smem(flash_bwd_q_kernel<64>, BwdQCfg<64>::SMEM_BYTES))) return rc;
      set = true;
    }
    flash_bwd_kv_kernel<64><<<grid, FA_THREADS, BwdKvCfg<64>::SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
    flash_bwd_q_kernel<64><<<grid, FA_THREADS, BwdQCfg<64>::SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
  } else {
    static bool set = false;
    if (!set) {
      if ((rc = set_max_smem(flash_bwd_kv_kernel<128>, BwdKvCfg<128>::SMEM_BYTES))) return rc;
      if ((rc = set_max_smem(flash_bwd_q_kernel<128>, BwdQCfg<128>::SMEM_BYTES))) return rc;
      set = true;
    }
    flash_bwd_kv_kernel<128><<<grid, FA_THREADS, BwdKvCfg<128>::SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
    flash_bwd_q_kernel<128><<<grid, FA_THREADS, BwdQCfg<128>::SMEM_BYTES, st>>>(tq, tk, tv, tdo, p);
  }
  return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
}

