// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   D[M,N] = epilogue( alpha * sum_k A(m,k) * B(n,k) )
//
// Operands are bf16, accumulation is fp32 in TMEM.  Each operand may be stored
// "K-major" (the reduction index is the contiguous one: A is [M,K], B is [N,K],
// which is the reference's MatMulNt / Linear convention, Core/FnMatrix/Blas/FnMatrixBlas.gen.h:7)
// or "MN-major" (stored as [K,M] / [K,N]), which is what the data-gradient
// (dX = dY * W) and weight-gradient (dW = dY^T * X) products need, so no
// transposed copies are ever made.
//
// Structure: persistent kernel, one CTA per SM (or one CTA pair per two SMs), 320 threads.
//   warp 0 (one lane)  TMA producer: cp.async.bulk.tensor tiles into a 4/6 stage smem ring (128B swizzle)
//   warp 1 (one lane)  tcgen05.mma issuer: 128 x BN x 16 MMAs (256 x 256 x 16 for a pair) into one of two TMEM accumulators
//   warps 2..9         epilogue, two warps per scheduler (warps 2..5 only in the GEMM -> reduce-scatter mode): tcgen05.ld the
//                      finished accumulator, fuse bias / GELU / residual / GELU-backward / accumulate, store bf16 (through
//                      TMA stores in the pair kernel) or fp32
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
// Split-K (for weight gradients whose output has too few tiles to fill 148 SMs) writes fp32
// partials to a workspace that a small second kernel reduces in a fixed order (deterministic).
//
// Replaces the reference's GemmTiled / GemmCmSgBf16 / GemmCmWgBf16 family
// (Source/Private/Oa/Core/Shader/Compute/Blas/Gemm/*.slang) with one kernel family.
#include <cstdlib>
#include "common.cuh"
#include "api.h"
#include <mutex>
#include <unordered_map>
#include <string>
#include <cstring>
#include <cstdio>

namespace oa {

struct GemmParams {
  int M, N, K;
  void* out;
  int ldc;
  int out_f32;
  const __nv_bfloat16* bias;       // [N] or null
  const __nv_bfloat16* residual;   // [M, ldr] or null
  int ldr;
  __nv_bfloat16* aux_out;          // pre-activation copy [M, ldaux] or null
  const __nv_bfloat16* aux_in;     // pre-activation input for GELU backward [M, ldaux] or null
  int ldaux;
  int act;                         // OA_ACT_*
  int accumulate;                  // out += result
  float alpha;
  int splits;                      // split-K factor; >1 => write fp32 partials to workspace
  float* workspace;                // [splits, M, N] fp32
  int group_m;
  int pair_group_m;                // m tiles per raster group of the CTA-pair kernel
  int epi_prefetch;                // CTA-pair kernel: fetch aux_in / residual one chunk ahead
  int tma_store;                   // CTA-pair kernel: bf16 output (and aux_out) leave through TMA stores
  int* status;
  int batch;                       // independent problems of the same shape (tensor maps are rank 3)
  long long sc_batch, sr_batch, saux_batch, sbias_batch;   // element strides between problems
  // Grouped (mixture-of-experts) modes; `batch` is then the number of groups and offsets[batch+1] are row offsets,
  // every group padded to a multiple of 128 rows.
  //   1: the ROWS of A / out are grouped (Y[r,:] = X[r,:] * W[g(r)]^T): A and out are flat [rows, .], B is batched.
  //   2: the REDUCTION is grouped (dW[g] = dY_g^T * X_g): A and B are flat [rows, .] MN-major, out is batched.
  int group_mode;
  const int* group_offsets;
  // Tensor-parallel modes (the GEMM and its collective are one kernel; peers are reached with plain loads / stores).
  //   1  all-gather -> GEMM: A is the local staging copy [M, K] of the row-sharded activation.  The epilogue warps of every
  //      CTA first push slabs of this rank's shard (tp_src) into the peers' staging buffers and count them in on the
  //      receiver; the TMA producer waits for the counter of the 128-row block it is about to load.  M tiles are visited
  //      own shard first (read in place), then in the order the peers' blocks arrive.
  //   2  GEMM -> reduce-scatter: every output tile belongs to the rank that owns its rows; the epilogue stores the bf16
  //      partial into slot `rank` of the owner's staging buffer and bumps the owner's per-block counter; after its tiles a
  //      CTA reduces blocks of this rank's own rows over the `world` slots (+ residual) into `out` [M / world, N].
  int tp_mode, tp_world, tp_rank, tp_comm;
  const __nv_bfloat16* tp_src; int tp_ld_src;
  PeerTable tp_bufs;                  // mode 1: staging [M, K] of every rank; mode 2: staging [world, M / world, N] of every rank
  PeerTable tp_flags;                 // u64 per 128-row block (mode 1: [world * blocks]; mode 2: [blocks]) on every rank
  unsigned long long* tp_sync;        // [0] epoch of this call site, [1] CTAs finished (device resident: graph replay safe)
  // single-CTA kernel: rank-3 map {N, rows, problems} of a bf16 output that leaves through TMA stores (tma_store set)
  alignas(64) CUtensorMap tm_out;
};

constexpr int BM = 128;
constexpr int BK = 64;       // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int EPI_ROW_BYTES = 144;      // 64 bf16 columns + 16 B pad
  // staging behind the ring: 4 warps x 32 rows of the reduce-scatter mode, or 8 warps x two 2 KB TMA-store buffers
  static constexpr int EPI_BYTES = (4 * 32 * EPI_ROW_BYTES > 8 * 4096) ? 4 * 32 * EPI_ROW_BYTES : 8 * 4096;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ + 1280 /*group tile prefix*/ + EPI_BYTES;
};

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int group_m, int& mi, int& ni) {
  int per_group = group_m * n_tiles;
  int g = t / per_group;
  int first_m = g * group_m;
  int gsz = min(m_tiles - first_m, group_m);
  int r = t - g * per_group;
  mi = first_m + (r % gsz);
  ni = r / gsz;
}

struct TileInfo {
  int bi;        // batch / group index (selects the B problem, bias row, output problem)
  int row0;      // first output row of the tile (global row for grouped-rows mode)
  int ni;        // n tile index
  int kb0, kb1;  // k-block range
  int split;
  int a_batch, b_batch;  // z coordinates for the A / B tensor maps
};

__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int t, const int* s_prefix, int m_tiles, int n_tiles,
                                                int mn_tiles, int tiles_per_batch, int kb_total, int kb_per_split) {
  TileInfo ti;
  if (p.group_mode == 1) {
    int lo = 0, hi = p.batch;            // largest g with s_prefix[g] <= t
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= t) lo = mid; else hi = mid;
    }
    const int g = lo;
    const int off = p.group_offsets[g];
    const int mt = (p.group_offsets[g + 1] - off) >> 7;
    const int local = t - s_prefix[g];
    ti.bi = g; ti.row0 = off + (local % mt) * BM; ti.ni = local / mt;
    ti.kb0 = 0; ti.kb1 = kb_total; ti.split = 0; ti.a_batch = 0; ti.b_batch = g;
    return ti;
  }
  int bi = t / tiles_per_batch;
  int tb = t - bi * tiles_per_batch;
  int split = tb / mn_tiles;
  int mi, ni;
  tile_coords(tb - split * mn_tiles, m_tiles, n_tiles, p.group_m, mi, ni);
  if (p.tp_mode) {
    const int per_rank = m_tiles / p.tp_world;
    const int step = mi / per_rank;
    const int who = p.tp_mode == 1 ? (p.tp_rank - step + p.tp_world) % p.tp_world      // own shard, then rank-1, rank-2, ...
                                   : (p.tp_rank + 1 + step) % p.tp_world;              // owners rank+1, ..., own rows last
    mi = who * per_rank + (mi - step * per_rank);
  }
  ti.bi = bi; ti.row0 = mi * BM; ti.ni = ni; ti.split = split;
  if (p.group_mode == 2) {
    ti.kb0 = p.group_offsets[bi] >> 6; ti.kb1 = p.group_offsets[bi + 1] >> 6; ti.a_batch = 0; ti.b_batch = 0;
  } else {
    ti.kb0 = split * kb_per_split; ti.kb1 = min(kb_total, ti.kb0 + kb_per_split); ti.a_batch = bi; ti.b_batch = bi;
  }
  return ti;
}

// `pre` (may be null): the four 16-byte pieces of this row's saved pre-activation (aux_in) or, when there is no aux_in, of its
// residual, loaded by the caller ahead of time so that the load latency is not paid between tcgen05.ld and the store.
// Output through TMA stores (CTA-pair kernel, bf16 output without accumulation): a warp's [32 rows x 32 columns] piece is
// written to a 2 KB shared-memory buffer in the 64-byte swizzle of the tensor map (conflict-free 16-byte stores) and one lane
// issues the bulk store, which writes whole 64-byte row segments and clips what lies outside the matrix.  Per-lane 16-byte
// global stores of 32 different rows cost one L1 pass per row and kept the epilogue of a K = 1024 product longer than its
// main loop.  Two buffers per warp: a buffer is rewritten once the store issued two stores ago has read it.
struct TmaStoreCtx {
  const CUtensorMap* out;
  const CUtensorMap* aux;
  uint8_t* buf;          // this warp's 2 x 2 KB
  uint32_t n;            // stores issued by this warp
  int row0;              // first row of the warp's 32
  int z;                 // problem index for a rank-3 map, -1 for a rank-2 map
};
// `w`: the lane's 32 columns as 16 packed bf16 pairs
__device__ __forceinline__ void tma_store_packed(TmaStoreCtx* ts, const CUtensorMap* m, const uint32_t* w, int col0) {
  const int lane = threadIdx.x & 31;
  uint8_t* b = ts->buf + (ts->n & 1) * 2048;
  if (lane == 0) tma_store_wait_read1();
  __syncwarp();
  const uint32_t base = smem_u32(b) + lane * 64;
  const int sw = (lane >> 1) & 3;                       // 64-byte swizzle: 16-byte piece index ^= address bits 7..8
#pragma unroll
  for (int g = 0; g < 4; ++g) st_shared_v4(base + ((g ^ sw) << 4), make_uint4(w[g * 4], w[g * 4 + 1], w[g * 4 + 2], w[g * 4 + 3]));
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    if (ts->z < 0) tma_store_2d(m, b, col0, ts->row0);
    else tma_store_3d(m, b, col0, ts->row0, ts->z);
    tma_store_commit();
  }
  ++ts->n;
}
__device__ __forceinline__ void tma_store_piece(TmaStoreCtx* ts, const CUtensorMap* m, const float* v, int col0) {
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
  tma_store_packed(ts, m, w, col0);
}

template <int BN>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const uint32_t* r, int row, int col0, int split, int bi,
                                               const uint4* pre = nullptr, TmaStoreCtx* ts = nullptr) {
  if (col0 >= p.N) return;                              // uniform over the warp
  if (ts ? ts->row0 >= p.M : row >= p.M) return;        // with TMA stores the whole warp stays (rows past M are clipped)
  // N is a multiple of 8, so every 8-column group is either fully inside or fully outside.
  int ncols = row < p.M ? min(32, p.N - col0) : 0;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;

  if (p.splits > 1) {
    float* w = p.workspace + (((size_t)split * p.batch + bi) * p.M + row) * p.N + col0;
#pragma unroll
    for (int g = 0; g < 8; ++g)
      if (g * 4 < ncols) *reinterpret_cast<float4*>(w + g * 4) = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
    return;
  }
  if (p.bias) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g * 8 < ncols) {
        uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + bi * p.sbias_batch + col0 + g * 8));
        float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
        v[g * 8 + 0] += f0.x; v[g * 8 + 1] += f0.y; v[g * 8 + 2] += f1.x; v[g * 8 + 3] += f1.y;
        v[g * 8 + 4] += f2.x; v[g * 8 + 5] += f2.y; v[g * 8 + 6] += f3.x; v[g * 8 + 7] += f3.y;
      }
    }
  }
  if (p.aux_out && ts) {
    tma_store_piece(ts, ts->aux, v, col0);
  } else if (p.aux_out) {
    __nv_bfloat16* a = p.aux_out + bi * p.saux_batch + (size_t)row * p.ldaux + col0;
#pragma unroll
    for (int g = 0; g < 4; ++g)
      if (g * 8 < ncols)
        *reinterpret_cast<uint4*>(a + g * 8) =
            make_uint4(pack_bf16x2(v[g * 8], v[g * 8 + 1]), pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]),
                       pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]), pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]));
  }
  if (p.act == OA_ACT_GELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_fast(v[i]);
  } else if (p.act == OA_ACT_RELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
  } else if (p.act == OA_ACT_SILU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = silu_f(v[i]);
  }
  if (p.aux_in) {  // multiply by d(act)/dz of the saved pre-activation (backward of a fused Linear+act)
    const __nv_bfloat16* a = p.aux_in + bi * p.saux_batch + (size_t)row * p.ldaux + col0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g * 8 < ncols) {
        uint4 b = pre ? pre[g] : *reinterpret_cast<const uint4*>(a + g * 8);
        uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 z = unpack_bf16x2(w[j]);
          if (p.act == OA_ACT_GELU_BWD) {
            v[g * 8 + 2 * j] *= gelu_tanh_grad_fast(z.x);
            v[g * 8 + 2 * j + 1] *= gelu_tanh_grad_fast(z.y);
          } else {  // OA_ACT_RELU_BWD
            v[g * 8 + 2 * j] = z.x > 0.f ? v[g * 8 + 2 * j] : 0.f;
            v[g * 8 + 2 * j + 1] = z.y > 0.f ? v[g * 8 + 2 * j + 1] : 0.f;
          }
        }
      }
    }
  }
  if (p.residual) {
    const __nv_bfloat16* a = p.residual + bi * p.sr_batch + (size_t)row * p.ldr + col0;
    const uint4* rpre = p.aux_in ? nullptr : pre;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g * 8 < ncols) {
        uint4 b = rpre ? rpre[g] : *reinterpret_cast<const uint4*>(a + g * 8);
        float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
        v[g * 8 + 0] += f0.x; v[g * 8 + 1] += f0.y; v[g * 8 + 2] += f1.x; v[g * 8 + 3] += f1.y;
        v[g * 8 + 4] += f2.x; v[g * 8 + 5] += f2.y; v[g * 8 + 6] += f3.x; v[g * 8 + 7] += f3.y;
      }
    }
  }
  if (ts) {
    tma_store_piece(ts, ts->out, v, col0);
  } else if (p.out_f32) {
    float* o = reinterpret_cast<float*>(p.out) + bi * p.sc_batch + (size_t)row * p.ldc + col0;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (g * 4 < ncols) {
        float4 x = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
        if (p.accumulate) {
          float4 c = *reinterpret_cast<float4*>(o + g * 4);
          x.x += c.x; x.y += c.y; x.z += c.z; x.w += c.w;
        }
        *reinterpret_cast<float4*>(o + g * 4) = x;
      }
    }
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + bi * p.sc_batch + (size_t)row * p.ldc + col0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (g * 8 < ncols) {
        if (p.accumulate) {
          uint4 b = *reinterpret_cast<uint4*>(o + g * 8);
          float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y), f2 = unpack_bf16x2(b.z), f3 = unpack_bf16x2(b.w);
          v[g * 8 + 0] += f0.x; v[g * 8 + 1] += f0.y; v[g * 8 + 2] += f1.x; v[g * 8 + 3] += f1.y;
          v[g * 8 + 4] += f2.x; v[g * 8 + 5] += f2.y; v[g * 8 + 6] += f3.x; v[g * 8 + 7] += f3.y;
        }
        *reinterpret_cast<uint4*>(o + g * 8) =
            make_uint4(pack_bf16x2(v[g * 8], v[g * 8 + 1]), pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]),
                       pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]), pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]));
      }
    }
  }
}

// Tensor-parallel mode 1: the four epilogue warps of EVERY CTA push a share of this rank's shard into the peers' staging
// buffers before their first accumulator is ready (they would idle through the first main loop anyway), so the NVLink
// traffic is issued from all SMs at once.  An item is one [128 rows x 512 columns] slab for one peer; peers are served
// nearest first (rank+1, rank+2, ...), which is the order in which the receivers consume the blocks.  Each slab is
// published by a release-add on the receiver's per-block counter.
constexpr int TP_SLAB = 512;
__device__ __forceinline__ void tp_push_shard(const GemmParams& p, unsigned long long epoch) {
  const int W = p.tp_world, r = p.tp_rank;
  const int blocks = (p.M / W) / BM;
  const int n_slabs = (p.K + TP_SLAB - 1) / TP_SLAB;
  const int et = (int)threadIdx.x - 64;                  // 0..127 over warps 2..5
  const int per_peer = blocks * n_slabs;
  constexpr int UNROLL = 8;
  for (int item = blockIdx.x; item < per_peer * (W - 1); item += gridDim.x) {
    const int j = item / per_peer, rem = item - j * per_peer;
    const int c = rem / n_slabs, sl = rem - c * n_slabs;
    const int peer = (r + 1 + j) % W;
    const int col0 = sl * TP_SLAB;
    const int vec_per_row = min(TP_SLAB, p.K - col0) >> 3;
    const int total_vec = BM * vec_per_row;
    const __nv_bfloat16* src = p.tp_src + (size_t)c * BM * p.tp_ld_src + col0;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.tp_bufs.ptr[peer]) + ((size_t)r * blocks + c) * BM * p.K + col0;
    for (int v0 = et; v0 < total_vec; v0 += 128 * UNROLL) {
      uint4 buf[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int v = v0 + u * 128;
        if (v < total_vec) {
          const int row = v / vec_per_row, cv = v - row * vec_per_row;
          buf[u] = *reinterpret_cast<const uint4*>(src + (size_t)row * p.tp_ld_src + cv * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int v = v0 + u * 128;
        if (v < total_vec) {
          const int row = v / vec_per_row, cv = v - row * vec_per_row;
          *reinterpret_cast<uint4*>(dst + (size_t)row * p.K + cv * 8) = buf[u];   // weak store; the fence below publishes it
        }
      }
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");        // the four epilogue warps only
    if (et == 0)
      red_release_sys_add(reinterpret_cast<unsigned long long*>(p.tp_flags.ptr[peer]) + (size_t)r * blocks + c, 1ull);
  }
}

// One [128 rows x 128 columns] unit of the row reduction: UN positions per thread are loaded (all `world` slots of each)
// before the first add, so that enough bytes are in flight to cover the L2 / HBM latency.
template <int UN>
__device__ __forceinline__ void tp_reduce_unit(const GemmParams& p, const __nv_bfloat16* stage, int rb, int sl, int Ms, int W) {
  for (int e0 = threadIdx.x; e0 < BM * 16; e0 += 192 * UN) {
    uint4 part[UN][MAX_RANKS];
    uint4 resid[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int e = e0 + u * 192;
      const int row = rb * BM + (e >> 4), col = sl * 128 + (e & 15) * 8;
      const bool live = e < BM * 16 && col < p.N;
#pragma unroll
      for (int src = 0; src < MAX_RANKS; ++src)
        if (src < W && live) part[u][src] = ld_peer_v4(stage + ((size_t)src * Ms + row) * p.N + col);
      if (p.residual && live) resid[u] = *reinterpret_cast<const uint4*>(p.residual + (size_t)row * p.ldr + col);
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int e = e0 + u * 192;
      const int row = rb * BM + (e >> 4), col = sl * 128 + (e & 15) * 8;
      if (e >= BM * 16 || col >= p.N) continue;
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
      for (int src = 0; src < MAX_RANKS; ++src) {
        if (src >= W) continue;
        const uint4 v = part[u][src];
        const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
        acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y; acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
      }
      if (p.residual) {
        const uint4 v = resid[u];
        const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
        acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y; acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
      }
      if (p.out_f32) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)row * p.ldc + col;
        *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      } else {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.ldc + col;
        *reinterpret_cast<uint4*>(o) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                                                  pack_bf16x2(acc[6], acc[7]));
      }
    }
  }
}

// Tensor-parallel mode 2, after the tiles: sum the `world` partial slots of this rank's own rows (+ residual) into `out`.
__device__ __forceinline__ void tp_reduce_rows(const GemmParams& p, int n_tiles, unsigned long long epoch, int* s_ok) {
  const int W = p.tp_world;
  const int Ms = p.M / W, blocks = Ms / BM;
  const int slabs = (p.N + 127) >> 7;
  const unsigned long long expect = epoch * (unsigned long long)(W * n_tiles * 4);
  const unsigned long long* cnt = reinterpret_cast<const unsigned long long*>(p.tp_flags.ptr[p.tp_rank]);
  const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(p.tp_bufs.ptr[p.tp_rank]);
  for (int u = blockIdx.x; u < blocks * slabs; u += gridDim.x) {
    const int rb = u / slabs, sl = u - rb * slabs;
    if (threadIdx.x == 0) {
      const bool ok = wait_ge_sys(cnt + rb, expect);
      if (!ok) report_error(p.status, OA_KERR_WAIT_PEER);
      *s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    const bool ok = *s_ok != 0;
    __syncthreads();
    if (!ok) break;
    if (W <= 2) tp_reduce_unit<4>(p, stage, rb, sl, Ms, W);
    else if (W <= 4) tp_reduce_unit<2>(p, stage, rb, sl, Ms, W);
    else tp_reduce_unit<1>(p, stage, rb, sl, Ms, W);
  }
}

template <int BN, int A_MN, int B_MN>
__global__ void __launch_bounds__(320, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * Cfg::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  if (p.group_mode == 1) pdl_wait();     // the prologue below reads the group offsets, which the previous kernel may have written
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // 4 epilogue warps (the GEMM -> reduce-scatter mode, whose staging and counters are laid out for four) or 8: two warps per
  // scheduler, the two of a TMEM lane quarter taking half of the accumulator's columns each
  const int epi_warps = (int)(blockDim.x >> 5) - 2;

  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int mn_tiles = m_tiles * n_tiles;
  const int tiles_per_batch = mn_tiles * p.splits;
  int* s_prefix = reinterpret_cast<int*>(smem + STAGES * Cfg::STAGE_BYTES + 256);
  uint8_t* s_epi = smem + STAGES * Cfg::STAGE_BYTES + 256 + 1280;     // staging: reduce-scatter tiles (4 warps) or TMA-store buffers (8 warps x 2 x 2 KB)
  // reduce-scatter mode only, behind its 18 KB of staging (the TMA-store buffers that share this region are off in that mode);
  // kept out of static shared memory: ring + staging already fill the 227 KB of a CTA to within 512 bytes
  unsigned long long* (*s_pend)[16] = reinterpret_cast<unsigned long long* (*)[16]>(s_epi + 4 * 32 * Cfg::EPI_ROW_BYTES);   // [4][16]: counters of stored tiles not yet published, per epilogue warp
  int& s_tp_ok = *reinterpret_cast<int*>(s_epi + 4 * 32 * Cfg::EPI_ROW_BYTES + 512);
  if (p.group_mode == 1 && threadIdx.x == 32) {
    int run = 0;
    for (int g = 0; g < p.batch; ++g) {
      s_prefix[g] = run;
      run += ((p.group_offsets[g + 1] - p.group_offsets[g]) >> 7) * n_tiles;
    }
    s_prefix[p.batch] = run;
  }
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_per_split = (kb_total + p.splits - 1) / p.splits;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.tp_mode == 1) tma_prefetch_desc(&tmA2);
    if (p.tma_store) tma_prefetch_desc(&p.tm_out);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], epi_warps);  // one arrive per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc<Cfg::TMEM_COLS>(tmem_slot);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = p.group_mode == 1 ? s_prefix[p.batch] : tiles_per_batch * p.batch;
  pdl_wait();                            // global memory (operands, flags, outputs) only from here on
  const int n_compute = (int)gridDim.x;
  unsigned long long tp_epoch = 0;
  if (p.tp_mode) tp_epoch = *reinterpret_cast<volatile unsigned long long*>(p.tp_sync) + 1;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += n_compute) {
        const TileInfo ti = decode_tile(p, t, s_prefix, m_tiles, n_tiles, mn_tiles, tiles_per_batch, kb_total, kb_per_split);
        const CUtensorMap* mapA = &tmA;
        int a_row0 = ti.row0;
        if (p.tp_mode == 1) {
          const int Ms = p.M / p.tp_world;
          if (ti.row0 / Ms == p.tp_rank) {
            mapA = &tmA2;                   // this rank's own rows are read in place (tmA2 covers the local shard)
            a_row0 = ti.row0 - p.tp_rank * Ms;
          } else {
            // the rows of this tile are pushed into the local staging buffer by a communication CTA of their owner
            const unsigned long long* flags = reinterpret_cast<const unsigned long long*>(p.tp_flags.ptr[p.tp_rank]);
            const unsigned long long n_slabs = (unsigned long long)((p.K + TP_SLAB - 1) / TP_SLAB);
            if (!wait_ge_sys(flags + ti.row0 / BM, tp_epoch * n_slabs)) {
              report_error(p.status, OA_KERR_WAIT_PEER);
              ok = false;
              break;
            }
            fence_proxy_async_global();   // generic-proxy writes (peer stores) before the async-proxy (TMA) reads below
          }
        }
        for (int kb = ti.kb0; kb < ti.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            report_error(p.status, OA_KERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          uint8_t* a = sA + stage * Cfg::A_BYTES;
          uint8_t* b = sB + stage * Cfg::B_BYTES;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d(a + j * (64 * BK * 2), mapA, &full[stage], a_row0 + j * 64, kb * BK, ti.a_batch);
          } else {
            tma_load_3d(a, mapA, &full[stage], kb * BK, a_row0, ti.a_batch);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(b + j * (64 * BK * 2), &tmB, &full[stage], ti.ni * BN + j * 64, kb * BK, ti.b_batch);
          } else {
            tma_load_3d(b, &tmB, &full[stage], kb * BK, ti.ni * BN, ti.b_batch);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      // K-major: 8-row groups are 1024 B apart; one UMMA_K step is 32 B inside the swizzled row.
      // MN-major: 64-element column groups are one [64 x BK] box (BK*128 B) apart, 8-k groups 1024 B apart;
      //           one UMMA_K step is 16 k-rows of 128 B.
      constexpr uint32_t a_lbo = A_MN ? BK * 128 : 16, a_sbo = 1024, a_kstep = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      constexpr uint32_t b_lbo = B_MN ? BK * 128 : 16, b_sbo = 1024, b_kstep = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // descriptors of stage 0, computed once: a later stage or k-step only adds to the 14-bit address field (no carry,
      // shared memory ends below 256 KB), which keeps the single issuing thread's instruction stream short
      const uint64_t da0 = umma_smem_desc_sw128(smem_u32(sA), a_lbo, a_sbo);
      const uint64_t db0 = umma_smem_desc_sw128(smem_u32(sB), b_lbo, b_sbo);
      for (int t = blockIdx.x; t < total_tiles && ok; t += n_compute) {
        const TileInfo ti = decode_tile(p, t, s_prefix, m_tiles, n_tiles, mn_tiles, tiles_per_batch, kb_total, kb_per_split);
        const int kb0 = ti.kb0, kb1 = ti.kb1;
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1)) {
          report_error(p.status, OA_KERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase)) {
            report_error(p.status, OA_KERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = da0 + (uint64_t)((stage * Cfg::A_BYTES) >> 4);
          const uint64_t db = db0 + (uint64_t)((stage * Cfg::B_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16(d_tmem, da + (uint64_t)((k * a_kstep) >> 4), db + (uint64_t)((k * b_kstep) >> 4), idesc, k > 0 ? 1u : accumulate);
          accumulate = 1;
          umma_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue warps (2..5); TMEM lane quadrant = warp % 4
    const int quad = warp & 3;
    const int c_per = (BN / 32) / (epi_warps >> 2);
    const int c_begin = ((warp - 2) >> 2) * c_per, c_end = c_begin + c_per;
    int acc = 0;
    uint32_t acc_phase = 0;
    int n_pend = 0;
    TmaStoreCtx tsc{&p.tm_out, nullptr, s_epi + (warp - 2) * 4096, 0u, 0, 0};
    TmaStoreCtx* ts = p.tma_store ? &tsc : nullptr;
    if (p.tp_mode == 1 && warp < 6) tp_push_shard(p, tp_epoch);   // warps 2..5: its work split and its named barrier count 128 threads
    for (int t = blockIdx.x; t < total_tiles; t += n_compute) {
      const TileInfo ti = decode_tile(p, t, s_prefix, m_tiles, n_tiles, mn_tiles, tiles_per_batch, kb_total, kb_per_split);
      const int bi = ti.bi, ni = ti.ni, split = ti.split, kb0 = ti.kb0, kb1 = ti.kb1;
      bool ok = mbar_wait(&tfull[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after();
      const int row = ti.row0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      const bool empty_split = (kb1 <= kb0);  // nothing accumulated: treat as zeros
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_ld_wait();
        if (c == c_end - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
        }
        if (empty_split) {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0;
        }
        if (p.tp_mode == 2) {
          // bf16 partial -> per-warp shared tile (64 columns wide) -> 128-byte row segments stored into the owner's slot
          uint8_t* se = s_epi + quad * (32 * Cfg::EPI_ROW_BYTES);
          uint8_t* my = se + lane * Cfg::EPI_ROW_BYTES + (c & 1) * 64;
#pragma unroll
          for (int g = 0; g < 4; ++g)
            *reinterpret_cast<uint4*>(my + g * 16) = make_uint4(
                pack_bf16x2(__uint_as_float(r[g * 8]) * p.alpha, __uint_as_float(r[g * 8 + 1]) * p.alpha),
                pack_bf16x2(__uint_as_float(r[g * 8 + 2]) * p.alpha, __uint_as_float(r[g * 8 + 3]) * p.alpha),
                pack_bf16x2(__uint_as_float(r[g * 8 + 4]) * p.alpha, __uint_as_float(r[g * 8 + 5]) * p.alpha),
                pack_bf16x2(__uint_as_float(r[g * 8 + 6]) * p.alpha, __uint_as_float(r[g * 8 + 7]) * p.alpha));
          if (c & 1) {
            __syncwarp();
            const int Ms = p.M / p.tp_world;
            const int owner = ti.row0 / Ms;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.tp_bufs.ptr[owner]) +
                                 ((size_t)p.tp_rank * Ms + (ti.row0 - owner * Ms) + quad * 32) * p.N;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int idx = it * 32 + lane, rr = idx >> 3, piece = idx & 7;
              const int col = ni * BN + (c - 1) * 32 + piece * 8;
              if (col < p.N)   // weak store; published by the fence + release below
                *reinterpret_cast<uint4*>(dst + (size_t)rr * p.N + col) = *reinterpret_cast<const uint4*>(se + rr * Cfg::EPI_ROW_BYTES + piece * 16);
            }
            __syncwarp();
          }
          if (c == BN / 32 - 1) {
            // publishing a tile costs a system-scope fence (a round trip over NVLink): tiles are counted in batches
            const int Ms = p.M / p.tp_world;
            const int owner = ti.row0 / Ms;
            if (lane == 0) s_pend[quad][n_pend] = reinterpret_cast<unsigned long long*>(p.tp_flags.ptr[owner]) + (ti.row0 - owner * Ms) / BM;
            if (++n_pend == 16) {
              __threadfence_system();
              __syncwarp();
              if (lane < n_pend) red_release_sys_add(s_pend[quad][lane], 1ull);
              __syncwarp();
              n_pend = 0;
            }
          }
        } else {
          tsc.row0 = ti.row0 + quad * 32;
          tsc.z = p.group_mode == 1 ? 0 : bi;      // rows-grouped output is one flat matrix; batched / reduction-grouped: one per problem
          epilogue_chunk<BN>(p, r, row, ni * BN + c * 32, split, bi, nullptr, ts);
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (ts && lane == 0) tma_store_wait_read0();       // the staging buffers stay valid until the last store has read them
    if (n_pend > 0) {
      __threadfence_system();
      __syncwarp();
      if (lane < n_pend) red_release_sys_add(s_pend[quad][lane], 1ull);
    }
  }
  if (p.tp_mode == 2) {
    __syncthreads();
    tp_reduce_rows(p, n_tiles, tp_epoch, &s_tp_ok);
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<Cfg::TMEM_COLS>(tmem_base);
  }
  if (p.tp_mode && threadIdx.x == 0) {
    // the call site's epoch advances once every CTA (each read it at its start) has finished
    __threadfence();
    const unsigned long long old = atomicAdd(p.tp_sync + 1, 1ull);
    if (old == gridDim.x - 1) {
      p.tp_sync[1] = 0;
      __threadfence();
      p.tp_sync[0] = tp_epoch;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): a cluster of two CTAs computes one 256 x 256 tile.  Each CTA loads its own 128 rows of
// A and its own 128 of the 256 B rows (32 KB per stage instead of 48 KB, so the ring is 6 deep and the L2 -> SM traffic
// per FLOP drops by a third); the even CTA issues tcgen05.mma.cta_group::2 (M = 256) for the pair; each CTA's TMEM holds
// its 128 accumulator rows and its own epilogue warps drain them.  Loads carry no multicast: the pair shares B because
// the MMA reads both halves, not because a copy is broadcast.  Used for plain 2-D problems with enough 256 x 256 tiles.
struct PairCfg {
  static constexpr int STAGES = 6;
  static constexpr int A_BYTES = BM * BK * 2;            // this CTA's 128 rows of A
  static constexpr int B_BYTES = 128 * BK * 2;           // this CTA's 128 of the tile's 256 rows of B
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 512;                  // two 256-column accumulators
  static constexpr int STORE_BYTES = 8 * 2 * 2048;       // TMA-store staging: two 2 KB buffers per epilogue warp
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STORE_BYTES + 1024 + 256;
  // Warps 0 and 1 load and issue; 4 or 8 epilogue warps follow.  A warp reads the TMEM lanes of its index modulo 4, so with
  // eight warps two of them share a lane quarter and take half of the accumulator's columns each: one warp per scheduler
  // leaves every dependency stall of the epilogue arithmetic exposed, two hide most of them.
  static constexpr int MAX_THREADS = 64 + 8 * 32;
};

#ifdef OA_GEMM_PROBE
// Diagnostic build only (-DOA_GEMM_PROBE): per CTA pair, clocks that the MMA issuer spent in total / waiting for loads /
// waiting for a drained accumulator, and clocks that the even CTA's producer spent waiting for a free stage.
__device__ long long g_pair_probe[128 * 4];
#endif

// LEAN: the instantiation for a plain bf16 product (scale, round, TMA store). Its epilogue is a few dozen instructions
// instead of the generic one's thousands, which the epilogue warps would otherwise keep fetching through the instruction
// caches that the MMA-issuing and the loading warp share with them.
template <int A_MN, int B_MN, int LEAN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg::MAX_THREADS, 1)
gemm_pair_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmC,
                      const __grid_constant__ CUtensorMap tmAux, const GemmParams p) {
  using Cfg = PairCfg;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * Cfg::A_BYTES;
  uint8_t* sC = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sC + Cfg::STORE_BYTES);
  uint64_t* full = bars;                 // used in the even CTA: bytes of both CTAs' loads
  uint64_t* empty = bars + STAGES;       // per CTA: the pair's MMA has consumed this CTA's stage
  uint64_t* tfull = bars + 2 * STAGES;   // per CTA: accumulator ready
  uint64_t* tempty = bars + 2 * STAGES + 2;   // even CTA: the epilogue warps of both CTAs have drained the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int epi_warps = (int)(blockDim.x >> 5) - 2;      // 4 or 8
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int m_tiles = (p.M + 255) / 256, n_tiles = (p.N + 255) / 256;
  const int mn_tiles = m_tiles * n_tiles;
  const int total_tiles = mn_tiles * p.splits;           // split-K: unit = (split, tile), partials go to the fp32 workspace
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb_per_split = (kb_total + p.splits - 1) / p.splits;
  // Tail wave: when the tiles left after the last full wave occupy at most half of the pairs, each of them is split into
  // two 256 x 128 units (an MMA of N = 128, 64 B rows per CTA), so the tail costs half a wave instead of a whole one.
  const int full_tiles = (total_tiles / n_pairs) * n_pairs;
  const int rem_tiles = total_tiles - full_tiles;
  const bool split_tail = p.splits == 1 && rem_tiles > 0 && 2 * rem_tiles <= n_pairs;
  const int total_units = split_tail ? full_tiles + 2 * rem_tiles : total_tiles;
  auto unit_tile = [&](int u, int& half) -> int {
    if (!split_tail || u < full_tiles) { half = -1; return u; }
    half = (u - full_tiles) & 1;
    return full_tiles + ((u - full_tiles) >> 1);
  };

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmB2);
    if (p.tma_store) { tma_prefetch_desc(&tmC); tma_prefetch_desc(&tmAux); }
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 2 * epi_warps); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc_pair<Cfg::TMEM_COLS>(tmem_slot); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                    // both CTAs' barriers exist before anything arrives on them from the other side
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                            // everything above ran under the previous kernel's tail; global memory from here on

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer (both CTAs; the bytes are credited to the even CTA's barrier)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
#ifdef OA_GEMM_PROBE
      long long w_empty = 0;
#endif
      for (int u = pair; u < total_units && ok; u += n_pairs) {
        int mi, ni, half;
        const int t = unit_tile(u, half);
        const int split = p.splits > 1 ? t / mn_tiles : 0;
        tile_coords(t - split * mn_tiles, m_tiles, n_tiles, p.pair_group_m, mi, ni);
        const int row0 = mi * 256 + (int)rank * 128;
        const int n0 = half < 0 ? ni * 256 + (int)rank * 128 : ni * 256 + half * 128 + (int)rank * 64;
        const uint32_t stage_bytes = half < 0 ? 2 * Cfg::STAGE_BYTES : 2 * (Cfg::A_BYTES + Cfg::B_BYTES / 2);
        const int kb0 = split * kb_per_split, kb1 = min(kb_total, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
#ifdef OA_GEMM_PROBE
          const long long c0 = clock64();
#endif
          if (!mbar_wait(&empty[stage], phase ^ 1)) { report_error(p.status, OA_KERR_WAIT_EMPTY); ok = false; break; }
#ifdef OA_GEMM_PROBE
          w_empty += clock64() - c0;
#endif
          if (leader) mbar_expect_tx(&full[stage], stage_bytes);
          uint8_t* a = sA + stage * Cfg::A_BYTES;
          uint8_t* b = sB + stage * Cfg::B_BYTES;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_3d_pair(a + j * (64 * BK * 2), &tmA, &full[stage], row0 + j * 64, kb * BK, 0);
          } else {
            tma_load_3d_pair(a, &tmA, &full[stage], kb * BK, row0, 0);
          }
          if (B_MN) {
            tma_load_3d_pair(b, &tmB, &full[stage], n0, kb * BK, 0);
            if (half < 0) tma_load_3d_pair(b + 64 * BK * 2, &tmB, &full[stage], n0 + 64, kb * BK, 0);
          } else if (half < 0) {
            tma_load_3d_pair(b, &tmB, &full[stage], kb * BK, n0, 0);
          } else {
            tma_load_3d_pair(b, &tmB2, &full[stage], kb * BK, n0, 0);      // 64 rows of B
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
#ifdef OA_GEMM_PROBE
      if (leader && pair < 128) g_pair_probe[pair * 4 + 3] = w_empty;
#endif
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer of the pair
      constexpr uint32_t idesc_full = umma_idesc_bf16(256, 256, A_MN, B_MN);
      constexpr uint32_t idesc_half = umma_idesc_bf16(256, 128, A_MN, B_MN);
      constexpr uint32_t a_lbo = A_MN ? BK * 128 : 16, a_kstep = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      constexpr uint32_t b_lbo = B_MN ? BK * 128 : 16, b_kstep = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      // The issuing thread is a single dependent instruction stream, so everything that does not change per k-block is
      // computed once: the descriptors of stage 0 (a later stage or k-step only adds to the 14-bit address field, which
      // cannot carry because shared memory ends below 256 KB) and the distance to the odd CTA's copy of a barrier.
      const uint64_t da0 = umma_smem_desc_sw128(smem_u32(sA), a_lbo, 1024);
      const uint64_t db0 = umma_smem_desc_sw128(smem_u32(sB), b_lbo, 1024);
      const uint32_t empty0 = smem_u32(&empty[0]), tfull0 = smem_u32(&tfull[0]);
      const uint32_t peer_delta = map_to_cta(empty0, 1) - empty0;
#ifdef OA_GEMM_PROBE
      long long w_full = 0, w_acc = 0;
      const long long t_begin = clock64();
#endif
      for (int u = pair; u < total_units && ok; u += n_pairs) {
        int half;
        const int t = unit_tile(u, half);
        const int split = p.splits > 1 ? t / mn_tiles : 0;
        const int kb0 = split * kb_per_split, kb1 = min(kb_total, kb0 + kb_per_split);
        const uint32_t idesc = half < 0 ? idesc_full : idesc_half;
#ifdef OA_GEMM_PROBE
        const long long c0 = clock64();
#endif
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1)) { report_error(p.status, OA_KERR_WAIT_TMEM_EMPTY); break; }
#ifdef OA_GEMM_PROBE
        w_acc += clock64() - c0;
#endif
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 256;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
#ifdef OA_GEMM_PROBE
          const long long c1 = clock64();
#endif
          if (!mbar_wait(&full[stage], phase)) { report_error(p.status, OA_KERR_WAIT_FULL); ok = false; break; }
#ifdef OA_GEMM_PROBE
          w_full += clock64() - c1;
#endif
          tc_fence_after();
          const uint64_t da = da0 + (uint64_t)((stage * Cfg::A_BYTES) >> 4);
          const uint64_t db = db0 + (uint64_t)((stage * Cfg::B_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            umma_f16_pair(d_tmem, da + (uint64_t)((k * a_kstep) >> 4), db + (uint64_t)((k * b_kstep) >> 4), idesc, k > 0 ? 1u : accumulate);
          }
          accumulate = 1;
          const uint32_t e = empty0 + stage * 8;
          umma_commit_pair(e);                         // this CTA's stage is free ...
          umma_commit_pair(e + peer_delta);            // ... and so is the odd CTA's
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        const uint32_t f = tfull0 + acc * 8;
        umma_commit_pair(f);
        umma_commit_pair(f + peer_delta);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
#ifdef OA_GEMM_PROBE
      if (pair < 128) {
        g_pair_probe[pair * 4 + 0] = clock64() - t_begin;
        g_pair_probe[pair * 4 + 1] = w_full;
        g_pair_probe[pair * 4 + 2] = w_acc;
      }
#endif
    }
  } else {
    // ---------------- epilogue warps of both CTAs: each drains its own 128 accumulator rows
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2, parts = epi_warps >> 2;      // which share of the unit's columns this warp drains
    int acc = 0;
    uint32_t acc_phase = 0;
    TmaStoreCtx tsc{&tmC, &tmAux, sC + (warp - 2) * 4096, 0u, 0, -1};
    TmaStoreCtx* ts = p.tma_store ? &tsc : nullptr;
    for (int u = pair; u < total_units; u += n_pairs) {
      int mi, ni, half;
      const int t = unit_tile(u, half);
      const int split = p.splits > 1 ? t / mn_tiles : 0;
      tile_coords(t - split * mn_tiles, m_tiles, n_tiles, p.pair_group_m, mi, ni);
      tsc.row0 = mi * 256 + (int)rank * 128 + quad * 32;
      bool ok = mbar_wait(&tfull[acc], acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_error(p.status, OA_KERR_WAIT_TMEM_FULL); break; }
      tc_fence_after();
      const int row = mi * 256 + (int)rank * 128 + quad * 32 + lane;
      const int chunks = (half < 0 ? 8 : 4) / parts;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * 256 + part * chunks * 32;
      const int col_base = ni * 256 + (half < 0 ? 0 : half * 128) + part * chunks * 32;
      if constexpr (LEAN == 5 || LEAN == 6) {
        // 5: split-K partial, the scaled fp32 accumulator goes to this split's slice of the workspace
        // 6: fp32 output, optionally added to what is there (weight gradients accumulated in place)
        float* wrow = LEAN == 5 ? p.workspace + ((size_t)split * p.M + row) * p.N : reinterpret_cast<float*>(p.out) + (size_t)row * p.ldc;
        const bool add = LEAN == 6 && p.accumulate;
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          if (c == chunks - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&tempty[acc]) & kPeerBitMask);
          }
          const int col0 = col_base + c * 32;
          if (row < p.M) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (col0 + g * 4 < p.N) {
                float4 x = make_float4(__uint_as_float(r[g * 4]) * p.alpha, __uint_as_float(r[g * 4 + 1]) * p.alpha,
                                       __uint_as_float(r[g * 4 + 2]) * p.alpha, __uint_as_float(r[g * 4 + 3]) * p.alpha);
                if (add) {
                  const float4 o = *reinterpret_cast<const float4*>(wrow + col0 + g * 4);
                  x.x += o.x; x.y += o.y; x.z += o.z; x.w += o.w;
                }
                *reinterpret_cast<float4*>(wrow + col0 + g * 4) = x;
              }
            }
          }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        continue;
      } else if constexpr (LEAN != 0) {
        // LEAN 1: scale, round, store.  2: + residual.  3: GELU with the pre-activation copy (two stores).  4: multiply by
        // gelu'(saved pre-activation).  The row of the residual / saved pre-activation is fetched one chunk ahead.
        const bool live = tsc.row0 < p.M;
        const __nv_bfloat16* pre_base = LEAN == 2 ? p.residual + (size_t)row * p.ldr : (LEAN == 4 ? p.aux_in + (size_t)row * p.ldaux : nullptr);
        uint4 nxt[4];
        auto prefetch = [&](int c) {
          const int col = col_base + c * 32;
#pragma unroll
          for (int g = 0; g < 4; ++g)
            nxt[g] = (row < p.M && col + g * 8 < p.N) ? __ldg(reinterpret_cast<const uint4*>(pre_base + col + g * 8)) : make_uint4(0, 0, 0, 0);
        };
        if constexpr (LEAN == 2 || LEAN == 4) prefetch(0);
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          uint32_t r[32];
          uint4 cur[4];
          if constexpr (LEAN == 2 || LEAN == 4) { cur[0] = nxt[0]; cur[1] = nxt[1]; cur[2] = nxt[2]; cur[3] = nxt[3]; }
          tmem_ld32(taddr + c * 32, r);
          if constexpr (LEAN == 2 || LEAN == 4) { if (c + 1 < chunks) prefetch(c + 1); }
          tmem_ld_wait();
          if (c == chunks - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&tempty[acc]) & kPeerBitMask);
          }
          const int col0 = col_base + c * 32;
          if (live && col0 < p.N) {
            uint32_t w[16];
            if constexpr (LEAN == 1) {
#pragma unroll
              for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * p.alpha, __uint_as_float(r[2 * i + 1]) * p.alpha);
            } else if constexpr (LEAN == 2) {
              const uint32_t* cw = reinterpret_cast<const uint32_t*>(cur);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float2 q = unpack_bf16x2(cw[i]);
                w[i] = pack_bf16x2(fmaf(__uint_as_float(r[2 * i]), p.alpha, q.x), fmaf(__uint_as_float(r[2 * i + 1]), p.alpha, q.y));
              }
            } else if constexpr (LEAN == 3) {
#pragma unroll
              for (int i = 0; i < 16; ++i) w[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * p.alpha, __uint_as_float(r[2 * i + 1]) * p.alpha);
              tma_store_packed(&tsc, &tmAux, w, col0);
#pragma unroll
              for (int i = 0; i < 16; ++i)
                w[i] = pack_bf16x2(gelu_tanh_fast(__uint_as_float(r[2 * i]) * p.alpha), gelu_tanh_fast(__uint_as_float(r[2 * i + 1]) * p.alpha));
            } else {
              const uint32_t* cw = reinterpret_cast<const uint32_t*>(cur);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float2 z = unpack_bf16x2(cw[i]);
                w[i] = pack_bf16x2(__uint_as_float(r[2 * i]) * p.alpha * gelu_tanh_grad_fast(z.x),
                                   __uint_as_float(r[2 * i + 1]) * p.alpha * gelu_tanh_grad_fast(z.y));
              }
            }
            tma_store_packed(&tsc, &tmC, w, col0);
          }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        continue;
      }
      // the saved pre-activation (or the residual) of chunk c + 1 is fetched while chunk c is worked on
      const __nv_bfloat16* pre_base = (p.splits > 1 || !p.epi_prefetch) ? nullptr : (p.aux_in ? p.aux_in + (size_t)row * p.ldaux : (p.residual ? p.residual + (size_t)row * p.ldr : nullptr));
      uint4 nxt[4];
      auto prefetch = [&](int c) {
        const int col = col_base + c * 32;
#pragma unroll
        for (int g = 0; g < 4; ++g)
          nxt[g] = (pre_base && row < p.M && col + g * 8 < p.N) ? __ldg(reinterpret_cast<const uint4*>(pre_base + col + g * 8)) : make_uint4(0, 0, 0, 0);
      };
      prefetch(0);
#pragma unroll 1
      for (int c = 0; c < chunks; ++c) {
        uint32_t r[32];
        uint4 cur[4] = {nxt[0], nxt[1], nxt[2], nxt[3]};
        tmem_ld32(taddr + c * 32, r);
        if (c + 1 < chunks) prefetch(c + 1);
        tmem_ld_wait();
        if (c == chunks - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(smem_u32(&tempty[acc]) & kPeerBitMask);    // the even CTA's barrier
        }
        epilogue_chunk<256>(p, r, row, col_base + c * 32, split, 0, pre_base ? cur : nullptr, ts);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (ts && lane == 0) tma_store_wait_read0();         // the staging buffers stay valid until the last store has read them
  }
  pdl_launch_dependents();               // this CTA's work is issued: the next kernel's CTAs may take the SM as it drains
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                    // neither CTA leaves (or frees TMEM) while the other may still touch it
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair<Cfg::TMEM_COLS>(tmem_base); }
}

template <int A_MN, int B_MN, int LEAN>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const CUtensorMap& tc,
                            const CUtensorMap& taux, const GemmParams& p, int grid, cudaStream_t st) {
  auto kfn = gemm_pair_bf16_kernel<A_MN, B_MN, LEAN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::SMEM_BYTES) != cudaSuccess) return OA_ERR_LAUNCH;
    attr_set = true;
  }
  static const int epi_warps = [] { const char* e = getenv("OA_GEMM_PAIR_EPI_WARPS"); return (e && atoi(e) == 4) ? 4 : 8; }();
  const cudaError_t e = launch_pdl(kfn, dim3(grid), dim3(64 + 32 * epi_warps), PairCfg::SMEM_BYTES, st, ta, tb, tb2, tc, taux, p);
  return (e == cudaSuccess && cudaGetLastError() == cudaSuccess) ? OA_OK : OA_ERR_LAUNCH;
}

// Fixed-order reduction of split-K partials (deterministic), then the plain store / accumulate epilogue.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N, void* out, int ldc,
                                     int out_f32, int accumulate, int batch, long long sc_batch) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i4 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t total4 = (size_t)batch * M * N / 4;
  if (i4 >= total4) return;
  size_t e = i4 * 4;
  size_t per = (size_t)M * N;
  int bi = (int)(e / per);
  size_t eb = e - (size_t)bi * per;
  int row = (int)(eb / N), col = (int)(eb % N);
  float4 s = *reinterpret_cast<const float4*>(ws + e);
  for (int k = 1; k < splits; ++k) {
    float4 x = *reinterpret_cast<const float4*>(ws + (size_t)k * batch * per + e);
    s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
  }
  if (out_f32) {
    float* o = reinterpret_cast<float*>(out) + bi * sc_batch + (size_t)row * ldc + col;
    if (accumulate) {
      float4 c = *reinterpret_cast<float4*>(o);
      s.x += c.x; s.y += c.y; s.z += c.z; s.w += c.w;
    }
    *reinterpret_cast<float4*>(o) = s;
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + bi * sc_batch + (size_t)row * ldc + col;
    if (accumulate) {
      uint2 c = *reinterpret_cast<uint2*>(o);
      float2 a = unpack_bf16x2(c.x), b = unpack_bf16x2(c.y);
      s.x += a.x; s.y += a.y; s.z += b.x; s.w += b.y;
    }
    *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16x2(s.x, s.y), pack_bf16x2(s.z, s.w));
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(f);
  });
  return fn;
}

// 2-D bf16 tensor map: inner (contiguous) extent `inner`, outer extent `outer`, row pitch `ld` elements.
int make_tmap_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer, int swizzle_bytes) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return OA_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15)) return OA_ERR_ALIGN;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OA_OK : OA_ERR_DRIVER;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
  return make_tmap_2d_bf16(out, ptr, inner, outer, ld, box_inner, box_outer, 128);
}

// 3-D bf16 tensor map: [batch][outer][inner], box = one [box_outer x box_inner] tile of one problem.
int make_tmap_3d_bf16(CUtensorMap* out, const void* ptr, uint64_t inner, uint64_t outer, uint64_t batch, uint64_t ld,
                      uint64_t batch_stride, uint32_t box_inner, uint32_t box_outer) {
  PFN_encodeTiled enc = get_encode();
  if (!enc) return OA_ERR_DRIVER;
  if (batch <= 1) batch_stride = ld * outer;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15) || ((batch_stride * 2) & 15)) return OA_ERR_ALIGN;
  cuuint64_t dims[3] = {inner, outer, batch < 1 ? 1 : batch};
  cuuint64_t strides[2] = {ld * 2, batch_stride * 2};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OA_OK : OA_ERR_DRIVER;
}

#ifdef OA_GEMM_PROBE
extern "C" int gemm_pair_probe_read(long long* host, int n) {
  return cudaMemcpyFromSymbol(host, g_pair_probe, sizeof(long long) * (n < 512 ? n : 512)) == cudaSuccess ? OA_OK : OA_ERR_DRIVER;
}
#endif

// Rank-3 store map {cols, rows, problems} with [32 x 32] boxes in the 64-byte swizzle, for the TMA-store epilogue of the
// single-CTA kernel.  Sets p.tma_store when the output qualifies: bf16, written (not accumulated, not split), no second
// output, pointer and pitches on 16-byte boundaries.  OA_GEMM_TMA_STORE=0 keeps the per-lane stores.
static void try_store_map(GemmParams& p, void* out, uint64_t cols, uint64_t rows, uint64_t problems, uint64_t ld, uint64_t problem_stride) {
  static const bool enabled = []() { const char* e = std::getenv("OA_GEMM_TMA_STORE"); return !(e && (e[0] == '0' || e[0] == 'p')); }();   // "pair": CTA-pair kernel only
  p.tma_store = 0;
  if (!enabled || p.out_f32 || p.accumulate || p.splits != 1 || p.aux_out || p.tp_mode) return;
  PFN_encodeTiled enc = get_encode();
  if (!enc) return;
  if (problems <= 1) { problems = 1; problem_stride = ld * rows; }
  if ((reinterpret_cast<uintptr_t>(out) & 15) || ((ld * 2) & 15) || ((problem_stride * 2) & 15)) return;
  cuuint64_t dims[3] = {cols, rows, problems};
  cuuint64_t strides[2] = {ld * 2, problem_stride * 2};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if (enc(&p.tm_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, out, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
    p.tma_store = 1;
}

int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int BN, int A_MN, int B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t st,
                       const CUtensorMap* ta2 = nullptr) {
  auto kfn = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::SMEM_BYTES) != cudaSuccess)
      return OA_ERR_LAUNCH;
    attr_set = true;
  }
  if (p.tp_mode) {   // kernels that wait on other ranks start the ordinary way; the reduce-scatter mode's staging is laid out for 4 warps
    kfn<<<grid, p.tp_mode == 2 ? 192 : 320, GemmCfg<BN>::SMEM_BYTES, st>>>(ta, tb, ta2 ? *ta2 : ta, p);
    return cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH;
  }
  const cudaError_t e = launch_pdl(kfn, dim3(grid), dim3(320), GemmCfg<BN>::SMEM_BYTES, st, ta, tb, ta2 ? *ta2 : ta, p);
  return (e == cudaSuccess && cudaGetLastError() == cudaSuccess) ? OA_OK : OA_ERR_LAUNCH;
}

}  // namespace oa

using namespace oa;

extern "C" int oa_gemm_plan_splits(int M, int N, int K, int bn, int sms) {
  // Choose a split-K factor so that the tile count fills the machine; only worth it for long K.
  int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  int kb = (K + BK - 1) / BK;
  if (tiles >= sms || kb < 16) return 1;
  int best = 1;
  double best_eff = 0;
  for (int s = 1; s <= 16 && kb / s >= 8; ++s) {
    int t = tiles * s;
    int waves = (t + sms - 1) / sms;
    double eff = (double)t / (waves * sms);
    if (eff > best_eff + 0.04) { best_eff = eff; best = s; }
  }
  return best;
}

extern "C" size_t oa_gemm_workspace_bytes(int M, int N, int K) {
  int bn = (N >= 256) ? 256 : 128;
  int s = oa_gemm_plan_splits(M, N, K, bn, 148);
  int s2 = oa_gemm_plan_splits(M, N, K, 128, 148);
  if (s2 > s) s = s2;
  return s > 1 ? (size_t)s * M * N * sizeof(float) : 0;
}

extern "C" int oa_gemm_bf16_batched(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc,
                                    int a_mn, int b_mn, const void* bias, const void* residual, int ldr, void* aux_out,
                                    const void* aux_in, int ldaux, int act, int out_f32, int accumulate, float alpha,
                                    void* workspace, size_t workspace_bytes, int force_bn, int batch, long long sa_batch,
                                    long long sb_batch, long long sc_batch, long long sr_batch, long long saux_batch,
                                    long long sbias_batch, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return OA_ERR_ARG;
  if ((N & 7) || (K & 7) || (a_mn && (M & 7))) return OA_ERR_ALIGN;
  if ((ldc & (out_f32 ? 3 : 7)) || (residual && (ldr & 7)) || ((aux_out || aux_in) && (ldaux & 7))) return OA_ERR_ALIGN;
  if (batch > 1 && ((sc_batch & 7) || (sr_batch & 7) || (saux_batch & 7) || (sbias_batch & 7))) return OA_ERR_ALIGN;
  int bn = force_bn ? force_bn : ((N >= 256) ? 256 : 128);
  int sms = num_sms();
  if (!force_bn && bn == 256) {
    // Prefer the 128-wide tile when it fills the machine noticeably better.
    long long t256 = (long long)batch * ((M + BM - 1) / BM) * ((N + 255) / 256), t128 = (long long)batch * ((M + BM - 1) / BM) * ((N + 127) / 128);
    double e256 = (double)t256 / (((t256 + sms - 1) / sms) * sms), e128 = (double)t128 / (((t128 + sms - 1) / sms) * sms);
    if (t256 < sms && e128 > e256 + 0.15) bn = 128;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldc = ldc; p.out_f32 = out_f32;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual; p.ldr = ldr;
  p.aux_out = (__nv_bfloat16*)aux_out; p.aux_in = (const __nv_bfloat16*)aux_in; p.ldaux = ldaux;
  p.act = act; p.accumulate = accumulate; p.alpha = alpha;
  p.status = status;
  p.group_m = 16;
  static const int pair_group = []() { const char* e = std::getenv("OA_GEMM_PAIR_GROUP"); int v = e ? atoi(e) : 8; return v > 0 ? v : 8; }();
  p.pair_group_m = pair_group;
  static const int epi_pf = []() { const char* e = std::getenv("OA_GEMM_EPI_PREFETCH"); return (e && e[0] == '0') ? 0 : 1; }();
  p.epi_prefetch = epi_pf;
  p.tma_store = 0;
  p.splits = 1;
  p.workspace = (float*)workspace;
  p.batch = batch; p.sc_batch = sc_batch; p.sr_batch = sr_batch; p.saux_batch = saux_batch; p.sbias_batch = sbias_batch;
  p.group_mode = 0; p.group_offsets = nullptr; p.tp_mode = 0; p.tp_comm = 0;
  bool plain = !bias && !residual && !aux_out && !aux_in && act == OA_ACT_NONE;
  const bool can_split = workspace && plain && (N % 4 == 0);
  CUtensorMap ta, tb;
  int rc;
  cudaStream_t st = (cudaStream_t)stream;
  // CTA-pair kernel: 2-D problems of at least one 256 x 256 tile (OA_GEMM_PAIR=0 switches it off).  With fewer tiles than CTA
  // pairs the reduction is split (fp32 partials in the workspace, fixed-order reduce) so that the pairs are filled: the
  // weight-gradient shapes (small M x N, K = tokens) run here.
  static const bool pair_enabled = []() { const char* e = std::getenv("OA_GEMM_PAIR"); return !(e && e[0] == '0'); }();
  const long long tiles2 = (long long)((M + 255) / 256) * ((N + 255) / 256);
  if (pair_enabled && !force_bn && batch == 1 && M >= 256 && N >= 256 && (sms & 1) == 0) {
    const int P = sms / 2;
    const int kb_total = (K + BK - 1) / BK;
    int ps = 0;                                             // 0: do not use the pair kernel
    if (tiles2 >= P) ps = 1;
    else {
      // Fewer tiles than CTA pairs: choose the split count by a cost model in microseconds.  A k-block of a 256 x 256 tile
      // takes about 0.36 us in steady state, draining a tile about 2.5 us; the partials cost (splits + 1) passes over the
      // fp32 output at the rate of the reduce kernel (about 4 TB/s).
      auto cost = [&](int s2) {
        const int per = (kb_total + s2 - 1) / s2;
        const long long u = tiles2 * s2;
        const double waves = (double)((u + P - 1) / P);
        return waves * (per * 0.36 + 2.5) + (s2 > 1 ? (s2 + 1.0) * (double)M * N * 4.0 / 4.0e6 : 0.0);
      };
      int best = 1;
      double best_cost = cost(1);
      if (can_split) {
        for (int s2 = 2; s2 <= 16 && kb_total / s2 >= 16; ++s2) {
          const int per = (kb_total + s2 - 1) / s2;
          if ((long long)(s2 - 1) * per >= kb_total) continue;                    // an empty split
          if ((size_t)s2 * M * N * sizeof(float) > workspace_bytes) break;
          const double c = cost(s2);
          if (c < best_cost * 0.97) { best_cost = c; best = s2; }
        }
      }
      // worth a CTA-pair launch when the pairs are reasonably filled for most of the run
      if ((double)(tiles2 * best) / P >= 0.5) ps = best;
    }
    if (ps > 0) {
      p.splits = ps;
      if (a_mn) rc = make_tmap_3d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, 1, (uint64_t)lda, 0, 64, BK);
      else      rc = make_tmap_3d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, 1, (uint64_t)lda, 0, BK, BM);
      if (rc) return rc;
      if (b_mn) rc = make_tmap_3d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, 1, (uint64_t)ldb, 0, 64, BK);
      else      rc = make_tmap_3d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, 1, (uint64_t)ldb, 0, BK, 128);
      if (rc) return rc;
      CUtensorMap tb2 = tb;                                  // 64-row boxes of K-major B for the half-width tail units
      if (!b_mn) { rc = make_tmap_3d_bf16(&tb2, B, (uint64_t)K, (uint64_t)N, 1, (uint64_t)ldb, 0, BK, 64); if (rc) return rc; }
      // bf16 output without accumulation leaves through TMA stores ([32 x 32] boxes, 64-byte swizzle); OA_GEMM_TMA_STORE=0
      // keeps the per-lane stores
      static const bool ts_enabled = []() { const char* e = std::getenv("OA_GEMM_TMA_STORE"); return !(e && e[0] == '0'); }();
      CUtensorMap tc = ta, taux = ta;
      p.tma_store = 0;
      if (ts_enabled && ps == 1 && !out_f32 && !accumulate &&
          make_tmap_2d_bf16(&tc, out, (uint64_t)N, (uint64_t)M, (uint64_t)ldc, 32, 32, 64) == OA_OK &&
          (!aux_out || make_tmap_2d_bf16(&taux, aux_out, (uint64_t)N, (uint64_t)M, (uint64_t)ldaux, 32, 32, 64) == OA_OK))
        p.tma_store = 1;
      const long long units = tiles2 * ps;
      const int pgrid = (int)(units * 2 < sms ? units * 2 : sms);
      // specialised epilogues (small code): plain, + residual, GELU with pre-activation copy, GELU backward; anything else
      // (bias, other activations, fp32 output, accumulation, split-K) takes the generic instantiation
      static const bool lean_enabled = []() { const char* e = std::getenv("OA_GEMM_LEAN"); return !(e && e[0] == '0'); }();
      int lean = 0;
      if (lean_enabled && ps > 1) lean = 5;         // split-K runs only for plain products (N a multiple of 4)
      else if (lean_enabled && plain && out_f32) lean = 6;
      else if (lean_enabled && p.tma_store && !bias) {
        if (plain) lean = 1;
        else if (residual && !aux_out && !aux_in && act == OA_ACT_NONE) lean = 2;
        else if (!residual && aux_out && !aux_in && act == OA_ACT_GELU) lean = 3;
        else if (!residual && !aux_out && aux_in && act == OA_ACT_GELU_BWD) lean = 4;
      }
#define OA_PAIR_CASE(L)                                                                                    \
      switch ((a_mn ? 2 : 0) | (b_mn ? 1 : 0)) {                                                          \
        case 0: rc = launch_gemm_pair<0, 0, L>(ta, tb, tb2, tc, taux, p, pgrid, st); break;               \
        case 1: rc = launch_gemm_pair<0, 1, L>(ta, tb, tb2, tc, taux, p, pgrid, st); break;               \
        case 2: rc = launch_gemm_pair<1, 0, L>(ta, tb, tb2, tc, taux, p, pgrid, st); break;               \
        default: rc = launch_gemm_pair<1, 1, L>(ta, tb, tb2, tc, taux, p, pgrid, st); break;              \
      }
      switch (lean) {
        case 1: OA_PAIR_CASE(1); break;
        case 2: OA_PAIR_CASE(2); break;
        case 3: OA_PAIR_CASE(3); break;
        case 4: OA_PAIR_CASE(4); break;
        case 5: OA_PAIR_CASE(5); break;
        case 6: OA_PAIR_CASE(6); break;
        default: OA_PAIR_CASE(0); break;
      }
#undef OA_PAIR_CASE
      if (rc) return rc;
      if (p.splits > 1) {
        size_t total4 = (size_t)M * N / 4;
        unsigned blocks = (unsigned)((total4 + 255) / 256);
        if (launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, st, (const float*)p.workspace, p.splits, M, N, out, ldc, out_f32,
                       accumulate, 1, 0LL) != cudaSuccess || cudaGetLastError() != cudaSuccess) return OA_ERR_LAUNCH;
      }
      return OA_OK;
    }
  }
  if (can_split) {
    int s = oa_gemm_plan_splits(M * batch, N, K, bn, sms);
    if (s > 1 && (size_t)s * batch * M * N * sizeof(float) <= workspace_bytes) p.splits = s;
  }
  if (a_mn) rc = make_tmap_3d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, batch, (uint64_t)lda, sa_batch, 64, BK);
  else      rc = make_tmap_3d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, batch, (uint64_t)lda, sa_batch, BK, BM);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_3d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, batch, (uint64_t)ldb, sb_batch, 64, BK);
  else      rc = make_tmap_3d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, batch, (uint64_t)ldb, sb_batch, BK, (uint32_t)bn);
  if (rc) return rc;
  long long tiles = (long long)batch * ((M + BM - 1) / BM) * ((N + bn - 1) / bn) * p.splits;
  int grid = tiles < sms ? (int)tiles : sms;
  try_store_map(p, out, (uint64_t)N, (uint64_t)M, (uint64_t)batch, (uint64_t)ldc, (uint64_t)sc_batch);
  int sel = (bn == 256 ? 4 : 0) | (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  switch (sel) {
    case 0: rc = launch_gemm<128, 0, 0>(ta, tb, p, grid, st); break;
    case 1: rc = launch_gemm<128, 0, 1>(ta, tb, p, grid, st); break;
    case 2: rc = launch_gemm<128, 1, 0>(ta, tb, p, grid, st); break;
    case 3: rc = launch_gemm<128, 1, 1>(ta, tb, p, grid, st); break;
    case 4: rc = launch_gemm<256, 0, 0>(ta, tb, p, grid, st); break;
    case 5: rc = launch_gemm<256, 0, 1>(ta, tb, p, grid, st); break;
    case 6: rc = launch_gemm<256, 1, 0>(ta, tb, p, grid, st); break;
    default: rc = launch_gemm<256, 1, 1>(ta, tb, p, grid, st); break;
  }
  if (rc) return rc;
  if (p.splits > 1) {
    size_t total4 = (size_t)batch * M * N / 4;
    int threads = 256;
    unsigned blocks = (unsigned)((total4 + threads - 1) / threads);
    splitk_reduce_kernel<<<blocks, threads, 0, st>>>(p.workspace, p.splits, M, N, out, ldc, out_f32, accumulate, batch, sc_batch);
    if (cudaGetLastError() != cudaSuccess) return OA_ERR_LAUNCH;
  }
  return OA_OK;
}

extern "C" int oa_gemm_bf16(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc,
                            int a_mn, int b_mn, const void* bias, const void* residual, int ldr, void* aux_out,
                            const void* aux_in, int ldaux, int act, int out_f32, int accumulate, float alpha,
                            void* workspace, size_t workspace_bytes, int force_bn, int* status, void* stream) {
  return oa_gemm_bf16_batched(A, B, out, M, N, K, lda, ldb, ldc, a_mn, b_mn, bias, residual, ldr, aux_out, aux_in, ldaux, act,
                              out_f32, accumulate, alpha, workspace, workspace_bytes, force_bn, 1, 0, 0, 0, 0, 0, 0, status, stream);
}

// Grouped GEMMs for mixture-of-experts layers (group segments padded to multiples of 128 rows, offsets on the device).
//   mode 1: out[r, :] = act(A[r, :] * B[g(r)]^T + bias[g(r)])   A [max_rows, K], B [groups, N, K] (or [groups, K, N] when b_mn)
//   mode 2: out[g]    = A_g^T * B_g (+ out[g])                  A [max_rows, M], B [max_rows, N], out [groups, M, N]
extern "C" int oa_gemm_bf16_grouped(int mode, const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb,
                                    int ldc, int b_mn, const void* bias, int act, void* aux_out, const void* aux_in, int ldaux,
                                    int out_f32, int accumulate, int groups, const int* offsets, long long max_rows,
                                    long long sb_batch, long long sc_batch, long long sbias_batch, int* status, void* stream) {
  if (mode != 1 && mode != 2) return OA_ERR_ARG;
  if (groups < 1 || groups > 256 || max_rows <= 0 || (max_rows & 127)) return OA_ERR_ARG;
  if ((N & 7) || (ldc & (out_f32 ? 3 : 7))) return OA_ERR_ALIGN;
  int sms = num_sms();
  GemmParams p;
  p.N = N; p.out = out; p.ldc = ldc; p.out_f32 = out_f32;
  p.bias = (const __nv_bfloat16*)bias; p.residual = nullptr; p.ldr = 0;
  p.aux_out = (__nv_bfloat16*)aux_out; p.aux_in = (const __nv_bfloat16*)aux_in; p.ldaux = ldaux;
  p.act = act; p.accumulate = accumulate; p.alpha = 1.f; p.status = status; p.group_m = 16; p.pair_group_m = 8; p.epi_prefetch = 0; p.tma_store = 0; p.splits = 1; p.workspace = nullptr;
  p.batch = groups; p.sr_batch = 0; p.saux_batch = 0; p.sbias_batch = sbias_batch;
  p.group_mode = mode; p.group_offsets = offsets; p.tp_mode = 0; p.tp_comm = 0;
  CUtensorMap ta, tb;
  int rc, bn, grid;
  if (mode == 1) {
    if (K & 7) return OA_ERR_ALIGN;
    p.M = (int)max_rows; p.K = K; p.sc_batch = 0;
    bn = (N >= 256) ? 256 : 128;
    if ((rc = make_tmap_3d_bf16(&ta, A, (uint64_t)K, (uint64_t)max_rows, 1, (uint64_t)lda, 0, BK, BM))) return rc;
    if (b_mn) rc = make_tmap_3d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, groups, (uint64_t)ldb, sb_batch, 64, BK);
    else      rc = make_tmap_3d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, groups, (uint64_t)ldb, sb_batch, BK, (uint32_t)bn);
    if (rc) return rc;
    grid = sms;   // the tile count lives on the device; surplus CTAs exit immediately
  } else {
    if ((M & 7)) return OA_ERR_ALIGN;
    p.M = M; p.K = (int)max_rows; p.sc_batch = sc_batch;
    bn = (N >= 256) ? 256 : 128;
    if ((rc = make_tmap_3d_bf16(&ta, A, (uint64_t)M, (uint64_t)max_rows, 1, (uint64_t)lda, 0, 64, BK))) return rc;
    if ((rc = make_tmap_3d_bf16(&tb, B, (uint64_t)N, (uint64_t)max_rows, 1, (uint64_t)ldb, 0, 64, BK))) return rc;
    long long tiles = (long long)groups * ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    grid = tiles < sms ? (int)tiles : sms;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == 1) try_store_map(p, out, (uint64_t)N, (uint64_t)max_rows, 1, (uint64_t)ldc, 0);
  else try_store_map(p, out, (uint64_t)N, (uint64_t)M, (uint64_t)groups, (uint64_t)ldc, (uint64_t)sc_batch);
  if (mode == 1) {
    if (bn == 256) rc = b_mn ? launch_gemm<256, 0, 1>(ta, tb, p, grid, st) : launch_gemm<256, 0, 0>(ta, tb, p, grid, st);
    else           rc = b_mn ? launch_gemm<128, 0, 1>(ta, tb, p, grid, st) : launch_gemm<128, 0, 0>(ta, tb, p, grid, st);
  } else {
    rc = bn == 256 ? launch_gemm<256, 1, 1>(ta, tb, p, grid, st) : launch_gemm<128, 1, 1>(ta, tb, p, grid, st);
  }
  return rc;
}

// Tensor-parallel GEMMs fused with their collective (modes described at GemmParams::tp_mode).
//   mode 1: out[M, N] = allgather_rows(src)[M, K] * B^T.  `stage_local` is this rank's staging buffer [M, K] (= bufs[rank]).
//   mode 2: out[M / world, N] = reduce_scatter_rows(A[M, K] * B^T) (+ residual [M / world, N]).
// bufs / flags are host arrays of `world` device pointers (every rank's staging buffer and flag array, peer mapped);
// sync2 is a device u64[2] that belongs to the call site.  M must be a multiple of 128 * world.
extern "C" int oa_gemm_bf16_tp(int mode, const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldc,
                               int b_mn, const void* residual, int ldr, int out_f32, float alpha, const void* src, int ld_src,
                               const void* const* bufs, const void* const* flags, void* sync2, int world, int rank,
                               int comm_ctas, int* status, void* stream) {
  if (mode != 1 && mode != 2) return OA_ERR_ARG;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return OA_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || (M % (BM * world))) return OA_ERR_ARG;
  if ((N & 7) || (K & 7) || (ldc & (out_f32 ? 3 : 7)) || (residual && (ldr & 7))) return OA_ERR_ALIGN;
  if (mode == 1 && ((ld_src & 7) || lda != K)) return OA_ERR_ALIGN;
  const int sms = num_sms();
  comm_ctas = 0;      // kept in the signature for callers; the push is spread over the epilogue warps of all CTAs
  const int bn = (N >= 256) ? 256 : 128;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldc = ldc; p.out_f32 = out_f32;
  p.bias = nullptr; p.residual = (const __nv_bfloat16*)residual; p.ldr = ldr;
  p.aux_out = nullptr; p.aux_in = nullptr; p.ldaux = 0;
  p.act = OA_ACT_NONE; p.accumulate = 0; p.alpha = alpha; p.status = status; p.group_m = 16; p.pair_group_m = 8; p.epi_prefetch = 0; p.tma_store = 0; p.splits = 1; p.workspace = nullptr;
  p.batch = 1; p.sc_batch = 0; p.sr_batch = 0; p.saux_batch = 0; p.sbias_batch = 0;
  p.group_mode = 0; p.group_offsets = nullptr;
  p.tp_mode = mode; p.tp_world = world; p.tp_rank = rank; p.tp_comm = comm_ctas;
  p.tp_src = (const __nv_bfloat16*)src; p.tp_ld_src = ld_src;
  for (int i = 0; i < MAX_RANKS; ++i) {
    p.tp_bufs.ptr[i] = i < world ? const_cast<void*>(bufs[i]) : nullptr;
    p.tp_flags.ptr[i] = i < world ? const_cast<void*>(flags[i]) : nullptr;
  }
  p.tp_sync = (unsigned long long*)sync2;
  if (mode == 2) p.residual = (const __nv_bfloat16*)residual;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_3d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, 1, (uint64_t)lda, 0, BK, BM))) return rc;
  if (b_mn) rc = make_tmap_3d_bf16(&tb, B, (uint64_t)N, (uint64_t)K, 1, (uint64_t)ldb, 0, 64, BK);
  else      rc = make_tmap_3d_bf16(&tb, B, (uint64_t)K, (uint64_t)N, 1, (uint64_t)ldb, 0, BK, (uint32_t)bn);
  if (rc) return rc;
  CUtensorMap ta2;
  const CUtensorMap* pa2 = nullptr;
  if (mode == 1) {     // this rank's own rows are read in place from the shard
    if ((rc = make_tmap_3d_bf16(&ta2, src, (uint64_t)K, (uint64_t)(M / world), 1, (uint64_t)ld_src, 0, BK, BM))) return rc;
    pa2 = &ta2;
  }
  // every CTA takes part in the protocol (communication CTAs, the row reduction, the epoch hand-over): a full grid always
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) rc = b_mn ? launch_gemm<256, 0, 1>(ta, tb, p, sms, st, pa2) : launch_gemm<256, 0, 0>(ta, tb, p, sms, st, pa2);
  else           rc = b_mn ? launch_gemm<128, 0, 1>(ta, tb, p, sms, st, pa2) : launch_gemm<128, 0, 0>(ta, tb, p, sms, st, pa2);
  return rc;
}
