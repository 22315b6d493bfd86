// Peer-memory communication kernels over NVLink / NVSwitch (one process per GPU, CUDA IPC mapped buffers).
//
// The reference has no device collectives: its OaCollective stages through host memory
// (Source/Private/Oa/Runtime/Distributed/Collective.cpp:75-247) and nothing in its optimizers synchronises
// gradients.  Here the data-parallel step is ONE kernel per bucket that fuses
//     gradient reduce-scatter (peer loads of every rank's bf16 gradient shard, fp32 sum)
//   + gradient scale / clip
//   + the partitioned Adam / AdamW update on this rank's fp32 master / m / v shard
//   + the parameter all-gather (bf16 write-back pushed straight into every peer's parameter arena)
// so gradients cross NVLink once as bf16 and parameters once as bf16, with no staging buffers.
//
// Synchronisation: monotonically increasing epochs in device memory (graph-replay safe).  `oa_peer_signal`
// publishes "my buffers are ready" to every peer's flag slot (fence.sys + st.release.sys); consumers poll
// their own slots with ld.acquire.sys under an iteration limit and report OA_KERR_WAIT_PEER to the status
// word when the limit runs out (no unbounded spin, no trap).  Kernels never wait on another kernel of the
// same GPU, and no block waits on another block, so co-residency is never required.
// Only plain peer loads / stores are used here (no TMA from peer memory, no cluster multicast).
#include "common.cuh"
#include "api.h"

namespace oa {

// Upper bound of every wait on a peer, in nanoseconds of wall time (set from the host with oa_set_peer_wait_ms).  Ranks
// drift apart by whole host phases (a data-loader stall, a checkpoint write), so the bound is wall time, not iterations.
__device__ unsigned long long g_peer_wait_ns = OA_WAIT_LIMIT_NS;

// Waits until every slot in `flags[0..world)` has reached `target`.  Returns false when the time limit runs out.
__device__ __forceinline__ bool wait_flags(const unsigned long long* flags, int world, unsigned long long target) {
  uint64_t t0 = 0;
  const unsigned long long limit = g_peer_wait_ns;
  for (int r = 0; r < world; ++r) {
    uint32_t it = 0;
    while (ld_acquire_sys(flags + r) < target) {
      if ((++it & 0x3f) == 0) {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit) return false;
        __nanosleep(it > 2048 ? 512 : 64);
      }
    }
  }
  return true;
}

// epoch_local[0] += 1, then write the new epoch into slot `rank` of every peer's flag array.
// flags_peers.ptr[r] points at rank r's array of `world` u64 slots for this channel.
__global__ void peer_signal_kernel(PeerTable flags_peers, unsigned long long* epoch_local, int rank, int world) {
  if (threadIdx.x == 0) {
    unsigned long long e = epoch_local[0] + 1;
    epoch_local[0] = e;
    __threadfence_system();
  }
  __syncthreads();
  unsigned long long e = epoch_local[0];
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned long long*>(flags_peers.ptr[threadIdx.x]) + rank, e);
  }
}

// Blocks the stream until all peers have signalled the current epoch of this channel (bounded).
__global__ void peer_wait_kernel(const unsigned long long* my_flags, const unsigned long long* epoch_local, int world,
                                 int* status) {
  if (threadIdx.x == 0) {
    if (!wait_flags(my_flags, world, epoch_local[0])) report_error(status, OA_KERR_WAIT_PEER);
  }
}

struct DpParams {
  PeerTable grads;      // every rank's bf16 gradient arena (same layout on all ranks)
  PeerTable params;     // every rank's bf16 parameter arena
  float* master;        // this rank's shard: fp32 master weights [shard]
  float* m;             // [shard]
  float* v;             // [shard]
  long long shard_lo;   // first element of this rank's shard (multiple of 8)
  long long shard_n;    // elements in this rank's shard (multiple of 8)
  const float* state;   // {step, lr, beta1, beta2, eps, wd, grad_scale, _} (step already advanced)
  const float* inv_clip;
  int decoupled;
  int rank, world;
  const unsigned long long* my_flags;     // readiness of every rank's gradients (channel A)
  const unsigned long long* epoch_local;
  int* status;
};

// One kernel: wait for every rank's gradients, reduce this rank's shard over all peers, Adam on the fp32
// master shard, push the bf16 result into every rank's parameter arena.  8 elements (16 bytes) per thread step.
__global__ void __launch_bounds__(256)
dp_reduce_adam_gather_kernel(const DpParams p) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    bool ok = wait_flags(p.my_flags, p.world, p.epoch_local[0]);
    if (!ok) report_error(p.status, OA_KERR_WAIT_PEER);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const float step = p.state[0], lr = p.state[1], b1 = p.state[2], b2 = p.state[3], eps = p.state[4], wd = p.state[5];
  const float gs = p.state[6] * (p.inv_clip ? p.inv_clip[0] : 1.f);
  const float bc1 = 1.f - powf(b1, step), bc2 = 1.f - powf(b2, step);
  const long long nvec = p.shard_n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const long long e = p.shard_lo + i * 8;   // element index in the arena
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int rr = 0; rr < MAX_RANKS; ++rr) {
      if (rr < p.world) {
        int r = (p.rank + rr) % p.world;      // start with the local copy, spread peer traffic
        uint4 x = ld_peer_v4(reinterpret_cast<const __nv_bfloat16*>(p.grads.ptr[r]) + e);
        float2 a = unpack_bf16x2(x.x), b = unpack_bf16x2(x.y), c = unpack_bf16x2(x.z), d = unpack_bf16x2(x.w);
        g[0] += a.x; g[1] += a.y; g[2] += b.x; g[3] += b.y; g[4] += c.x; g[5] += c.y; g[6] += d.x; g[7] += d.y;
      }
    }
    float4 w0 = *reinterpret_cast<const float4*>(p.master + i * 8), w1 = *reinterpret_cast<const float4*>(p.master + i * 8 + 4);
    float4 m0 = *reinterpret_cast<const float4*>(p.m + i * 8), m1 = *reinterpret_cast<const float4*>(p.m + i * 8 + 4);
    float4 v0 = *reinterpret_cast<const float4*>(p.v + i * 8), v1 = *reinterpret_cast<const float4*>(p.v + i * 8 + 4);
    float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gj = g[j] * gs;
      float wj = w[j];
      if (p.decoupled) wj -= lr * wd * wj; else gj += wd * wj;
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      w[j] = wj - lr * (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
    }
    *reinterpret_cast<float4*>(p.master + i * 8) = make_float4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<float4*>(p.master + i * 8 + 4) = make_float4(w[4], w[5], w[6], w[7]);
    *reinterpret_cast<float4*>(p.m + i * 8) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(p.m + i * 8 + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
    *reinterpret_cast<float4*>(p.v + i * 8) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    *reinterpret_cast<float4*>(p.v + i * 8 + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    uint4 out = make_uint4(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]), pack_bf16x2(w[4], w[5]), pack_bf16x2(w[6], w[7]));
#pragma unroll
    for (int rr = 0; rr < MAX_RANKS; ++rr) {
      if (rr < p.world) {
        int r = (p.rank + rr) % p.world;
        st_peer_v4(reinterpret_cast<__nv_bfloat16*>(p.params.ptr[r]) + e, out);
      }
    }
  }
}

// ---- gradient-norm clipping under the fused step.  The norm is that of the SUMMED gradient, so each rank sums its shard over
// the peers once more (sum of squares only, nothing written back), publishes the scalar to every rank, and the clip
// coefficient is computed from the `world` scalars in rank order: the same value, bit for bit, on every rank.
constexpr int DP_SUMSQ_BLOCKS = 296;
__global__ void __launch_bounds__(256)
dp_shard_sumsq_kernel(PeerTable grads, long long shard_lo, long long shard_n, int rank, int world, float* partial, int accumulate) {
  __shared__ float s_w[8];
  const long long nvec = shard_n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const long long e = shard_lo + i * 8;
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int rr = 0; rr < MAX_RANKS; ++rr) {
      if (rr < world) {
        const int r = (rank + rr) % world;
        const uint4 x = ld_peer_v4(reinterpret_cast<const __nv_bfloat16*>(grads.ptr[r]) + e);
        const float2 a = unpack_bf16x2(x.x), b = unpack_bf16x2(x.y), c = unpack_bf16x2(x.z), d = unpack_bf16x2(x.w);
        g[0] += a.x; g[1] += a.y; g[2] += b.x; g[3] += b.y; g[4] += c.x; g[5] += c.y; g[6] += d.x; g[7] += d.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc = fmaf(g[j], g[j], acc);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += s_w[w];
    partial[blockIdx.x] = accumulate ? partial[blockIdx.x] + t : t;
  }
}
// One warp: sum of the block partials in a fixed order, written into slot `rank` (16-byte slots) of every rank.
__global__ void dp_sumsq_publish_kernel(const float* partial, int n_partial, PeerTable slots, int rank, int world) {
  float t = 0.f;
  for (int i = threadIdx.x; i < n_partial; i += 32) t += partial[i];
  t = warp_sum(t);
  if (threadIdx.x < world)
    *reinterpret_cast<volatile float*>(reinterpret_cast<float*>(slots.ptr[threadIdx.x]) + rank * 4) = t;
  __threadfence_system();
}
__global__ void dp_clip_finalize_kernel(const float* slots, int world, const float* extra, float max_norm, float* coef) {
  float t = extra ? extra[0] : 0.f;
  for (int r = 0; r < world; ++r) t += *reinterpret_cast<const volatile float*>(slots + r * 4);
  const float nrm = sqrtf(t);
  coef[0] = nrm > max_norm ? max_norm / (nrm + 1e-6f) : 1.f;
  coef[1] = nrm;
}

// Generic peer collectives on fp32 / bf16 buffers (OaCollective verbs), pull-based, bounded by the caller's
// signal / wait kernels: out[i] = reduce_r in[r][lo + i].
template <typename T>
__global__ void peer_reduce_kernel(PeerTable in, T* out, long long lo, long long n, int world, int op) {
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) {
      const T* src = reinterpret_cast<const T*>(in.ptr[r]) + lo + i;
      float x;
      if constexpr (sizeof(T) == 4) x = *reinterpret_cast<const volatile float*>(src);
      else { unsigned short u = *reinterpret_cast<const volatile unsigned short*>(src); __nv_bfloat16_raw raw; raw.x = u; x = __bfloat162float(__nv_bfloat16(raw)); }
      if (r == 0) acc = x;
      else acc = op == 0 ? acc + x : (op == 1 ? fmaxf(acc, x) : fminf(acc, x));
    }
    if constexpr (sizeof(T) == 4) out[i] = acc; else out[i] = __float2bfloat16_rn(acc);
  }
}
// dst_peers[r][dst_off + i] = src[i] for every r (all-gather / broadcast push), 16 bytes per thread step.
__global__ void peer_push_kernel(PeerTable dst, long long dst_off_bytes, const void* src, long long nbytes, int world) {
  long long nvec = nbytes / 16;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    uint4 x = reinterpret_cast<const uint4*>(src)[i];
    for (int r = 0; r < world; ++r)
      st_peer_v4(reinterpret_cast<char*>(dst.ptr[r]) + dst_off_bytes + i * 16, x);
  }
}

// ---- one-shot all-reduce for small bf16 messages (tensor-parallel decoding: a [batch, d_model] partial sum per GEMM)
// ONE kernel: CTA c pushes its 2048-element range of `src` into slot `rank` of every rank's staging buffer, adds 1 to counter c
// of every rank (release), waits until its own counter c shows all `world` pushes of this call (bounded), then sums the `world`
// slots of its range in fp32 (+ residual) into `out`.  A CTA only ever waits for the same-index CTAs of the peers, never for a
// CTA of its own grid, so no co-residency is assumed.  Two staging halves alternate by call parity: a rank can only start
// call k+2 after every rank has pushed for call k+1, i.e. after every rank finished reading call k.  The call index lives
// in device memory (sync[0] = calls completed, sync[1] = CTAs done in the current call, sync[2 + c] = calls in which CTA c
// took part: messages of different sizes use different numbers of CTAs), so the kernel replays in a graph.
struct ArParams {
  PeerTable slots;        // every rank's staging buffer: [2 halves][world slots][slot_elems] bf16
  PeerTable counters;     // every rank's counter array: u64 per CTA
  const __nv_bfloat16* src;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  unsigned long long* sync;
  int* status;
  long long n, slot_elems;
  int world, rank;
};

__global__ void __launch_bounds__(256) peer_allreduce_oneshot_kernel(ArParams p) {
  __shared__ int s_ok;
  const unsigned long long call = p.sync[0];
  const long long half_off = (long long)(call & 1) * p.world * p.slot_elems;
  const long long i0 = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;
  const bool live = i0 < p.n;                            // n is a multiple of 8
  if (live) {
    const uint4 v = *reinterpret_cast<const uint4*>(p.src + i0);
    for (int q = 0; q < p.world; ++q) {
      const int r = (p.rank + q) % p.world;              // start with the own slot, spread the peers
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.slots.ptr[r]) + half_off + (long long)p.rank * p.slot_elems + i0) = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int r = 0; r < p.world; ++r)
      red_release_sys_add(reinterpret_cast<unsigned long long*>(p.counters.ptr[r]) + blockIdx.x, 1ull);
    const unsigned long long seen = p.sync[2 + blockIdx.x];
    const bool ok = wait_ge_sys(reinterpret_cast<const unsigned long long*>(p.counters.ptr[p.rank]) + blockIdx.x,
                                (seen + 1) * (unsigned long long)p.world);
    p.sync[2 + blockIdx.x] = seen + 1;
    if (!ok) report_error(p.status, OA_KERR_WAIT_PEER);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (live && s_ok) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(p.slots.ptr[p.rank]) + half_off + i0;
    for (int r = 0; r < p.world; ++r) {
      const uint4 v = ld_peer_v4(mine + (long long)r * p.slot_elems);     // peer-written data: read through L2
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    if (p.residual) {
      const uint4 v = *reinterpret_cast<const uint4*>(p.residual + i0);
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    *reinterpret_cast<uint4*>(p.out + i0) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                       pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned long long done = atomicAdd(&p.sync[1], 1ull) + 1ull;
    if (done == gridDim.x) { p.sync[1] = 0ull; __threadfence(); p.sync[0] = call + 1ull; }
  }
}

}  // namespace oa

using namespace oa;
#define ST ((cudaStream_t)stream)
#define CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? OA_OK : OA_ERR_LAUNCH)

static PeerTable make_table(const void* const* ptrs, int world) {
  PeerTable t;
  for (int i = 0; i < MAX_RANKS; ++i) t.ptr[i] = i < world ? const_cast<void*>(ptrs[i]) : nullptr;
  return t;
}

// ---- IPC-mapped buffers (host side) -------------------------------------------------------------
extern "C" int oa_ipc_alloc(size_t bytes, void** out) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return OA_ERR_DRIVER; }
  if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaFree(p); return OA_ERR_DRIVER; }
  *out = p;
  return OA_OK;
}
extern "C" int oa_ipc_free(void* p) { return cudaFree(p) == cudaSuccess ? OA_OK : OA_ERR_DRIVER; }
extern "C" int oa_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaGetLastError(); return OA_ERR_DRIVER; }
  memcpy(handle64, &h, sizeof(h));
  return OA_OK;
}
extern "C" int oa_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return OA_ERR_DRIVER; }
  *out = p;
  return OA_OK;
}
extern "C" int oa_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? OA_OK : OA_ERR_DRIVER; }

// ---- launches -----------------------------------------------------------------------------------
extern "C" int oa_peer_signal(const void* const* flags_peers, void* epoch_local, int rank, int world, void* stream) {
  if (world < 1 || world > MAX_RANKS) return OA_ERR_ARG;
  peer_signal_kernel<<<1, 32, 0, ST>>>(make_table(flags_peers, world), (unsigned long long*)epoch_local, rank, world);
  return CHECK_LAUNCH();
}
extern "C" int oa_peer_wait(const void* my_flags, const void* epoch_local, int world, int* status, void* stream) {
  if (world < 1 || world > MAX_RANKS) return OA_ERR_ARG;
  peer_wait_kernel<<<1, 32, 0, ST>>>((const unsigned long long*)my_flags, (const unsigned long long*)epoch_local, world, status);
  return CHECK_LAUNCH();
}
extern "C" int oa_dp_reduce_adam_gather(const void* const* grad_peers, const void* const* param_peers, float* master, float* m,
                                        float* v, long long shard_lo, long long shard_n, const float* state,
                                        const float* inv_clip, int decoupled, int rank, int world, const void* my_flags,
                                        const void* epoch_local, int* status, int max_blocks, void* stream) {
  if (world < 1 || world > MAX_RANKS) return OA_ERR_ARG;
  if ((shard_lo & 7) || (shard_n & 7)) return OA_ERR_ALIGN;
  if (shard_n == 0) return OA_OK;
  DpParams p;
  p.grads = make_table(grad_peers, world);
  p.params = make_table(param_peers, world);
  p.master = master; p.m = m; p.v = v;
  p.shard_lo = shard_lo; p.shard_n = shard_n; p.state = state; p.inv_clip = inv_clip; p.decoupled = decoupled;
  p.rank = rank; p.world = world;
  p.my_flags = (const unsigned long long*)my_flags; p.epoch_local = (const unsigned long long*)epoch_local; p.status = status;
  long long blocks = (shard_n / 8 + 255) / 256;
  long long cap = max_blocks > 0 ? max_blocks : 148 * 4;
  if (blocks > cap) blocks = cap;
  dp_reduce_adam_gather_kernel<<<(int)blocks, 256, 0, ST>>>(p);
  return CHECK_LAUNCH();
}
// Peer-to-peer attributes of the link from device `src` to device `dst` as the driver reports them:
// out[0] = access supported, out[1] = native atomics supported (true over NVLink, false over plain PCIe), out[2] = performance rank.
extern "C" int oa_p2p_attributes(int src, int dst, int* out) {
  if (!out) return OA_ERR_ARG;
  int v = 0;
  if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrAccessSupported, src, dst) != cudaSuccess) { cudaGetLastError(); return OA_ERR_DRIVER; }
  out[0] = v;
  if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrNativeAtomicSupported, src, dst) != cudaSuccess) { cudaGetLastError(); return OA_ERR_DRIVER; }
  out[1] = v;
  if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrPerformanceRank, src, dst) != cudaSuccess) { cudaGetLastError(); return OA_ERR_DRIVER; }
  out[2] = v;
  return OA_OK;
}
extern "C" int oa_set_peer_wait_ms(long long ms) {
  if (ms <= 0) return OA_ERR_ARG;
  const unsigned long long ns = (unsigned long long)ms * 1000000ull;
  return cudaMemcpyToSymbol(g_peer_wait_ns, &ns, sizeof(ns)) == cudaSuccess ? OA_OK : OA_ERR_DRIVER;
}
extern "C" int oa_dp_sumsq_blocks(void) { return DP_SUMSQ_BLOCKS; }
extern "C" int oa_dp_shard_sumsq(const void* const* grad_peers, long long shard_lo, long long shard_n, int rank, int world,
                                 float* partial, int accumulate, void* stream) {
  if (world < 1 || world > MAX_RANKS) return OA_ERR_ARG;
  if ((shard_lo & 7) || (shard_n & 7)) return OA_ERR_ALIGN;
  dp_shard_sumsq_kernel<<<DP_SUMSQ_BLOCKS, 256, 0, ST>>>(make_table(grad_peers, world), shard_lo, shard_n, rank, world, partial, accumulate);
  return CHECK_LAUNCH();
}
extern "C" int oa_dp_sumsq_publish(const float* partial, const void* const* slot_peers, int rank, int world, void* stream) {
  if (world < 1 || world > MAX_RANKS) return OA_ERR_ARG;
  dp_sumsq_publish_kernel<<<1, 32, 0, ST>>>(partial, DP_SUMSQ_BLOCKS, make_table(slot_peers, world), rank, world);
  return CHECK_LAUNCH();
}
extern "C" int oa_dp_clip_finalize(const float* slots, int world, const float* extra, float max_norm, float* coef, void* stream) {
  if (world < 1 || world > MAX_RANKS) return OA_ERR_ARG;
  dp_clip_finalize_kernel<<<1, 1, 0, ST>>>(slots, world, extra, max_norm, coef);
  return CHECK_LAUNCH();
}
extern "C" int oa_peer_reduce(int dtype, const void* const* in_peers, void* out, long long lo, long long n, int world, int op,
                              void* stream) {
  if (world < 1 || world > MAX_RANKS) return OA_ERR_ARG;
  if (n <= 0) return OA_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (dtype == OA_F32) peer_reduce_kernel<float><<<(int)blocks, 256, 0, ST>>>(make_table(in_peers, world), (float*)out, lo, n, world, op);
  else if (dtype == OA_BF16) peer_reduce_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, ST>>>(make_table(in_peers, world), (__nv_bfloat16*)out, lo, n, world, op);
  else return OA_ERR_UNSUPPORTED;
  return CHECK_LAUNCH();
}
extern "C" int oa_peer_push(const void* const* dst_peers, long long dst_off_bytes, const void* src, long long nbytes, int world,
                            void* stream) {
  if (world < 1 || world > MAX_RANKS) return OA_ERR_ARG;
  if ((nbytes & 15) || (dst_off_bytes & 15)) return OA_ERR_ALIGN;
  if (nbytes <= 0) return OA_OK;
  long long blocks = (nbytes / 16 + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  peer_push_kernel<<<(int)blocks, 256, 0, ST>>>(make_table(dst_peers, world), dst_off_bytes, src, nbytes, world);
  return CHECK_LAUNCH();
}

// out = sum over ranks of src (+ residual), n bf16 elements (multiple of 8, n <= slot_elems); see peer_allreduce_oneshot_kernel.
extern "C" int oa_peer_allreduce_oneshot(const void* const* slots_peers, const void* const* counters_peers, const void* src,
                                         const void* residual, void* out, void* sync2, long long n, long long slot_elems, int world,
                                         int rank, int max_ctas, int* status, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return OA_ERR_ARG;
  if (n <= 0 || (n & 7) || n > slot_elems || (slot_elems & 7)) return OA_ERR_ALIGN;
  const long long ctas = (n / 8 + 255) / 256;
  if (ctas > max_ctas) return OA_ERR_ARG;
  ArParams p;
  p.slots = make_table(slots_peers, world);
  p.counters = make_table(counters_peers, world);
  p.src = (const __nv_bfloat16*)src; p.residual = (const __nv_bfloat16*)residual; p.out = (__nv_bfloat16*)out;
  p.sync = (unsigned long long*)sync2; p.status = status; p.n = n; p.slot_elems = slot_elems; p.world = world; p.rank = rank;
  peer_allreduce_oneshot_kernel<<<(int)ctas, 256, 0, ST>>>(p);
  return CHECK_LAUNCH();
}
