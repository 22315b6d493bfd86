// Host emulation of the device-side synchronisation protocols, built with -fsanitize=thread.
//
// Every "GPU" is a host thread that runs its kernels in stream order; every CTA of a kernel is a thread of its own that is
// joined at the end of the kernel (a kernel boundary orders everything before it on that GPU, and nothing on another GPU).
// Peer-visible memory is plain (non-atomic) host memory, so the race detector sees each load and store that the device
// code performs on staging buffers, gradient and parameter arenas; flags are std::atomic words accessed with exactly the
// orderings of the device code:
//     st.release.sys / red.release.sys.add (after __threadfence_system)  ->  store / fetch_add(memory_order_release)
//     ld.acquire.sys in a bounded polling loop                           ->  load(memory_order_acquire) under a time limit
// Random pauses between the steps of every thread vary the interleaving from run to run (seeded: a failure names its seed).
//
// Protocols covered (kernels/comm.cu, kernels/gemm_tcgen05.cu, parallel/dp.py, parallel/tp.py):
//   dp        bucketed fused data-parallel step: gradients-ready channel, reduce + update + parameter push in one kernel,
//             parameters-complete channel, optional clip-norm scalar exchange on a third channel
//   tp        tensor-parallel call sites: mode 1 (communication CTAs push row slabs, compute CTAs wait per row block,
//             counters grow by `slabs` per call) and mode 2 (partial tiles stored into the owner's slots, four counted
//             releases per tile, the owner's reduce waits per row block), the per-site epoch word that advances when the
//             last CTA leaves, and the ready/ack round that separates two consecutive uses of one site
//   ep        expert-parallel dispatch / combine: three rounds per layer forward, two backward, per-layer row buffers, one
//             shared pair of gradient staging buffers with no round after a layer's last pull
//   timeout   a rank that never signals: the others' bounded waits run out, set the status word and return
// Negative controls (`dp-no-ack`, `tp-no-fence`) drop one ordering edge on purpose; the detector must report them, which
// shows that the harness can see the hazards the protocols are there to prevent.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <functional>
#include <memory>
#include <string>
#include <thread>
#include <vector>

namespace {

using u64 = unsigned long long;
using Flag = std::atomic<u64>;

constexpr int KERR_WAIT_PEER = 7;
std::chrono::milliseconds g_wait_limit{20000};
std::atomic<int> g_failures{0};

#define EXPECT(cond)                                                                         \
  do {                                                                                       \
    if (!(cond)) {                                                                           \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);                 \
      g_failures.fetch_add(1);                                                               \
    }                                                                                        \
  } while (0)

struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0x1234567ull) {}
  uint32_t next() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return (uint32_t)(s >> 16); }
};

// A pause of random length and kind: none, a yield, a short spin, a sleep of a few microseconds.
void jitter(Rng& rng) {
  const uint32_t r = rng.next();
  switch (r & 7) {
    case 0: case 1: case 2: return;
    case 3: case 4: std::this_thread::yield(); return;
    case 5: case 6: { volatile uint32_t x = 0; for (uint32_t i = 0; i < ((r >> 3) & 1023); ++i) x += i; return; }
    default: std::this_thread::sleep_for(std::chrono::microseconds((r >> 3) & 63)); return;
  }
}

// ld.acquire.sys polling loop with the wall-clock bound of wait_flags() / wait_ge_sys().
bool wait_ge(const Flag& f, u64 target) {
  uint32_t it = 0;
  std::chrono::steady_clock::time_point t0;
  bool timed = false;
  while (f.load(std::memory_order_acquire) < target) {
    if ((++it & 0x3f) == 0) {
      const auto now = std::chrono::steady_clock::now();
      if (!timed) { t0 = now; timed = true; }
      else if (now - t0 > g_wait_limit) return false;
      std::this_thread::yield();
    }
  }
  return true;
}

bool wait_flags(const Flag* flags, int world, u64 target) {
  for (int r = 0; r < world; ++r)
    if (!wait_ge(flags[r], target)) return false;
  return true;
}

// One kernel launch: `ctas` threads run body(cta), all joined before the next kernel of this GPU starts.
void launch(int ctas, const std::function<void(int)>& body) {
  std::vector<std::thread> ts;
  for (int c = 0; c < ctas; ++c) ts.emplace_back(body, c);
  for (auto& t : ts) t.join();
}

// A ready/ack channel (OaPeerChannel): flags[receiver][sender], one epoch word per rank.
struct Channel {
  int world;
  std::unique_ptr<Flag[]> flags;        // [world][world]
  std::vector<u64> epoch;               // device-resident, touched only by its own rank's kernels
  explicit Channel(int w) : world(w), flags(new Flag[w * w]), epoch(w, 0) {
    for (int i = 0; i < w * w; ++i) flags[i].store(0, std::memory_order_relaxed);
  }
  void signal(int rank) {               // peer_signal_kernel
    const u64 e = ++epoch[rank];
    for (int p = 0; p < world; ++p) flags[p * world + rank].store(e, std::memory_order_release);
  }
  bool wait(int rank, int* status) {    // peer_wait_kernel
    if (!wait_flags(&flags[rank * world], world, epoch[rank])) { *status = KERR_WAIT_PEER; return false; }
    return true;
  }
};

float grad_value(int rank, int step, long long i, float param) {
  return float((rank * 31 + step * 17 + i * 7) % 23 - 11) * 0.125f + param * 0.0625f;
}

}  // namespace

// ------------------------------------------------------------------------------------------------ data-parallel step
namespace {

struct DpWorld {
  int W, buckets, ctas, steps;
  long long n;                       // elements of the arena; bucket b covers [b * n / buckets, (b + 1) * n / buckets)
  bool clip, param_ack;
  std::vector<std::vector<float>> grads, params, master, slots;
  Channel ch_grads, ch_params, ch_norm;
  std::vector<int> status;
  DpWorld(int W_, int buckets_, int ctas_, int steps_, long long n_, bool clip_, bool ack)
      : W(W_), buckets(buckets_), ctas(ctas_), steps(steps_), n(n_), clip(clip_), param_ack(ack), grads(W_, std::vector<float>(n_, 0.f)),
        params(W_, std::vector<float>(n_)), master(W_, std::vector<float>(n_ / W_)), slots(W_, std::vector<float>(W_, 0.f)),
        ch_grads(W_), ch_params(W_), ch_norm(W_), status(W_, 0) {
    for (int r = 0; r < W; ++r)
      for (long long i = 0; i < n; ++i) params[r][i] = float(i % 13) * 0.5f - 3.f;
    for (int r = 0; r < W; ++r)
      for (int b = 0; b < buckets; ++b)
        for (long long k = 0; k < shard_n(); ++k) master[r][b * shard_n() + k] = params[r][shard_lo(b, r) + k];
  }
  long long bucket_n() const { return n / buckets; }
  long long shard_n() const { return bucket_n() / W; }
  long long shard_lo(int b, int r) const { return b * bucket_n() + r * shard_n(); }
};

constexpr float kLr = 0.03125f, kMaxNorm = 40.f;

// Sum of every rank's gradient at element e in the order of the owner's kernel (its own copy first).
float peer_sum(const DpWorld& w, int owner, long long e) {
  float g = 0.f;
  for (int rr = 0; rr < w.W; ++rr) g += w.grads[(owner + rr) % w.W][e];
  return g;
}

void dp_rank(DpWorld& w, int r, uint64_t seed) {
  Rng rng(seed * 977 + r);
  int& status = w.status[r];
  for (int step = 0; step < w.steps && !status; ++step) {
    jitter(rng);
    // backward pass of this rank: reads its parameter arena, writes its gradient arena
    for (long long i = 0; i < w.n; ++i) w.grads[r][i] = grad_value(r, step, i, w.params[r][i]);
    float coef = 1.f;
    if (w.clip) {
      w.ch_grads.signal(r);
      if (!w.ch_grads.wait(r, &status)) break;
      float partial = 0.f;                                       // dp_shard_sumsq_kernel over this rank's shards
      for (int b = 0; b < w.buckets; ++b)
        for (long long k = 0; k < w.shard_n(); ++k) { const float s = peer_sum(w, r, w.shard_lo(b, r) + k); partial += s * s; }
      jitter(rng);
      for (int p = 0; p < w.W; ++p) w.slots[p][r] = partial;      // dp_sumsq_publish_kernel (plain peer stores)
      w.ch_norm.signal(r);
      if (!w.ch_norm.wait(r, &status)) break;
      float total = 0.f;                                         // dp_clip_finalize_kernel: rank order, same bits everywhere
      for (int q = 0; q < w.W; ++q) total += w.slots[r][q];
      const float norm = std::sqrt(total);
      coef = norm > kMaxNorm ? kMaxNorm / norm : 1.f;
    }
    for (int b = 0; b < w.buckets && !status; ++b) {
      jitter(rng);
      w.ch_grads.signal(r);                                      // "my gradients of this bucket are final"
      const u64 target = w.ch_grads.epoch[r];
      std::atomic<int> bad{0};
      launch(w.ctas, [&, b, target](int cta) {                   // dp_reduce_adam_gather_kernel
        Rng local(seed * 131 + r * 17 + b * 5 + cta);
        jitter(local);
        if (!wait_flags(&w.ch_grads.flags[r * w.W], w.W, target)) { bad.store(1); return; }
        for (long long k = cta; k < w.shard_n(); k += w.ctas) {
          const long long e = w.shard_lo(b, r) + k;
          const float g = peer_sum(w, r, e) * coef;
          float& m = w.master[r][b * w.shard_n() + k];
          m -= kLr * g;
          for (int rr = 0; rr < w.W; ++rr) w.params[(r + rr) % w.W][e] = m;   // st_peer into every rank's parameter arena
          if ((k & 63) == 0) jitter(local);
        }
      });
      if (bad.load()) status = KERR_WAIT_PEER;
    }
    if (status) break;
    if (w.param_ack) {                                           // parameters of every rank are complete
      w.ch_params.signal(r);
      if (!w.ch_params.wait(r, &status)) break;
    }
  }
}

// The same arithmetic in lock step on one thread.
std::vector<float> dp_serial(int W, int buckets, int steps, long long n, bool clip) {
  DpWorld w(W, buckets, 1, steps, n, clip, true);
  for (int step = 0; step < steps; ++step) {
    for (int r = 0; r < W; ++r)
      for (long long i = 0; i < n; ++i) w.grads[r][i] = grad_value(r, step, i, w.params[r][i]);
    float coef = 1.f;
    if (clip) {
      float total = 0.f;
      for (int q = 0; q < W; ++q) {
        float partial = 0.f;
        for (int b = 0; b < buckets; ++b)
          for (long long k = 0; k < w.shard_n(); ++k) { const float s = peer_sum(w, q, w.shard_lo(b, q) + k); partial += s * s; }
        total += partial;
      }
      const float norm = std::sqrt(total);
      coef = norm > kMaxNorm ? kMaxNorm / norm : 1.f;
    }
    for (int b = 0; b < buckets; ++b)
      for (int r = 0; r < W; ++r)
        for (long long k = 0; k < w.shard_n(); ++k) {
          const long long e = w.shard_lo(b, r) + k;
          float& m = w.master[r][b * w.shard_n() + k];
          m -= kLr * peer_sum(w, r, e) * coef;
          for (int p = 0; p < W; ++p) w.params[p][e] = m;
        }
  }
  return w.params[0];
}

void run_dp(int W, int buckets, bool clip, bool ack, uint64_t seed) {
  const long long n = 8LL * W * buckets * 24;
  const int steps = 5;
  DpWorld w(W, buckets, 3, steps, n, clip, ack);
  std::vector<std::thread> ranks;
  for (int r = 0; r < W; ++r) ranks.emplace_back(dp_rank, std::ref(w), r, seed);
  for (auto& t : ranks) t.join();
  for (int r = 0; r < W; ++r) EXPECT(w.status[r] == 0);
  if (ack) {
    const std::vector<float> want = dp_serial(W, buckets, steps, n, clip);
    for (int r = 0; r < W; ++r) EXPECT(std::memcmp(w.params[r].data(), want.data(), n * sizeof(float)) == 0);
  }
}

// One rank never takes part: every wait of the others runs out, sets the status word and returns; nothing hangs.
void run_timeout(int W) {
  const auto saved = g_wait_limit;
  g_wait_limit = std::chrono::milliseconds(60);
  DpWorld w(W, 2, 2, 2, 8LL * W * 2 * 8, false, true);
  std::vector<std::thread> ranks;
  const auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r + 1 < W; ++r) ranks.emplace_back(dp_rank, std::ref(w), r, 1);       // rank W - 1 never starts
  for (auto& t : ranks) t.join();
  const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
  for (int r = 0; r + 1 < W; ++r) EXPECT(w.status[r] == KERR_WAIT_PEER);
  EXPECT(ms < 5000);
  g_wait_limit = saved;
}

}  // namespace

// ------------------------------------------------------------------------------------------- tensor-parallel call sites
namespace {

constexpr int BM = 4, BN = 4, SLAB = 4;     // rows per block (one per epilogue warp), columns per tile, columns per pushed slab

struct TpSite {
  int mode, W, blocks, slabs, n_tiles;      // blocks: row blocks per rank; mode 1: K = slabs * SLAB; mode 2: N = n_tiles * BN
  int M, Ms, K, N;
  std::vector<std::vector<float>> stage;    // mode 1: [M][K] gathered rows; mode 2: [W][Ms][N] partial slots
  std::vector<std::unique_ptr<Flag[]>> flags;
  std::vector<std::unique_ptr<Flag[]>> sync;   // per rank {epoch of this call site, CTAs finished}
  TpSite(int mode_, int W_, int blocks_, int cols) : mode(mode_), W(W_), blocks(blocks_), slabs(cols), n_tiles(cols) {
    Ms = blocks * BM; M = Ms * W; K = slabs * SLAB; N = n_tiles * BN;
    const int n_flags = mode == 1 ? M / BM : Ms / BM;
    for (int r = 0; r < W; ++r) {
      stage.emplace_back((size_t)M * (mode == 1 ? K : N), -1.f);
      flags.emplace_back(new Flag[n_flags]);
      for (int i = 0; i < n_flags; ++i) flags.back()[i].store(0, std::memory_order_relaxed);
      sync.emplace_back(new Flag[2]);
      sync.back()[0].store(0, std::memory_order_relaxed);
      sync.back()[1].store(0, std::memory_order_relaxed);
    }
  }
};

float x_value(int rank, u64 call, int row, int col) { return float((rank * 13 + (int)(call % 97) * 7 + row * 3 + col) % 29) - 14.f; }

// The call site's epoch advances once every CTA (each read it at its start) has finished.
void leave_site(TpSite& s, int r, u64 epoch, int n_ctas) {
  const u64 old = s.sync[r][1].fetch_add(1, std::memory_order_acq_rel);
  if (old == (u64)n_ctas - 1) {
    s.sync[r][1].store(0, std::memory_order_relaxed);
    s.sync[r][0].store(epoch, std::memory_order_release);
  }
}

// Mode 1: all-gather -> GEMM.  Returns false when a wait ran out.
bool tp_allgather_gemm(TpSite& s, int r, u64 call, uint64_t seed, std::atomic<int>& wrong) {
  const int W = s.W, blocks = s.blocks;
  float* mine = s.stage[r].data();
  for (int row = 0; row < s.Ms; ++row)                                       // the producer writes this rank's own rows in place
    for (int c = 0; c < s.K; ++c) mine[(size_t)(r * s.Ms + row) * s.K + c] = x_value(r, call, row, c);
  const int n_comm = 2, n_comp = 3, n_ctas = n_comm + n_comp;
  std::atomic<int> bad{0};
  launch(n_ctas, [&](int cta) {
    Rng rng(seed * 7919 + r * 101 + call * 13 + cta);
    const u64 epoch = s.sync[r][0].load(std::memory_order_acquire) + 1;
    if (epoch != call) wrong.fetch_add(1);
    jitter(rng);
    if (cta < n_comm) {
      const int per_peer = blocks * s.slabs;
      for (int item = cta; item < per_peer * (W - 1); item += n_comm) {
        const int j = item / per_peer, rem = item - j * per_peer;
        const int c = rem / s.slabs, sl = rem - c * s.slabs;
        const int peer = (r + 1 + j) % W;
        const float* src = mine + (size_t)(r * s.Ms + c * BM) * s.K + sl * SLAB;
        float* dst = s.stage[peer].data() + (size_t)(r * blocks + c) * BM * s.K + sl * SLAB;
        for (int row = 0; row < BM; ++row)
          for (int k = 0; k < SLAB; ++k) dst[(size_t)row * s.K + k] = src[(size_t)row * s.K + k];   // weak stores
        s.flags[peer][r * blocks + c].fetch_add(1, std::memory_order_release);                     // fence + red.release.sys.add
        jitter(rng);
      }
    } else {
      for (int rb = cta - n_comm; rb < W * blocks; rb += n_comp) {
        const int owner = rb / blocks;
        if (owner != r && !wait_ge(s.flags[r][rb], call * (u64)s.slabs)) { bad.store(1); break; }
        float sum = 0.f, want = 0.f;
        for (int row = 0; row < BM; ++row)
          for (int c = 0; c < s.K; ++c) {
            sum += mine[(size_t)(rb * BM + row) * s.K + c];
            want += x_value(owner, call, (rb - owner * blocks) * BM + row, c);
          }
        if (sum != want) wrong.fetch_add(1);
        jitter(rng);
      }
    }
    leave_site(s, r, epoch, n_ctas);
  });
  return bad.load() == 0;
}

// Mode 2: GEMM -> reduce-scatter.
bool tp_gemm_reduce_scatter(TpSite& s, int r, u64 call, uint64_t seed, std::atomic<int>& wrong) {
  const int W = s.W, blocks = s.blocks, n_ctas = 3;
  std::atomic<int> bad{0};
  launch(n_ctas, [&](int cta) {
    Rng rng(seed * 6007 + r * 211 + call * 17 + cta);
    const u64 epoch = s.sync[r][0].load(std::memory_order_acquire) + 1;
    if (epoch != call) wrong.fetch_add(1);
    // partial tiles into the owner's slot of this rank; the releases of up to three tiles are batched behind one fence
    std::vector<Flag*> pending[BM];
    auto flush = [&](int q) { for (Flag* f : pending[q]) f->fetch_add(1, std::memory_order_release); pending[q].clear(); };
    for (int t = cta; t < W * blocks * s.n_tiles; t += n_ctas) {
      const int mb = t / s.n_tiles, nt = t - mb * s.n_tiles;
      const int owner = mb / blocks, lb = mb - owner * blocks;
      float* dst = s.stage[owner].data() + ((size_t)r * s.Ms + lb * BM) * s.N + nt * BN;
      for (int q = 0; q < BM; ++q) {                                          // one epilogue warp per row
        for (int c = 0; c < BN; ++c) dst[(size_t)q * s.N + c] = x_value(r, call, mb * BM + q, nt * BN + c);
        pending[q].push_back(&s.flags[owner][lb]);
        if (pending[q].size() == 3) flush(q);
      }
      jitter(rng);
    }
    for (int q = 0; q < BM; ++q) flush(q);
    // the owner's reduce of its own rows over the W slots
    const u64 expect = call * (u64)(W * s.n_tiles * BM);
    const float* st = s.stage[r].data();
    for (int u = cta; u < blocks * s.n_tiles; u += n_ctas) {
      const int rb = u / s.n_tiles, sl = u - rb * s.n_tiles;
      if (!wait_ge(s.flags[r][rb], expect)) { bad.store(1); break; }
      for (int q = 0; q < BM; ++q)
        for (int c = 0; c < BN; ++c) {
          float sum = 0.f, want = 0.f;
          for (int w = 0; w < W; ++w) {
            sum += st[((size_t)w * s.Ms + rb * BM + q) * s.N + sl * BN + c];
            want += x_value(w, call, (r * blocks + rb) * BM + q, sl * BN + c);
          }
          if (sum != want) wrong.fetch_add(1);
        }
      jitter(rng);
    }
    leave_site(s, r, epoch, n_ctas);
  });
  return bad.load() == 0;
}

// `order` lists the site used by each call of a step; `fence` is the ready/ack round before a site that was also the one
// used last (OaTpArena.enter_site).
void run_tp(int W, const std::vector<int>& order, bool fence, uint64_t seed, bool check_values) {
  std::vector<std::unique_ptr<TpSite>> sites;
  sites.emplace_back(new TpSite(1, W, 2, 3));
  sites.emplace_back(new TpSite(2, W, 2, 3));
  sites.emplace_back(new TpSite(1, W, 1, 2));
  Channel ack(W);
  std::atomic<int> wrong{0};
  std::vector<int> status(W, 0);
  std::vector<std::thread> ranks;
  for (int r = 0; r < W; ++r)
    ranks.emplace_back([&, r] {
      Rng rng(seed * 31 + r);
      std::vector<u64> calls(sites.size(), 0);
      int last = -1;
      for (int step = 0; step < 6 && !status[r]; ++step)
        for (int id : order) {
          jitter(rng);
          if (id == last && fence) {
            ack.signal(r);
            if (!ack.wait(r, &status[r])) break;
          }
          last = id;
          TpSite& s = *sites[id];
          const u64 call = ++calls[id];
          const bool ok = s.mode == 1 ? tp_allgather_gemm(s, r, call, seed, wrong) : tp_gemm_reduce_scatter(s, r, call, seed, wrong);
          if (!ok) { status[r] = KERR_WAIT_PEER; break; }
        }
    });
  for (auto& t : ranks) t.join();
  for (int r = 0; r < W; ++r) EXPECT(status[r] == 0);
  if (check_values) EXPECT(wrong.load() == 0);
}

}  // namespace

// ------------------------------------------------------------------------------------------- expert-parallel dispatch
namespace {

// parallel/ep.py: three ready/ack rounds per layer forward (counts, rows landed, outputs ready), two backward (output
// gradients landed, token gradients ready).  Row buffers px / po are per layer; the gradient staging pair is shared by all
// layers and there is NO round after the last pull of a layer.
struct EpWorld {
  int W, layers, R;                                   // R rows from every source to every owner
  std::vector<std::vector<std::vector<float>>> px, po; // [layer][rank][W * R]
  std::vector<std::vector<float>> dpo, dpx, counts;    // [rank][W * R], [rank][W]
  std::vector<Channel> ch;                             // 5 per layer
  EpWorld(int W_, int layers_, int R_) : W(W_), layers(layers_), R(R_) {
    for (int l = 0; l < layers; ++l) {
      px.emplace_back(W, std::vector<float>(W * R, -1.f));
      po.emplace_back(W, std::vector<float>(W * R, -1.f));
      for (int c = 0; c < 5; ++c) ch.emplace_back(W);
    }
    dpo.assign(W, std::vector<float>(W * R, -1.f));
    dpx.assign(W, std::vector<float>(W * R, -1.f));
    counts.assign(W, std::vector<float>(W, 0.f));
  }
};

float ep_value(int rank, int step, int layer, int owner, int j) { return float((rank * 7 + step * 5 + layer * 3 + owner * 11 + j) % 31) - 15.f; }

void run_ep(int W, int layers, uint64_t seed) {
  EpWorld w(W, layers, 6);
  std::atomic<int> wrong{0};
  std::vector<int> status(W, 0);
  std::vector<std::thread> ranks;
  for (int r = 0; r < W; ++r)
    ranks.emplace_back([&, r] {
      Rng rng(seed * 53 + r);
      int& st = status[r];
      auto round = [&](int layer, int c) { Channel& ch = w.ch[layer * 5 + c]; ch.signal(r); return ch.wait(r, &st); };
      for (int step = 0; step < 5 && !st; ++step) {
        for (int l = 0; l < layers && !st; ++l) {                       // forward
          jitter(rng);
          for (int p = 0; p < W; ++p) w.counts[p][r] = float(w.R);        // counts into every peer's table row
          if (!round(l, 0)) break;
          for (int p = 0; p < W; ++p) if (w.counts[r][p] != float(w.R)) wrong.fetch_add(1);
          for (int o = 0; o < W; ++o)                                     // dispatch: rows into the owners' buffers
            for (int j = 0; j < w.R; ++j) w.px[l][o][r * w.R + j] = ep_value(r, step, l, o, j);
          jitter(rng);
          if (!round(l, 1)) break;
          for (int i = 0; i < W * w.R; ++i) w.po[l][r][i] = 2.f * w.px[l][r][i];   // this owner's experts
          jitter(rng);
          if (!round(l, 2)) break;
          for (int o = 0; o < W; ++o)                                     // combine: pull from the owners
            for (int j = 0; j < w.R; ++j)
              if (w.po[l][o][r * w.R + j] != 2.f * ep_value(r, step, l, o, j)) wrong.fetch_add(1);
        }
        for (int l = layers - 1; l >= 0 && !st; --l) {                  // backward
          jitter(rng);
          for (int o = 0; o < W; ++o)                                     // dgate: pulled dot products with the saved outputs
            for (int j = 0; j < w.R; ++j)
              if (w.po[l][o][r * w.R + j] != 2.f * ep_value(r, step, l, o, j)) wrong.fetch_add(1);
          for (int o = 0; o < W; ++o)
            for (int j = 0; j < w.R; ++j) w.dpo[o][r * w.R + j] = 3.f * ep_value(r, step, l, o, j);
          jitter(rng);
          if (!round(l, 3)) break;
          for (int i = 0; i < W * w.R; ++i) w.dpx[r][i] = w.dpo[r][i] + w.px[l][r][i];   // dX (and dW from the saved rows)
          jitter(rng);
          if (!round(l, 4)) break;
          for (int o = 0; o < W; ++o)
            for (int j = 0; j < w.R; ++j)
              if (w.dpx[o][r * w.R + j] != 4.f * ep_value(r, step, l, o, j)) wrong.fetch_add(1);
        }
      }
    });
  for (auto& t : ranks) t.join();
  for (int r = 0; r < W; ++r) EXPECT(status[r] == 0);
  EXPECT(wrong.load() == 0);
}

}  // namespace

int main(int argc, char** argv) {
  const std::string what = argc > 1 ? argv[1] : "all";
  const uint64_t seed = argc > 2 ? std::strtoull(argv[2], nullptr, 10) : 1;
  std::printf("protocol emulation: %s, seed %llu\n", what.c_str(), (unsigned long long)seed);
  if (what == "dp" || what == "all")
    for (int W = 2; W <= 4; ++W) {
      run_dp(W, 1, false, true, seed);
      run_dp(W, 3, false, true, seed + 1);
      run_dp(W, 2, true, true, seed + 2);
    }
  if (what == "tp" || what == "all")
    for (int W = 2; W <= 4; ++W) {
      run_tp(W, {0, 1}, true, seed, true);            // all-gather site, reduce-scatter site, alternating
      run_tp(W, {0, 1, 2, 1}, true, seed + 1, true);
      run_tp(W, {0, 0, 1, 1}, true, seed + 2, true);  // the same site twice in a row: separated by the ready/ack round
      run_tp(W, {2}, true, seed + 3, true);
    }
  if (what == "ep" || what == "all")
    for (int W = 2; W <= 4; ++W) {
      run_ep(W, 1, seed);                               // one layer: the shared gradient buffers are reused by the very next use
      run_ep(W, 3, seed + 1);
    }
  if (what == "timeout" || what == "all") run_timeout(3);
  // negative controls: the detector must report these
  if (what == "dp-no-ack") run_dp(3, 2, false, false, seed);
  if (what == "tp-no-fence") run_tp(3, {0, 0}, false, seed, false);
  const int failed = g_failures.load();
  std::printf(failed ? "FAILED (%d)\n" : "ok\n", failed);
  return failed ? 1 : 0;
}
