// Host-side primitives of the core layer: vector math on fp32 spans, streaming copies, CPU topology,
// spinlock / reader-writer lock, a bounded channel and a pinned worker pool with waitable tasks.
//
// Parity: Source/Public/Oa/Core/Simd.h:17-29 (OaSimd), Core/Memory.h:30-156 (OaMemcpyNT, OaMemEqual,
// OaAlignedAlloc), Core/Thread.h:26-470 (OaCpuTopology, OaSpinlock, OaRwLock, OaChannel, OaTask,
// OaThreadPool).  The reference routes vector math through Highway; here the loops are written on GCC
// vector types and compiled twice (baseline and AVX2+FMA) with the choice made once per process.  The
// pool's job here is feeding the GPU: sharded copies into pinned upload buffers and dataset decoding.
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <shared_mutex>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include <immintrin.h>
#include <pthread.h>
#include <sched.h>
#include <unistd.h>

namespace {

typedef float v8f __attribute__((vector_size(32), aligned(4)));

#define OA_SIMD_BODY(NAME, EXPR_VEC, EXPR_SCALAR)                                        \
  static void NAME##_base(float* a, const float* b, float s, int64_t n) {                \
    int64_t i = 0;                                                                       \
    for (; i + 8 <= n; i += 8) {                                                         \
      v8f x = *reinterpret_cast<const v8f*>(a + i);                                      \
      v8f y = b ? *reinterpret_cast<const v8f*>(b + i) : x;                              \
      (void)y; (void)s;                                                                  \
      *reinterpret_cast<v8f*>(a + i) = (EXPR_VEC);                                       \
    }                                                                                    \
    for (; i < n; ++i) { float x = a[i]; float y = b ? b[i] : x; (void)y; a[i] = (EXPR_SCALAR); } \
  }                                                                                      \
  __attribute__((target("avx2,fma"))) static void NAME##_avx2(float* a, const float* b, float s, int64_t n) { \
    int64_t i = 0;                                                                       \
    for (; i + 8 <= n; i += 8) {                                                         \
      v8f x = *reinterpret_cast<const v8f*>(a + i);                                      \
      v8f y = b ? *reinterpret_cast<const v8f*>(b + i) : x;                              \
      (void)y; (void)s;                                                                  \
      *reinterpret_cast<v8f*>(a + i) = (EXPR_VEC);                                       \
    }                                                                                    \
    for (; i < n; ++i) { float x = a[i]; float y = b ? b[i] : x; (void)y; a[i] = (EXPR_SCALAR); } \
  }

OA_SIMD_BODY(k_scale, x * s, x * s)
OA_SIMD_BODY(k_add, x + y, x + y)
OA_SIMD_BODY(k_sub, x - y, x - y)
OA_SIMD_BODY(k_mul, x * y, x * y)
OA_SIMD_BODY(k_div, x / y, x / y)
OA_SIMD_BODY(k_neg, -x, -x)

static float dot_base(const float* a, const float* b, int64_t n) {
  v8f acc0 = {0, 0, 0, 0, 0, 0, 0, 0}, acc1 = acc0;
  int64_t i = 0;
  for (; i + 16 <= n; i += 16) {
    acc0 += *reinterpret_cast<const v8f*>(a + i) * *reinterpret_cast<const v8f*>(b + i);
    acc1 += *reinterpret_cast<const v8f*>(a + i + 8) * *reinterpret_cast<const v8f*>(b + i + 8);
  }
  acc0 += acc1;
  float s = 0.f;
  for (int k = 0; k < 8; ++k) s += acc0[k];
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}
__attribute__((target("avx2,fma"))) static float dot_avx2(const float* a, const float* b, int64_t n) {
  v8f acc0 = {0, 0, 0, 0, 0, 0, 0, 0}, acc1 = acc0;
  int64_t i = 0;
  for (; i + 16 <= n; i += 16) {
    acc0 += *reinterpret_cast<const v8f*>(a + i) * *reinterpret_cast<const v8f*>(b + i);
    acc1 += *reinterpret_cast<const v8f*>(a + i + 8) * *reinterpret_cast<const v8f*>(b + i + 8);
  }
  acc0 += acc1;
  float s = 0.f;
  for (int k = 0; k < 8; ++k) s += acc0[k];
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}

static bool has_avx2() {
  static const bool v = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  return v;
}

// Streaming copy: 32-byte non-temporal stores once the destination is aligned, so that a large staging copy
// does not evict the working set from the caches.
__attribute__((target("avx2"))) static void copy_nt_avx2(uint8_t* d, const uint8_t* s, size_t n) {
  size_t head = (32 - (reinterpret_cast<uintptr_t>(d) & 31)) & 31;
  if (head > n) head = n;
  std::memcpy(d, s, head);
  d += head; s += head; n -= head;
  size_t i = 0;
  for (; i + 32 <= n; i += 32)
    _mm256_stream_si256(reinterpret_cast<__m256i*>(d + i), _mm256_loadu_si256(reinterpret_cast<const __m256i*>(s + i)));
  _mm_sfence();
  std::memcpy(d + i, s + i, n - i);
}

}  // namespace

extern "C" {

int oa_simd_level() { return has_avx2() ? 2 : 1; }
float oa_simd_dot_f32(const float* a, const float* b, int64_t n) { return has_avx2() ? dot_avx2(a, b, n) : dot_base(a, b, n); }
#define OA_SIMD_EXPORT(NAME, KERNEL, HAS_B, HAS_S)                                                   \
  void NAME(float* a, const float* b, float s, int64_t n) {                                          \
    if (has_avx2()) KERNEL##_avx2(a, HAS_B ? b : nullptr, s, n); else KERNEL##_base(a, HAS_B ? b : nullptr, s, n); \
  }
OA_SIMD_EXPORT(oa_simd_scale_f32, k_scale, 0, 1)
OA_SIMD_EXPORT(oa_simd_add_f32, k_add, 1, 0)
OA_SIMD_EXPORT(oa_simd_sub_f32, k_sub, 1, 0)
OA_SIMD_EXPORT(oa_simd_mul_f32, k_mul, 1, 0)
OA_SIMD_EXPORT(oa_simd_div_f32, k_div, 1, 0)
OA_SIMD_EXPORT(oa_simd_neg_f32, k_neg, 0, 0)

void* oa_memcpy_nt(void* dst, const void* src, size_t n) {
  if (n >= (256u << 10) && has_avx2()) copy_nt_avx2(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), n);
  else std::memcpy(dst, src, n);
  return dst;
}
int oa_mem_equal(const void* a, const void* b, size_t n) { return std::memcmp(a, b, n) == 0; }
void* oa_aligned_alloc(size_t size, size_t alignment) {
  void* p = nullptr;
  if (alignment < sizeof(void*)) alignment = sizeof(void*);
  return posix_memalign(&p, alignment, size ? size : alignment) == 0 ? p : nullptr;
}
void oa_aligned_free(void* p) { std::free(p); }

}  // extern "C"

// ------------------------------------------------------------------------------------------ CPU topology
namespace {

struct CoreInfo { int id, package, numa, max_khz, core_id; };
struct Topology {
  std::vector<CoreInfo> cores;
  int physical = 0, logical = 0, numa_nodes = 1, packages = 1;
};

static bool read_int(const std::string& path, int* out) {
  std::ifstream f(path);
  long v;
  if (!(f >> v)) return false;
  *out = (int)v;
  return true;
}

// "0-3,8,10-11" -> ids
static std::vector<int> parse_cpulist(const std::string& s) {
  std::vector<int> out;
  std::stringstream ss(s);
  std::string tok;
  while (std::getline(ss, tok, ',')) {
    if (tok.empty()) continue;
    size_t dash = tok.find('-');
    int a = std::atoi(tok.substr(0, dash).c_str());
    int b = dash == std::string::npos ? a : std::atoi(tok.substr(dash + 1).c_str());
    for (int i = a; i <= b; ++i) out.push_back(i);
  }
  return out;
}

static Topology detect_topology() {
  Topology t;
  cpu_set_t set;
  CPU_ZERO(&set);
  std::vector<int> allowed;
  if (sched_getaffinity(0, sizeof(set), &set) == 0)
    for (int i = 0; i < CPU_SETSIZE; ++i) if (CPU_ISSET(i, &set)) allowed.push_back(i);
  if (allowed.empty()) { long n = sysconf(_SC_NPROCESSORS_ONLN); for (int i = 0; i < (n > 0 ? n : 1); ++i) allowed.push_back(i); }
  std::map<int, int> numa_of;
  for (int node = 0; node < 64; ++node) {
    std::ifstream f("/sys/devices/system/node/node" + std::to_string(node) + "/cpulist");
    std::string line;
    if (!std::getline(f, line)) continue;
    for (int c : parse_cpulist(line)) numa_of[c] = node;
    t.numa_nodes = node + 1;
  }
  std::set<std::pair<int, int>> phys;
  std::set<int> pkgs;
  for (int c : allowed) {
    CoreInfo ci{c, 0, 0, 0, c};
    std::string base = "/sys/devices/system/cpu/cpu" + std::to_string(c);
    read_int(base + "/topology/physical_package_id", &ci.package);
    read_int(base + "/topology/core_id", &ci.core_id);
    read_int(base + "/cpufreq/cpuinfo_max_freq", &ci.max_khz);
    auto it = numa_of.find(c);
    ci.numa = it == numa_of.end() ? 0 : it->second;
    phys.insert({ci.package, ci.core_id});
    pkgs.insert(ci.package);
    t.cores.push_back(ci);
  }
  t.logical = (int)t.cores.size();
  t.physical = (int)phys.size();
  t.packages = pkgs.empty() ? 1 : (int)pkgs.size();
  return t;
}

// ------------------------------------------------------------------------------------------ locks
struct Spinlock {
  std::atomic<bool> held{false};
  void lock() {
    for (;;) {
      if (!held.exchange(true, std::memory_order_acquire)) return;
      while (held.load(std::memory_order_relaxed)) __builtin_ia32_pause();
    }
  }
  bool try_lock() { return !held.load(std::memory_order_relaxed) && !held.exchange(true, std::memory_order_acquire); }
  void unlock() { held.store(false, std::memory_order_release); }
};

// Bounded multi-producer multi-consumer queue of 64-bit values with close semantics: Send blocks while full and
// fails once closed; Recv drains what is left after a close and then fails.
struct Channel {
  std::mutex m;
  std::condition_variable not_full, not_empty;
  std::deque<uint64_t> q;
  size_t cap;
  bool closed = false;
  explicit Channel(size_t c) : cap(c ? c : 1) {}
};

struct Task {
  std::mutex m;
  std::condition_variable cv;
  bool done = false;
  int status = 0;
};

typedef int (*JobFn)(void*);

struct Pool {
  std::mutex m;
  std::condition_variable cv;
  std::deque<std::function<void()>> jobs;
  std::vector<std::thread> workers;
  std::map<uint64_t, std::shared_ptr<Task>> tasks;
  uint64_t next_task = 1;
  bool stopping = false;
  std::atomic<uint64_t> executed{0};
};

static void pool_worker(Pool* p, int core) {
  if (core >= 0) {
    cpu_set_t set;
    CPU_ZERO(&set);
    CPU_SET(core, &set);
    pthread_setaffinity_np(pthread_self(), sizeof(set), &set);   // best effort
  }
  for (;;) {
    std::function<void()> job;
    {
      std::unique_lock<std::mutex> lk(p->m);
      p->cv.wait(lk, [&] { return p->stopping || !p->jobs.empty(); });
      if (p->jobs.empty()) return;            // stopping and drained
      job = std::move(p->jobs.front());
      p->jobs.pop_front();
    }
    job();
    p->executed.fetch_add(1, std::memory_order_relaxed);
  }
}

static uint64_t pool_submit(Pool* p, std::function<int()> fn) {
  auto task = std::make_shared<Task>();
  uint64_t id;
  {
    std::lock_guard<std::mutex> lk(p->m);
    if (p->stopping) return 0;
    id = p->next_task++;
    p->tasks[id] = task;
    p->jobs.emplace_back([task, fn] {
      int st = fn();
      { std::lock_guard<std::mutex> g(task->m); task->status = st; task->done = true; }
      task->cv.notify_all();
    });
  }
  p->cv.notify_one();
  return id;
}

static int pool_wait(Pool* p, uint64_t id) {
  std::shared_ptr<Task> task;
  {
    std::lock_guard<std::mutex> lk(p->m);
    auto it = p->tasks.find(id);
    if (it == p->tasks.end()) return -1;
    task = it->second;
  }
  int st;
  {
    std::unique_lock<std::mutex> lk(task->m);
    task->cv.wait(lk, [&] { return task->done; });
    st = task->status;
  }
  std::lock_guard<std::mutex> lk(p->m);
  p->tasks.erase(id);
  return st;
}

}  // namespace

extern "C" {

void* oa_cpu_topology_detect() { return new Topology(detect_topology()); }
void oa_cpu_topology_destroy(void* h) { delete static_cast<Topology*>(h); }
// what: 0 logical, 1 physical, 2 NUMA nodes, 3 packages
int oa_cpu_topology_count(void* h, int what) {
  auto* t = static_cast<Topology*>(h);
  return what == 0 ? t->logical : what == 1 ? t->physical : what == 2 ? t->numa_nodes : t->packages;
}
// out = {id, package, numa, max_khz, core_id}
int oa_cpu_topology_core(void* h, int i, int* out) {
  auto* t = static_cast<Topology*>(h);
  if (i < 0 || i >= (int)t->cores.size()) return -1;
  const CoreInfo& c = t->cores[i];
  out[0] = c.id; out[1] = c.package; out[2] = c.numa; out[3] = c.max_khz; out[4] = c.core_id;
  return 0;
}

// `threads` threads each add 1 to a plain counter `iters` times under the spinlock; returns the counter.
uint64_t oa_spinlock_stress(int threads, int iters) {
  Spinlock lock;
  uint64_t counter = 0;
  std::vector<std::thread> ts;
  for (int t = 0; t < threads; ++t)
    ts.emplace_back([&] { for (int i = 0; i < iters; ++i) { lock.lock(); ++counter; lock.unlock(); } });
  for (auto& t : ts) t.join();
  return counter;
}

// Readers check that the two halves of a pair written under the writer lock always agree; returns torn reads.
uint64_t oa_rwlock_stress(int readers, int writers, int iters) {
  std::shared_mutex rw;
  uint64_t a = 0, b = 0;
  std::atomic<uint64_t> torn{0};
  std::vector<std::thread> ts;
  for (int w = 0; w < writers; ++w)
    ts.emplace_back([&] { for (int i = 0; i < iters; ++i) { std::unique_lock<std::shared_mutex> g(rw); ++a; ++b; } });
  for (int r = 0; r < readers; ++r)
    ts.emplace_back([&] { for (int i = 0; i < iters; ++i) { std::shared_lock<std::shared_mutex> g(rw); if (a != b) torn.fetch_add(1); } });
  for (auto& t : ts) t.join();
  return torn.load() + (a == (uint64_t)writers * iters ? 0 : 1);
}

void* oa_channel_create(uint64_t capacity) { return new Channel(capacity); }
void oa_channel_destroy(void* h) { delete static_cast<Channel*>(h); }
int oa_channel_send(void* h, uint64_t v, int blocking) {
  auto* c = static_cast<Channel*>(h);
  std::unique_lock<std::mutex> lk(c->m);
  if (blocking) c->not_full.wait(lk, [&] { return c->closed || c->q.size() < c->cap; });
  if (c->closed || c->q.size() >= c->cap) return 0;
  c->q.push_back(v);
  lk.unlock();
  c->not_empty.notify_one();
  return 1;
}
int oa_channel_recv(void* h, uint64_t* out, int blocking) {
  auto* c = static_cast<Channel*>(h);
  std::unique_lock<std::mutex> lk(c->m);
  if (blocking) c->not_empty.wait(lk, [&] { return c->closed || !c->q.empty(); });
  if (c->q.empty()) return 0;
  *out = c->q.front();
  c->q.pop_front();
  lk.unlock();
  c->not_full.notify_one();
  return 1;
}
void oa_channel_close(void* h) {
  auto* c = static_cast<Channel*>(h);
  { std::lock_guard<std::mutex> lk(c->m); c->closed = true; }
  c->not_full.notify_all();
  c->not_empty.notify_all();
}
uint64_t oa_channel_size(void* h) { auto* c = static_cast<Channel*>(h); std::lock_guard<std::mutex> lk(c->m); return c->q.size(); }

// core_ids may be null (no pinning); otherwise worker i is pinned to core_ids[i % n_ids].
void* oa_pool_create(int workers, const int* core_ids, int n_ids) {
  auto* p = new Pool();
  if (workers <= 0) { workers = (int)std::thread::hardware_concurrency(); if (workers <= 0) workers = 1; }
  for (int i = 0; i < workers; ++i) p->workers.emplace_back(pool_worker, p, (core_ids && n_ids > 0) ? core_ids[i % n_ids] : -1);
  return p;
}
int oa_pool_num_workers(void* h) { return (int)static_cast<Pool*>(h)->workers.size(); }
uint64_t oa_pool_executed(void* h) { return static_cast<Pool*>(h)->executed.load(); }
uint64_t oa_pool_submit(void* h, JobFn fn, void* arg) { return pool_submit(static_cast<Pool*>(h), [fn, arg] { return fn(arg); }); }
int oa_pool_wait(void* h, uint64_t task) { return pool_wait(static_cast<Pool*>(h), task); }
// Stops intake, drains queued jobs, joins every worker.
void oa_pool_shutdown(void* h) {
  auto* p = static_cast<Pool*>(h);
  { std::lock_guard<std::mutex> lk(p->m); p->stopping = true; }
  p->cv.notify_all();
  for (auto& t : p->workers) if (t.joinable()) t.join();
  p->workers.clear();
}
void oa_pool_destroy(void* h) { oa_pool_shutdown(h); delete static_cast<Pool*>(h); }

// Copies `bytes` from src to dst in `shards` contiguous pieces on the pool (streaming stores for large pieces) and
// waits for all of them: the host half of a batched upload into a pinned staging buffer.
int oa_pool_parallel_copy(void* h, void* dst, const void* src, uint64_t bytes, int shards) {
  auto* p = static_cast<Pool*>(h);
  if (shards <= 0) shards = (int)p->workers.size();
  if (shards <= 0) return -1;
  uint64_t per = ((bytes + shards - 1) / shards + 63) & ~uint64_t(63);
  std::vector<uint64_t> ids;
  for (uint64_t off = 0; off < bytes; off += per) {
    uint64_t n = bytes - off < per ? bytes - off : per;
    uint8_t* d = static_cast<uint8_t*>(dst) + off;
    const uint8_t* s = static_cast<const uint8_t*>(src) + off;
    uint64_t id = pool_submit(p, [d, s, n] { oa_memcpy_nt(d, s, n); return 0; });
    if (!id) return -1;
    ids.push_back(id);
  }
  int rc = 0;
  for (uint64_t id : ids) rc |= pool_wait(p, id);
  return rc;
}

// sum_i a[i]*b[i] split over the pool, partial sums added in shard order (deterministic for a fixed shard count).
double oa_pool_parallel_dot(void* h, const float* a, const float* b, int64_t n, int shards) {
  auto* p = static_cast<Pool*>(h);
  if (shards <= 0) shards = (int)p->workers.size();
  std::vector<double> part(shards, 0.0);
  std::vector<uint64_t> ids;
  int64_t per = (n + shards - 1) / shards;
  for (int s = 0; s < shards; ++s) {
    int64_t lo = s * per, hi = lo + per < n ? lo + per : n;
    if (lo >= hi) break;
    double* out = &part[s];
    ids.push_back(pool_submit(p, [=] { *out = oa_simd_dot_f32(a + lo, b + lo, hi - lo); return 0; }));
  }
  for (uint64_t id : ids) pool_wait(p, id);
  double total = 0.0;
  for (double v : part) total += v;
  return total;
}

}  // extern "C"
