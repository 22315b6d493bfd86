// Exercises the native runtime's C API (compute graph, GEMM plan cache, host pool / channel / locks, .oam files, the
// asynchronous reader, the allocation session) from one plain executable, so that the whole runtime can be built with
// -fsanitize=address,undefined (memory errors, leaks, undefined arithmetic) or -fsanitize=thread (data races in the pool,
// channel, reader and lock code) and run without Python in the process.  Every check prints its name; the program exits
// non-zero on the first failed expectation, and the sanitizers abort it on their own findings.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

extern "C" {
// graph.cpp
void* oa_graph_create();
void oa_graph_destroy(void*);
void oa_graph_clear(void*);
int oa_graph_add_node(void*, const char*, const uint64_t*, const uint64_t*, const uint32_t*, int, const void*, int, uint32_t);
int oa_graph_num_nodes(void*);
uint64_t oa_graph_hash(void*);
uint64_t oa_graph_node_hash(void*, int);
int oa_graph_num_barriers(void*);
int oa_graph_num_levels(void*);
int oa_graph_node_level(void*, int);
int oa_graph_node_deps(void*, int, int*, int);
int oa_graph_num_buffers(void*);
void oa_graph_buffer_at(void*, int, uint64_t*, uint64_t*, int*, int*, int*);
void oa_graph_memory(void*, uint64_t*, uint64_t*);
const char* oa_graph_node_kernel(void*, int);
// plan_cache.cpp
void* oa_plan_cache_create();
void oa_plan_cache_destroy(void*);
int oa_plan_cache_lookup(void*, int, int, int, int, int, int, int, int*, int*);
void oa_plan_cache_record(void*, int, int, int, int, int, int, int, int, int, float);
int oa_plan_cache_size(void*);
void oa_plan_cache_stats(void*, uint64_t*, uint64_t*);
int oa_plan_cache_timing(void*, int, int, int, int, int, int, int, float*, float*, int*);
int oa_plan_cache_save(void*, const char*);
int oa_plan_cache_load(void*, const char*);
// host.cpp
float oa_simd_dot_f32(const float*, const float*, int64_t);
void* oa_memcpy_nt(void*, const void*, size_t);
int oa_mem_equal(const void*, const void*, size_t);
void* oa_aligned_alloc(size_t, size_t);
void oa_aligned_free(void*);
void* oa_cpu_topology_detect();
void oa_cpu_topology_destroy(void*);
int oa_cpu_topology_count(void*, int);
uint64_t oa_spinlock_stress(int, int);
uint64_t oa_rwlock_stress(int, int, int);
void* oa_channel_create(uint64_t);
void oa_channel_destroy(void*);
int oa_channel_send(void*, uint64_t, int);
int oa_channel_recv(void*, uint64_t*, int);
void oa_channel_close(void*);
typedef int (*JobFn)(void*);
void* oa_pool_create(int, const int*, int);
int oa_pool_num_workers(void*);
uint64_t oa_pool_executed(void*);
uint64_t oa_pool_submit(void*, JobFn, void*);
int oa_pool_wait(void*, uint64_t);
void oa_pool_destroy(void*);
int oa_pool_parallel_copy(void*, void*, const void*, uint64_t, int);
double oa_pool_parallel_dot(void*, const float*, const float*, int64_t, int);
// oam.cpp
void* oam_create();
void oam_destroy(void*);
void* oam_load(const char*);
const char* oam_last_error();
uint64_t oam_hash(const uint8_t*, uint64_t);
int oam_save(void*, const char*);
void oam_set_config(void*, const char*, uint32_t, uint32_t, uint32_t, int, int, int, uint32_t, const uint8_t*, uint64_t);
void oam_get_config(void*, char*, uint32_t*, uint32_t*, uint32_t*, int*, uint32_t*);
void oam_add_tensor(void*, int, const char*, int, int, const uint64_t*, const void*, uint64_t);
uint32_t oam_num_tensors(void*, int);
const void* oam_tensor_at(void*, int, uint32_t, char*, int*, int*, uint64_t*, uint64_t*);
void oam_set_optimizer(void*, const char*, float, float, float, float, float, int64_t, const float*, uint64_t, const float*, uint64_t,
                       const float*, uint64_t);
void oam_get_optimizer(void*, char*, float*, int64_t*, uint64_t*, const float**, const float**, const float**);
void oam_set_progress(void*, int, int64_t, uint64_t, uint64_t, float, float, int, const char*);
void oam_get_progress(void*, int*, int64_t*, uint64_t*, uint64_t*, float*, float*, int*, char*);
int oam_has_optimizer(void*);
// reader.cpp
void* oa_reader_open(const char*, int, int);
void oa_reader_close(void*);
int64_t oa_reader_file_size(void*);
int oa_reader_submit(void*, void*, int64_t, int64_t);
int oa_reader_wait(void*, int);
// session.cpp
void* oa_session_create();
void oa_session_destroy(void*);
int oa_session_begin_frame(void*);
int oa_session_request(void*, uint64_t, int*, uint64_t*);
int oa_session_end_frame(void*);
int oa_session_trim(void*);
uint64_t oa_session_stat(void*, int);
}

#define EXPECT(cond)                                                              \
  do {                                                                            \
    if (!(cond)) {                                                                \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);      \
      std::exit(1);                                                               \
    }                                                                             \
  } while (0)

static std::string g_dir = "/tmp";

static void check_graph() {
  void* g = oa_graph_create();
  // a -> b -> c chain plus an independent node, then a write-after-read hazard on buffer 1
  const uint64_t ids0[] = {1, 2}, by0[] = {4096, 4096};
  const uint32_t ac0[] = {1, 2};
  const uint64_t ids1[] = {2, 3}, by1[] = {4096, 8192};
  const uint64_t ids2[] = {7, 8}, by2[] = {512, 512};
  const uint64_t ids3[] = {3, 1}, by3[] = {8192, 4096};
  const float push[2] = {1.5f, 2.5f};
  EXPECT(oa_graph_add_node(g, "Relu", ids0, by0, ac0, 2, push, sizeof(push), 0) == 0);
  EXPECT(oa_graph_add_node(g, "Scale", ids1, by1, ac0, 2, nullptr, 0, 0) == 1);
  EXPECT(oa_graph_add_node(g, "Copy", ids2, by2, ac0, 2, nullptr, 0, 1) == 2);
  EXPECT(oa_graph_add_node(g, "Add", ids3, by3, ac0, 2, nullptr, 0, 0) == 3);
  EXPECT(oa_graph_num_nodes(g) == 4);
  const uint64_t h = oa_graph_hash(g);
  EXPECT(h != 0 && oa_graph_node_hash(g, 0) != oa_graph_node_hash(g, 1));
  EXPECT(oa_graph_num_levels(g) >= 3);
  EXPECT(oa_graph_node_level(g, 0) == 0 && oa_graph_node_level(g, 2) == 0);
  EXPECT(oa_graph_node_level(g, 1) > oa_graph_node_level(g, 0));
  EXPECT(oa_graph_node_level(g, 3) > oa_graph_node_level(g, 1));
  int deps[8];
  EXPECT(oa_graph_node_deps(g, 3, deps, 8) >= 1);
  EXPECT(oa_graph_node_deps(g, 3, deps, 0) >= 0);   // a zero-capacity query must not write
  EXPECT(oa_graph_num_barriers(g) >= 0);
  const int nb = oa_graph_num_buffers(g);
  EXPECT(nb == 5);
  for (int k = 0; k < nb; ++k) {
    uint64_t id, bytes; int first, last, group;
    oa_graph_buffer_at(g, k, &id, &bytes, &first, &last, &group);
    EXPECT(first <= last && bytes > 0);
  }
  uint64_t naive = 0, aliased = 0;
  oa_graph_memory(g, &naive, &aliased);
  EXPECT(aliased <= naive && naive >= 4096 * 2 + 8192 + 1024);
  EXPECT(std::strcmp(oa_graph_node_kernel(g, 1), "Scale") == 0);
  // the hash is structural: same nodes in a new graph give the same value; one more node changes it
  void* g2 = oa_graph_create();
  oa_graph_add_node(g2, "Relu", ids0, by0, ac0, 2, push, sizeof(push), 0);
  oa_graph_add_node(g2, "Scale", ids1, by1, ac0, 2, nullptr, 0, 0);
  oa_graph_add_node(g2, "Copy", ids2, by2, ac0, 2, nullptr, 0, 1);
  oa_graph_add_node(g2, "Add", ids3, by3, ac0, 2, nullptr, 0, 0);
  EXPECT(oa_graph_hash(g2) == h);
  oa_graph_add_node(g2, "Add", ids3, by3, ac0, 2, nullptr, 0, 0);
  EXPECT(oa_graph_hash(g2) != h);
  oa_graph_clear(g2);
  EXPECT(oa_graph_num_nodes(g2) == 0 && oa_graph_num_levels(g2) == 0);
  // a wide graph: many nodes, push constants longer than the stored prefix
  std::vector<uint8_t> long_push(300, 7);
  for (int i = 0; i < 2000; ++i) {
    const uint64_t ids[] = {uint64_t(100 + i % 17), uint64_t(200 + i % 13), uint64_t(300 + i)};
    const uint64_t by[] = {64, 128, 256};
    const uint32_t ac[] = {1, 3, 2};
    oa_graph_add_node(g2, "Wide", ids, by, ac, 3, long_push.data(), (int)long_push.size(), uint32_t(i % 3));
  }
  EXPECT(oa_graph_num_levels(g2) > 1 && oa_graph_hash(g2) != 0);
  oa_graph_destroy(g2);
  oa_graph_destroy(g);
  std::puts("graph ok");
}

static void check_plan_cache() {
  void* c = oa_plan_cache_create();
  int bn = 0, sp = 0;
  EXPECT(oa_plan_cache_lookup(c, 8192, 4096, 1024, 0, 0, 0, 1, &bn, &sp) == 0);
  oa_plan_cache_record(c, 8192, 4096, 1024, 0, 0, 0, 1, 128, 1, 50.f);
  oa_plan_cache_record(c, 8192, 4096, 1024, 0, 0, 0, 1, 256, 1, 40.f);
  oa_plan_cache_record(c, 8192, 4096, 1024, 0, 0, 0, 1, 64, 2, 70.f);
  EXPECT(oa_plan_cache_lookup(c, 8192, 4096, 1024, 0, 0, 0, 1, &bn, &sp) == 1 && bn == 256 && sp == 1);
  // several threads record and look up different shapes at once
  std::vector<std::thread> ts;
  for (int t = 0; t < 4; ++t)
    ts.emplace_back([c, t] {
      for (int i = 0; i < 200; ++i) {
        oa_plan_cache_record(c, 128 * (i % 9 + 1), 256 * (t + 1), 512, i % 3, 0, 0, 1, 128, 1, float(10 + (i * 7 + t) % 31));
        int b, s;
        oa_plan_cache_lookup(c, 128 * (i % 9 + 1), 256 * (t + 1), 512, i % 3, 0, 0, 1, &b, &s);
      }
    });
  for (auto& t : ts) t.join();
  EXPECT(oa_plan_cache_size(c) > 1);
  uint64_t hits = 0, misses = 0;
  oa_plan_cache_stats(c, &hits, &misses);
  EXPECT(hits > 0 && misses > 0);
  float med = 0, p95 = 0; int n = 0;
  EXPECT(oa_plan_cache_timing(c, 8192, 4096, 1024, 0, 0, 0, 1, &med, &p95, &n) == 1 && n >= 1 && p95 >= med);
  const std::string path = g_dir + "/plans.bin";
  EXPECT(oa_plan_cache_save(c, path.c_str()) == 0);
  void* d = oa_plan_cache_create();
  EXPECT(oa_plan_cache_load(d, path.c_str()) == 0);
  EXPECT(oa_plan_cache_size(d) == oa_plan_cache_size(c));
  EXPECT(oa_plan_cache_lookup(d, 8192, 4096, 1024, 0, 0, 0, 1, &bn, &sp) == 1 && bn == 256);
  EXPECT(oa_plan_cache_load(d, (g_dir + "/no_such_plans.bin").c_str()) != 0);
  // a truncated file must be refused, not read past its end
  {
    FILE* f = std::fopen(path.c_str(), "rb");
    EXPECT(f != nullptr);
    std::vector<uint8_t> all(1 << 20);
    const size_t got = std::fread(all.data(), 1, all.size(), f);
    std::fclose(f);
    const std::string cut = g_dir + "/plans_cut.bin";
    f = std::fopen(cut.c_str(), "wb");
    std::fwrite(all.data(), 1, got > 9 ? got - 9 : got / 2, f);
    std::fclose(f);
    void* e = oa_plan_cache_create();
    (void)oa_plan_cache_load(e, cut.c_str());       // either outcome is fine; it must not touch memory out of bounds
    oa_plan_cache_destroy(e);
  }
  oa_plan_cache_destroy(d);
  oa_plan_cache_destroy(c);
  std::puts("plan cache ok");
}

static int job_add(void* arg) {
  static_cast<std::atomic<uint64_t>*>(arg)->fetch_add(1, std::memory_order_relaxed);
  return 0;
}

static void check_host() {
  // aligned allocation, streaming copy with every head/tail misalignment, dot product with a ragged tail
  uint8_t* a = static_cast<uint8_t*>(oa_aligned_alloc(1 << 16, 256));
  uint8_t* b = static_cast<uint8_t*>(oa_aligned_alloc(1 << 16, 256));
  EXPECT(a && b && (reinterpret_cast<uintptr_t>(a) & 255) == 0);
  for (int i = 0; i < (1 << 16); ++i) a[i] = uint8_t(i * 131 + 7);
  for (int off = 0; off < 70; off += 7)
    for (size_t n : {size_t(0), size_t(1), size_t(31), size_t(64), size_t(4097), size_t(60000)}) {
      std::memset(b, 0, 1 << 16);
      oa_memcpy_nt(b + off, a + (off * 3) % 61, n);
      EXPECT(oa_mem_equal(b + off, a + (off * 3) % 61, n));
      EXPECT(b[off + n] == 0);
    }
  std::vector<float> x(1003), y(1003);
  double want = 0;
  for (int i = 0; i < 1003; ++i) { x[i] = float(i % 7) - 3.f; y[i] = float(i % 5) * 0.5f; want += double(x[i]) * y[i]; }
  EXPECT(std::abs(oa_simd_dot_f32(x.data(), y.data(), 1003) - want) < 1e-2);
  EXPECT(oa_simd_dot_f32(x.data(), y.data(), 0) == 0.f);
  void* topo = oa_cpu_topology_detect();
  EXPECT(oa_cpu_topology_count(topo, 0) >= 1);
  oa_cpu_topology_destroy(topo);
  // locks
  EXPECT(oa_spinlock_stress(4, 20000) == 80000);
  EXPECT(oa_rwlock_stress(3, 2, 5000) == 0);
  // bounded channel: two producers, two consumers, close wakes the blocked side
  void* ch = oa_channel_create(8);
  std::atomic<uint64_t> sum{0}, got{0};
  std::vector<std::thread> ts;
  for (int p = 0; p < 2; ++p)
    ts.emplace_back([ch, p] { for (uint64_t i = 1; i <= 2000; ++i) EXPECT(oa_channel_send(ch, i + uint64_t(p) * 10000, 1) == 1); });
  for (int c = 0; c < 2; ++c)
    ts.emplace_back([&, ch] {
      uint64_t v;
      while (oa_channel_recv(ch, &v, 1)) { sum.fetch_add(v); got.fetch_add(1); }
    });
  ts[0].join(); ts[1].join();
  oa_channel_close(ch);
  ts[2].join(); ts[3].join();
  EXPECT(got.load() == 4000);
  EXPECT(sum.load() == 2 * (2000ull * 2001 / 2) + 2000ull * 10000);
  EXPECT(oa_channel_send(ch, 1, 0) == 0);
  oa_channel_destroy(ch);
  // worker pool: submit from several threads, wait for every task, sharded copy and dot
  void* pool = oa_pool_create(4, nullptr, 0);
  EXPECT(oa_pool_num_workers(pool) == 4);
  std::atomic<uint64_t> ran{0};
  std::vector<std::thread> subs;
  for (int t = 0; t < 3; ++t)
    subs.emplace_back([&, pool] {
      std::vector<uint64_t> ids;
      for (int i = 0; i < 300; ++i) ids.push_back(oa_pool_submit(pool, job_add, &ran));
      for (uint64_t id : ids) EXPECT(id != 0 && oa_pool_wait(pool, id) == 0);
    });
  for (auto& t : subs) t.join();
  EXPECT(ran.load() == 900 && oa_pool_executed(pool) >= 900);
  std::memset(b, 0, 1 << 16);
  EXPECT(oa_pool_parallel_copy(pool, b, a, 65531, 5) == 0 && oa_mem_equal(a, b, 65531) && b[65531] == 0);
  EXPECT(oa_pool_parallel_copy(pool, b, a, 0, 3) == 0);
  EXPECT(std::abs(oa_pool_parallel_dot(pool, x.data(), y.data(), 1003, 7) - want) < 1e-6);
  oa_pool_destroy(pool);
  oa_aligned_free(a);
  oa_aligned_free(b);
  std::puts("host ok");
}

static void check_oam() {
  void* m = oam_create();
  const uint8_t cfg[] = {1, 2, 3, 4, 5, 6, 7, 8, 9};
  oam_set_config(m, "an-architecture-name-longer-than-the-31-bytes-that-are-kept", 64, 2, 256, 2, 1, 2, 5, cfg, sizeof(cfg));
  std::vector<float> w0(64 * 32), w1(7), st(33);
  for (size_t i = 0; i < w0.size(); ++i) w0[i] = float(i) * 0.25f;
  for (size_t i = 0; i < w1.size(); ++i) w1[i] = -float(i);
  for (size_t i = 0; i < st.size(); ++i) st[i] = 1.f / float(i + 1);
  const uint64_t s0[] = {64, 32}, s1[] = {7}, s2[] = {3, 11};
  const std::string long_name(300, 'n');
  const uint64_t sz[] = {0};
  {
    void* wrong = oam_create();                       // 7 float32 elements declared, 5 supplied: refused at save
    oam_set_config(wrong, "x", 1, 1, 1, 0, 0, 0, 0, cfg, 0);
    oam_add_tensor(wrong, 0, "short", 0, 1, s1, w1.data(), 20);
    EXPECT(oam_save(wrong, (g_dir + "/wrong.oam").c_str()) != 0 && std::strstr(oam_last_error(), "short") != nullptr);
    oam_destroy(wrong);
  }
  oam_add_tensor(m, 0, "layers.0.weight", 0, 2, s0, w0.data(), w0.size() * 4);
  oam_add_tensor(m, 0, long_name.c_str(), 0, 1, s1, w1.data(), w1.size() * 4);
  oam_add_tensor(m, 0, "empty", 0, 1, sz, nullptr, 0);
  oam_add_tensor(m, 1, "layers.0.state", 0, 2, s2, st.data(), st.size() * 4);
  std::vector<float> am(100, 0.5f), av(100, 0.25f), mu(10, 2.f);
  oam_set_optimizer(m, "an-optimizer-name-beyond-15", 1e-3f, 0.9f, 0.95f, 1e-8f, 0.1f, 77, am.data(), am.size(), av.data(), av.size(),
                    mu.data(), mu.size());
  EXPECT(oam_save(m, (g_dir + "/refused.oam").c_str()) != 0 && std::strlen(oam_last_error()) > 0);   // unknown optimizer type
  oam_set_optimizer(m, "MuonAdamW", 1e-3f, 0.9f, 0.95f, 1e-8f, 0.1f, 77, am.data(), am.size(), av.data(), av.size(), mu.data(), mu.size());
  oam_set_progress(m, 2, 1234, 1u << 20, 99, 3e-4f, 1.5f, 1, "a-metric-name-that-is-longer-than-thirty-one-bytes");
  const std::string path = g_dir + "/model.oam";
  EXPECT(oam_save(m, path.c_str()) == 0);
  void* r = oam_load(path.c_str());
  EXPECT(r != nullptr);
  char arch[32]; uint32_t dm, nl, dv, flags; int dt[3];
  oam_get_config(r, arch, &dm, &nl, &dv, dt, &flags);
  EXPECT(dm == 64 && nl == 2 && dv == 256 && flags == 5 && arch[31] == 0 && std::strlen(arch) == 31);
  EXPECT(oam_num_tensors(r, 0) == 3 && oam_num_tensors(r, 1) == 1);
  char name[128]; int dtype, rank; uint64_t shape[8], bytes;
  const void* p = oam_tensor_at(r, 0, 0, name, &dtype, &rank, shape, &bytes);
  EXPECT(p && bytes == w0.size() * 4 && rank == 2 && shape[0] == 64 && std::memcmp(p, w0.data(), bytes) == 0);
  p = oam_tensor_at(r, 0, 1, name, &dtype, &rank, shape, &bytes);
  EXPECT(p && bytes == 28 && name[127] == 0 && std::memcmp(p, w1.data(), bytes) == 0);
  p = oam_tensor_at(r, 1, 0, name, &dtype, &rank, shape, &bytes);
  EXPECT(p && bytes == st.size() * 4 && std::memcmp(p, st.data(), bytes) == 0);
  EXPECT(oam_tensor_at(r, 0, 99, name, &dtype, &rank, shape, &bytes) == nullptr);
  EXPECT(oam_has_optimizer(r));
  char type16[16]; float hyper[5]; int64_t step; uint64_t counts[3]; const float *pm, *pv, *pmu;
  oam_get_optimizer(r, type16, hyper, &step, counts, &pm, &pv, &pmu);
  EXPECT(step == 77 && counts[0] == 100 && counts[1] == 100 && counts[2] == 10 && pm[99] == 0.5f && pmu[9] == 2.f && std::strcmp(type16, "MuonAdamW") == 0);
  int phase, lower; int64_t pstep; uint64_t seen, env; float lr, best; char metric[32];
  oam_get_progress(r, &phase, &pstep, &seen, &env, &lr, &best, &lower, metric);
  EXPECT(phase == 2 && pstep == 1234 && seen == (1u << 20) && env == 99 && lower == 1 && metric[31] == 0);
  oam_destroy(r);
  // damaged files: every truncation point and a flipped byte in each region must be refused with an error, never read
  // out of bounds
  std::vector<uint8_t> file;
  {
    FILE* f = std::fopen(path.c_str(), "rb");
    EXPECT(f != nullptr);
    std::fseek(f, 0, SEEK_END);
    file.resize((size_t)std::ftell(f));
    std::fseek(f, 0, SEEK_SET);
    EXPECT(std::fread(file.data(), 1, file.size(), f) == file.size());
    std::fclose(f);
  }
  const std::string bad = g_dir + "/model_bad.oam";
  auto write_bad = [&](const std::vector<uint8_t>& v) {
    FILE* f = std::fopen(bad.c_str(), "wb");
    EXPECT(f != nullptr);
    if (!v.empty()) std::fwrite(v.data(), 1, v.size(), f);
    std::fclose(f);
  };
  int refused = 0, tried = 0;
  for (size_t cut = 0; cut < file.size(); cut += (cut < 600 ? 13 : 997)) {
    write_bad(std::vector<uint8_t>(file.begin(), file.begin() + cut));
    void* h = oam_load(bad.c_str());
    ++tried;
    if (!h) { ++refused; EXPECT(std::strlen(oam_last_error()) > 0); }
    else oam_destroy(h);
  }
  EXPECT(refused == tried);
  for (size_t pos = 0; pos < file.size(); pos += (pos < 600 ? 5 : 389)) {
    std::vector<uint8_t> v = file;
    v[pos] ^= 0xA5;
    write_bad(v);
    void* h = oam_load(bad.c_str());      // a flip in padding may load; anything else must be refused; neither may fault
    if (h) oam_destroy(h);
  }
  EXPECT(oam_load((g_dir + "/no_such.oam").c_str()) == nullptr);
  EXPECT(oam_hash(cfg, sizeof(cfg)) != oam_hash(cfg, sizeof(cfg) - 1));
  EXPECT(oam_save(m, (g_dir + "/made_dir/x.oam").c_str()) == 0);          // missing parent folders are created
  EXPECT(oam_save(m, (path + "/under_a_file/x.oam").c_str()) != 0);       // a parent that is a regular file is an error
  oam_destroy(m);
  std::puts("oam ok");
}

static void check_reader() {
  const std::string path = g_dir + "/blob.bin";
  std::vector<uint8_t> data(3 << 20);
  for (size_t i = 0; i < data.size(); ++i) data[i] = uint8_t((i * 2654435761u) >> 13);
  {
    FILE* f = std::fopen(path.c_str(), "wb");
    EXPECT(f != nullptr);
    std::fwrite(data.data(), 1, data.size(), f);
    std::fclose(f);
  }
  EXPECT(oa_reader_open((g_dir + "/no_such_blob.bin").c_str(), 4, 2) == nullptr);
  void* r = oa_reader_open(path.c_str(), 8, 3);
  EXPECT(r && oa_reader_file_size(r) == (int64_t)data.size());
  std::vector<uint8_t> out(data.size(), 0);
  const int64_t piece = 200000;
  int in_flight = 0, total = 0;
  for (int64_t off = 0; off < (int64_t)data.size(); off += piece) {
    const int64_t n = std::min<int64_t>(piece, (int64_t)data.size() - off);
    int rc = oa_reader_submit(r, out.data() + off, off, n);
    if (rc == -2) {                                   // queue full: drain at least one, then retry
      const int done = oa_reader_wait(r, 1);
      EXPECT(done > 0);
      in_flight -= done; total += done;
      rc = oa_reader_submit(r, out.data() + off, off, n);
    }
    EXPECT(rc == 0);
    ++in_flight;
  }
  while (in_flight > 0) {
    const int done = oa_reader_wait(r, in_flight);
    EXPECT(done > 0);
    in_flight -= done; total += done;
  }
  EXPECT(total == 16 && out == data);
  EXPECT(oa_reader_submit(r, out.data(), (int64_t)data.size() - 10, 11) == -1);   // past the end
  EXPECT(oa_reader_submit(r, nullptr, 0, 1) == -1);
  EXPECT(oa_reader_wait(r, 1) == 0);                                               // nothing in flight: returns at once
  oa_reader_close(r);
  // closing with reads still queued must join cleanly
  r = oa_reader_open(path.c_str(), 8, 1);
  for (int i = 0; i < 6; ++i) EXPECT(oa_reader_submit(r, out.data() + i * piece, i * piece, piece) == 0);
  oa_reader_wait(r, 6);
  oa_reader_close(r);
  std::puts("reader ok");
}

static void check_session() {
  void* s = oa_session_create();
  EXPECT(oa_session_end_frame(s) == -1);
  int reused; uint64_t cap;
  for (int frame = 0; frame < 4; ++frame) {
    EXPECT(oa_session_begin_frame(s) == 0);
    EXPECT(oa_session_begin_frame(s) == -1);
    for (int i = 0; i < 50; ++i) {
      const int ord = oa_session_request(s, uint64_t(1000 + i * 37 + (frame == 2 && i == 7 ? 100000 : 0)), &reused, &cap);
      EXPECT(ord == i && cap >= 1000 && (cap & 511) == 0);
      EXPECT(frame == 0 ? reused == 0 : (frame == 2 && i == 7 ? reused == 0 : reused == 1));
    }
    const int stable = oa_session_end_frame(s);
    EXPECT(stable == (frame == 1 || frame == 3 ? 1 : 0));
  }
  EXPECT(oa_session_stat(s, 0) == 4 && oa_session_stat(s, 1) == 2 && oa_session_stat(s, 2) == 50 && oa_session_stat(s, 3) > 50000);
  oa_session_begin_frame(s);
  for (int i = 0; i < 10; ++i) oa_session_request(s, 64, &reused, &cap);
  oa_session_end_frame(s);
  EXPECT(oa_session_trim(s) == 40 && oa_session_stat(s, 2) == 10);
  EXPECT(oa_session_request(s, 64, &reused, &cap) == -1);
  oa_session_destroy(s);
  std::puts("session ok");
}

int main(int argc, char** argv) {
  if (argc > 1) g_dir = argv[1];
  check_graph();
  check_plan_cache();
  check_host();
  check_oam();
  check_reader();
  check_session();
  std::puts("all ok");
  return 0;
}
