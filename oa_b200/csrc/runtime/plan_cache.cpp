// GEMM plan cache and tuner bookkeeping (native).  The reference routes every GEMM through a registry of tile variants
// with a tuner that records median / p95 timings and persists the winners in var/gemm_route_cache.bin
// (Source/Public/Oa/Runtime/GemmRouteCache.h, Source/Private/Oa/Runtime/Gemm/Router.cpp:470-560, Tuner.h:44-74).
// Here there is ONE kernel family, so a "plan" is its launch configuration: N tile (128 / 256), split-K factor and,
// for the tensor-parallel modes, the role.  The cache maps (M, N, K, layout, epilogue, role, world) -> plan, keeps the
// timing samples a tuner feeds it, picks the plan with the best median, and persists to a small binary file
// (magic, version, count, records; FNV-1a checksum; written to a temporary and renamed).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace {

struct Key {
  int32_t M, N, K, layout, epilogue, role, world;
  bool operator<(const Key& o) const { return std::memcmp(this, &o, sizeof(Key)) < 0; }
};
struct Plan { int32_t bn, splits; float median_us, p95_us; int32_t samples; };
struct Candidate { Plan plan; std::vector<float> us; };

struct Cache {
  std::mutex mu;
  std::map<Key, Plan> best;
  std::map<Key, std::vector<Candidate>> trials;
  uint64_t hits = 0, misses = 0;
};

constexpr uint32_t kMagic = 0x43504147u;   // "GAPC"
constexpr uint32_t kVersion = 1;

uint64_t fnv(const void* d, size_t n) {
  uint64_t h = 0xCBF29CE484222325ull;
  const auto* p = static_cast<const uint8_t*>(d);
  for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 0x100000001B3ull; }
  return h;
}

struct Record { Key key; Plan plan; };

}  // namespace

extern "C" {

void* oa_plan_cache_create() { return new Cache(); }
void oa_plan_cache_destroy(void* c) { delete static_cast<Cache*>(c); }

// Returns 1 and fills bn / splits when a plan is known.
int oa_plan_cache_lookup(void* c, int M, int N, int K, int layout, int epilogue, int role, int world, int* bn, int* splits) {
  auto* C = static_cast<Cache*>(c);
  std::lock_guard<std::mutex> lock(C->mu);
  auto it = C->best.find(Key{M, N, K, layout, epilogue, role, world});
  if (it == C->best.end()) { ++C->misses; return 0; }
  ++C->hits;
  *bn = it->second.bn; *splits = it->second.splits;
  return 1;
}

// One timing sample (microseconds) of a candidate plan; the best plan of the key is re-elected by median.
void oa_plan_cache_record(void* c, int M, int N, int K, int layout, int epilogue, int role, int world, int bn, int splits, float us) {
  auto* C = static_cast<Cache*>(c);
  std::lock_guard<std::mutex> lock(C->mu);
  const Key k{M, N, K, layout, epilogue, role, world};
  auto& cands = C->trials[k];
  Candidate* cur = nullptr;
  for (auto& cd : cands) if (cd.plan.bn == bn && cd.plan.splits == splits) cur = &cd;
  if (!cur) { cands.push_back(Candidate{Plan{bn, splits, 0.f, 0.f, 0}, {}}); cur = &cands.back(); }
  cur->us.push_back(us);
  std::vector<float> s = cur->us;
  std::sort(s.begin(), s.end());
  cur->plan.median_us = s[s.size() / 2];
  cur->plan.p95_us = s[std::min(s.size() - 1, (size_t)(0.95 * s.size()))];
  cur->plan.samples = (int32_t)s.size();
  const Candidate* win = &cands[0];
  for (const auto& cd : cands) if (cd.plan.median_us < win->plan.median_us) win = &cd;
  C->best[k] = win->plan;
}

void oa_plan_cache_set(void* c, int M, int N, int K, int layout, int epilogue, int role, int world, int bn, int splits) {
  auto* C = static_cast<Cache*>(c);
  std::lock_guard<std::mutex> lock(C->mu);
  C->best[Key{M, N, K, layout, epilogue, role, world}] = Plan{bn, splits, 0.f, 0.f, 0};
}

int oa_plan_cache_size(void* c) { auto* C = static_cast<Cache*>(c); std::lock_guard<std::mutex> lock(C->mu); return (int)C->best.size(); }

void oa_plan_cache_stats(void* c, uint64_t* hits, uint64_t* misses) {
  auto* C = static_cast<Cache*>(c);
  std::lock_guard<std::mutex> lock(C->mu);
  *hits = C->hits; *misses = C->misses;
}

int oa_plan_cache_timing(void* c, int M, int N, int K, int layout, int epilogue, int role, int world, float* median_us, float* p95_us, int* samples) {
  auto* C = static_cast<Cache*>(c);
  std::lock_guard<std::mutex> lock(C->mu);
  auto it = C->best.find(Key{M, N, K, layout, epilogue, role, world});
  if (it == C->best.end()) return 0;
  *median_us = it->second.median_us; *p95_us = it->second.p95_us; *samples = it->second.samples;
  return 1;
}

// 0 ok, 1 io error
int oa_plan_cache_save(void* c, const char* path) {
  auto* C = static_cast<Cache*>(c);
  std::vector<Record> recs;
  {
    std::lock_guard<std::mutex> lock(C->mu);
    for (const auto& kv : C->best) recs.push_back(Record{kv.first, kv.second});
  }
  const std::string tmp = std::string(path) + ".tmp";
  FILE* f = std::fopen(tmp.c_str(), "wb");
  if (!f) return 1;
  const uint32_t head[3] = {kMagic, kVersion, (uint32_t)recs.size()};
  const uint64_t sum = fnv(recs.data(), recs.size() * sizeof(Record));
  bool ok = std::fwrite(head, sizeof(head), 1, f) == 1 && std::fwrite(&sum, sizeof(sum), 1, f) == 1 &&
            (recs.empty() || std::fwrite(recs.data(), sizeof(Record), recs.size(), f) == recs.size());
  ok = (std::fclose(f) == 0) && ok;
  if (!ok) { std::remove(tmp.c_str()); return 1; }
  return std::rename(tmp.c_str(), path) == 0 ? 0 : 1;
}

// 0 ok, 1 missing, 2 corrupt (nothing is loaded from a corrupt file)
int oa_plan_cache_load(void* c, const char* path) {
  auto* C = static_cast<Cache*>(c);
  FILE* f = std::fopen(path, "rb");
  if (!f) return 1;
  uint32_t head[3];
  uint64_t sum = 0;
  std::vector<Record> recs;
  bool ok = std::fread(head, sizeof(head), 1, f) == 1 && std::fread(&sum, sizeof(sum), 1, f) == 1 && head[0] == kMagic && head[1] == kVersion &&
            head[2] < (1u << 24);
  if (ok) {
    recs.resize(head[2]);
    ok = recs.empty() || std::fread(recs.data(), sizeof(Record), recs.size(), f) == recs.size();
    ok = ok && fnv(recs.data(), recs.size() * sizeof(Record)) == sum;
  }
  std::fclose(f);
  if (!ok) return 2;
  std::lock_guard<std::mutex> lock(C->mu);
  for (const Record& r : recs) C->best[r.key] = r.plan;
  return 0;
}

}  // extern "C"
