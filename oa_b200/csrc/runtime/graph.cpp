// Compute-graph IR of the executor (native).  The reference records every dispatch as a node (kernel name, buffers with
// access flags, push data, queue hint), derives RAW / WAR / WAW hazards per buffer into barriers, hashes nodes with FNV-1a
// to reuse compiled command buffers, and computes buffer lifetimes / alias groups
// (Source/Public/Oa/Runtime/ComputeGraph.h, Source/Private/Oa/Runtime/ComputeGraph.cpp:481-714, 1480-1499).
// On CUDA the stream already orders kernels, so here the IR serves what is left of that job:
//   * a structural hash of a recorded step: a captured CUDA graph may be replayed only while the step still records the
//     same node sequence on the same buffers (replay-safety check of the training program);
//   * dependency levels from the hazards: nodes of one level are independent and may run on different streams
//     (the multi-queue execution of the reference);
//   * buffer lifetimes -> alias groups: temporaries whose lifetimes do not overlap can share one allocation
//     (stable resource frame of the execution session);
//   * reports (node / barrier / level counts, bytes) for OA_GRAPH_REPORT.
// C ABI; no CUDA dependency.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace {

constexpr uint64_t kFnvOffset = 0xCBF29CE484222325ull, kFnvPrime = 0x100000001B3ull;

inline uint64_t fnv(uint64_t h, const void* data, size_t n) {
  const auto* p = static_cast<const uint8_t*>(data);
  for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= kFnvPrime; }
  return h;
}

enum Access : uint32_t { kRead = 1, kWrite = 2 };

struct BufferUse { uint64_t id; uint64_t bytes; uint32_t access; };

struct Node {
  std::string kernel;
  std::vector<BufferUse> uses;
  std::vector<uint8_t> push;
  uint32_t queue = 0;
  uint64_t hash = 0;
  int level = 0;
  std::vector<int> deps;       // node indices this node must wait for
};

struct Lifetime { uint64_t id, bytes; int first, last; int group; };

struct Graph {
  std::vector<Node> nodes;
  // analysis results
  bool analysed = false;
  int barriers = 0, levels = 0;
  uint64_t hash = kFnvOffset;
  std::vector<Lifetime> lifetimes;
  uint64_t bytes_naive = 0, bytes_aliased = 0;
};

void analyse(Graph& g) {
  if (g.analysed) return;
  struct Last { int writer = -1; std::vector<int> readers; };
  std::map<uint64_t, Last> last;
  std::map<uint64_t, Lifetime> life;
  g.barriers = 0; g.levels = 0; g.hash = kFnvOffset;
  for (int i = 0; i < (int)g.nodes.size(); ++i) {
    Node& n = g.nodes[i];
    n.deps.clear();
    uint64_t h = fnv(kFnvOffset, n.kernel.data(), n.kernel.size());
    h = fnv(h, n.push.data(), n.push.size());
    h = fnv(h, &n.queue, sizeof(n.queue));
    for (const BufferUse& u : n.uses) {
      h = fnv(h, &u, sizeof(u.id) + sizeof(u.bytes) + sizeof(u.access));
      Last& l = last[u.id];
      if (u.access & kWrite) {                     // WAW on the last writer, WAR on every reader since
        if (l.writer >= 0) n.deps.push_back(l.writer);
        for (int r : l.readers) n.deps.push_back(r);
      } else if (l.writer >= 0) {                  // RAW
        n.deps.push_back(l.writer);
      }
      auto it = life.find(u.id);
      if (it == life.end()) life[u.id] = Lifetime{u.id, u.bytes, i, i, -1};
      else { it->second.last = i; it->second.bytes = std::max(it->second.bytes, u.bytes); }
    }
    for (const BufferUse& u : n.uses) {            // update after all uses of the node were checked
      Last& l = last[u.id];
      if (u.access & kWrite) { l.writer = i; l.readers.clear(); }
      else l.readers.push_back(i);
    }
    std::sort(n.deps.begin(), n.deps.end());
    n.deps.erase(std::unique(n.deps.begin(), n.deps.end()), n.deps.end());
    n.deps.erase(std::remove(n.deps.begin(), n.deps.end(), i), n.deps.end());
    n.level = 0;
    for (int d : n.deps) n.level = std::max(n.level, g.nodes[d].level + 1);
    if (!n.deps.empty()) ++g.barriers;             // one barrier in front of a node with hazards
    g.levels = std::max(g.levels, n.level + 1);
    n.hash = h;
    g.hash = fnv(g.hash, &h, sizeof(h));
  }
  // alias groups: greedy interval colouring in order of first use; a buffer joins the first group whose last occupant
  // died before it is born (the group grows to the largest member)
  g.lifetimes.clear();
  for (auto& kv : life) g.lifetimes.push_back(kv.second);
  std::sort(g.lifetimes.begin(), g.lifetimes.end(), [](const Lifetime& a, const Lifetime& b) { return a.first < b.first || (a.first == b.first && a.id < b.id); });
  std::vector<int> group_free_at;
  std::vector<uint64_t> group_bytes;
  g.bytes_naive = 0;
  for (Lifetime& lt : g.lifetimes) {
    g.bytes_naive += lt.bytes;
    int chosen = -1;
    for (int k = 0; k < (int)group_free_at.size(); ++k)
      if (group_free_at[k] < lt.first) { chosen = k; break; }
    if (chosen < 0) { chosen = (int)group_free_at.size(); group_free_at.push_back(0); group_bytes.push_back(0); }
    group_free_at[chosen] = lt.last;
    group_bytes[chosen] = std::max(group_bytes[chosen], lt.bytes);
    lt.group = chosen;
  }
  g.bytes_aliased = 0;
  for (uint64_t b : group_bytes) g.bytes_aliased += b;
  g.analysed = true;
}

}  // namespace

extern "C" {

void* oa_graph_create() { return new Graph(); }
void oa_graph_destroy(void* g) { delete static_cast<Graph*>(g); }
void oa_graph_clear(void* g) { auto* G = static_cast<Graph*>(g); G->nodes.clear(); G->analysed = false; }

// Appends a node; buffers are (id, bytes, access) triples with access = 1 read, 2 write, 3 both.  Returns its index.
int oa_graph_add_node(void* g, const char* kernel, const uint64_t* buffer_ids, const uint64_t* buffer_bytes, const uint32_t* access,
                      int n_buffers, const void* push, int push_bytes, uint32_t queue) {
  auto* G = static_cast<Graph*>(g);
  Node n;
  n.kernel = kernel ? kernel : "";
  for (int i = 0; i < n_buffers; ++i) n.uses.push_back(BufferUse{buffer_ids[i], buffer_bytes[i], access[i]});
  if (push && push_bytes > 0) n.push.assign(static_cast<const uint8_t*>(push), static_cast<const uint8_t*>(push) + std::min(push_bytes, 128));
  n.queue = queue;
  G->nodes.push_back(std::move(n));
  G->analysed = false;
  return (int)G->nodes.size() - 1;
}

int oa_graph_num_nodes(void* g) { return (int)static_cast<Graph*>(g)->nodes.size(); }
uint64_t oa_graph_hash(void* g) { auto* G = static_cast<Graph*>(g); analyse(*G); return G->hash; }
uint64_t oa_graph_node_hash(void* g, int i) { auto* G = static_cast<Graph*>(g); analyse(*G); return G->nodes[i].hash; }
int oa_graph_num_barriers(void* g) { auto* G = static_cast<Graph*>(g); analyse(*G); return G->barriers; }
int oa_graph_num_levels(void* g) { auto* G = static_cast<Graph*>(g); analyse(*G); return G->levels; }
int oa_graph_node_level(void* g, int i) { auto* G = static_cast<Graph*>(g); analyse(*G); return G->nodes[i].level; }

// Writes up to `cap` dependency indices of node i; returns how many the node has.
int oa_graph_node_deps(void* g, int i, int* out, int cap) {
  auto* G = static_cast<Graph*>(g);
  analyse(*G);
  const auto& d = G->nodes[i].deps;
  for (int k = 0; k < (int)d.size() && k < cap; ++k) out[k] = d[k];
  return (int)d.size();
}

int oa_graph_num_buffers(void* g) { auto* G = static_cast<Graph*>(g); analyse(*G); return (int)G->lifetimes.size(); }

// Lifetime record k (in order of first use): id, bytes, first node, last node, alias group.
void oa_graph_buffer_at(void* g, int k, uint64_t* id, uint64_t* bytes, int* first, int* last, int* group) {
  auto* G = static_cast<Graph*>(g);
  analyse(*G);
  const Lifetime& lt = G->lifetimes[k];
  *id = lt.id; *bytes = lt.bytes; *first = lt.first; *last = lt.last; *group = lt.group;
}

void oa_graph_memory(void* g, uint64_t* naive_bytes, uint64_t* aliased_bytes) {
  auto* G = static_cast<Graph*>(g);
  analyse(*G);
  *naive_bytes = G->bytes_naive; *aliased_bytes = G->bytes_aliased;
}

const char* oa_graph_node_kernel(void* g, int i) { return static_cast<Graph*>(g)->nodes[i].kernel.c_str(); }

}  // extern "C"
