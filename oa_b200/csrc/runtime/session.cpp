// Execution session and execution plan: the bookkeeping between recording and replay.
//
// Parity: Source/Private/Oa/Runtime/ExecutionSession.h:22-177 (stable resource frame, reusable graphs, cross-graph
// batch hazards), Source/Private/Oa/Runtime/ExecutionPlan.{h,cpp} (immutable compiled-graph owner).
//
// A CUDA graph bakes device addresses into its kernel nodes, so a step can only be replayed if every temporary it
// asks for lands at the address it had when the step was captured.  The session therefore hands out temporaries by
// ORDINAL inside a frame: the n-th request of a step reuses the slot of the n-th request of the step before when
// it fits, and a frame is "stable" when every request was served that way.  The allocator behind a slot lives with
// the caller (a caching-allocator block or a private pool); the session only decides reuse and tracks sizes.
#include <algorithm>
#include <cstdint>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

extern "C" {
uint64_t oa_graph_hash(void* g);
uint64_t oa_graph_node_hash(void* g, int i);
int oa_graph_num_nodes(void* g);
}

namespace {

struct Slot { uint64_t capacity = 0; uint64_t requested = 0; uint32_t generation = 0; };

struct BatchGraph { std::map<uint64_t, uint32_t> access; };   // buffer id -> 1 read, 2 write, 3 both

struct Session {
  std::vector<Slot> slots;
  uint32_t cursor = 0, last_count = 0;
  uint64_t frame = 0, stable_frames = 0;
  bool in_frame = false, changed = false;
  // graphs that finished executing, by structural hash, ready to be re-armed instead of rebuilt
  std::unordered_map<uint64_t, uint32_t> reusable;
  uint64_t reuse_hits = 0, reuse_misses = 0;
  // asynchronous batch: graphs submitted without an intermediate wait
  bool in_batch = false;
  std::vector<BatchGraph> batch;
  uint64_t pending_event = 0;
};

struct Plan {
  uint64_t graph_hash = 0;
  std::vector<uint64_t> node_hashes;
  uint64_t replays = 0;
  uint64_t session_frame = 0;
};

}  // namespace

extern "C" {

void* oa_session_create() { return new Session(); }
void oa_session_destroy(void* h) { delete static_cast<Session*>(h); }

int oa_session_begin_frame(void* h) {
  auto* s = static_cast<Session*>(h);
  if (s->in_frame) return -1;
  s->in_frame = true; s->changed = false; s->cursor = 0;
  return 0;
}
// Returns the slot ordinal.  *reused = 1 when the slot already holds at least `bytes` (same address as last frame);
// 0 when the slot is new or had to grow, in which case *capacity is what the caller must now allocate for it.
int oa_session_request(void* h, uint64_t bytes, int* reused, uint64_t* capacity) {
  auto* s = static_cast<Session*>(h);
  if (!s->in_frame) return -1;
  uint32_t ord = s->cursor++;
  if (ord >= s->slots.size()) { s->slots.emplace_back(); }
  Slot& slot = s->slots[ord];
  slot.requested = bytes;
  if (slot.capacity >= bytes && slot.capacity != 0) { *reused = 1; }
  else {
    slot.capacity = (bytes + 511) & ~uint64_t(511);
    if (slot.capacity == 0) slot.capacity = 512;
    ++slot.generation;
    s->changed = true;
    *reused = 0;
  }
  *capacity = slot.capacity;
  return (int)ord;
}
// Returns 1 when the frame was stable: nothing grew and the request count equals that of the frame before.
int oa_session_end_frame(void* h) {
  auto* s = static_cast<Session*>(h);
  if (!s->in_frame) return -1;
  s->in_frame = false;
  bool stable = !s->changed && s->frame > 0 && s->cursor == s->last_count;
  s->last_count = s->cursor;
  ++s->frame;
  if (stable) ++s->stable_frames;
  return stable ? 1 : 0;
}
// Drops slots beyond the last frame's request count (their memory can be released); returns how many.
int oa_session_trim(void* h) {
  auto* s = static_cast<Session*>(h);
  int dropped = (int)s->slots.size() - (int)s->last_count;
  if (dropped > 0) s->slots.resize(s->last_count);
  return dropped > 0 ? dropped : 0;
}
// what: 0 frames, 1 stable frames, 2 slots, 3 bytes held, 4 reuse hits, 5 reuse misses, 6 pending event
uint64_t oa_session_stat(void* h, int what) {
  auto* s = static_cast<Session*>(h);
  switch (what) {
    case 0: return s->frame;
    case 1: return s->stable_frames;
    case 2: return s->slots.size();
    case 3: { uint64_t t = 0; for (auto& x : s->slots) t += x.capacity; return t; }
    case 4: return s->reuse_hits;
    case 5: return s->reuse_misses;
    case 6: return s->pending_event;
  }
  return 0;
}
uint32_t oa_session_slot_generation(void* h, uint32_t ord) { auto* s = static_cast<Session*>(h); return ord < s->slots.size() ? s->slots[ord].generation : 0; }

// A graph whose execution completed is parked under its structural hash; recording the same structure again takes
// it back instead of building a new one.
void oa_session_park_graph(void* h, uint64_t hash) { ++static_cast<Session*>(h)->reusable[hash]; }
int oa_session_take_graph(void* h, uint64_t hash) {
  auto* s = static_cast<Session*>(h);
  auto it = s->reusable.find(hash);
  if (it == s->reusable.end() || it->second == 0) { ++s->reuse_misses; return 0; }
  if (--it->second == 0) s->reusable.erase(it);
  ++s->reuse_hits;
  return 1;
}

int oa_session_batch_begin(void* h) { auto* s = static_cast<Session*>(h); if (s->in_batch) return -1; s->in_batch = true; s->batch.clear(); return 0; }
// Adds a graph (its external buffers and how it touches them) to the open batch.  Returns the number of earlier
// graphs of the batch it conflicts with (read-after-write, write-after-read, write-after-write); `deps` receives
// their indices (up to cap).  A conflict means the submission must wait on that graph's event.
int oa_session_batch_add(void* h, const uint64_t* buffers, const uint32_t* access, int n, int* deps, int cap) {
  auto* s = static_cast<Session*>(h);
  if (!s->in_batch) return -1;
  BatchGraph g;
  for (int i = 0; i < n; ++i) g.access[buffers[i]] |= access[i] & 3u;
  int found = 0;
  for (size_t k = 0; k < s->batch.size(); ++k) {
    bool conflict = false;
    for (auto& kv : g.access) {
      auto it = s->batch[k].access.find(kv.first);
      if (it == s->batch[k].access.end()) continue;
      if ((kv.second & 2u) || (it->second & 2u)) { conflict = true; break; }
    }
    if (conflict) { if (found < cap && deps) deps[found] = (int)k; ++found; }
  }
  s->batch.push_back(std::move(g));
  return found;
}
// Closes the batch; returns how many graphs it held and records the event that completes it.
int oa_session_batch_end(void* h, uint64_t event) {
  auto* s = static_cast<Session*>(h);
  if (!s->in_batch) return -1;
  s->in_batch = false; s->pending_event = event;
  int n = (int)s->batch.size();
  s->batch.clear();
  return n;
}

// ---- execution plan: what was compiled, kept to decide whether a newly recorded graph may replay it
void* oa_plan_create(void* graph, void* session) {
  auto* p = new Plan();
  p->graph_hash = oa_graph_hash(graph);
  int n = oa_graph_num_nodes(graph);
  for (int i = 0; i < n; ++i) p->node_hashes.push_back(oa_graph_node_hash(graph, i));
  if (session) p->session_frame = static_cast<Session*>(session)->frame;
  return p;
}
void oa_plan_destroy(void* h) { delete static_cast<Plan*>(h); }
uint64_t oa_plan_hash(void* h) { return static_cast<Plan*>(h)->graph_hash; }
int oa_plan_num_nodes(void* h) { return (int)static_cast<Plan*>(h)->node_hashes.size(); }
uint64_t oa_plan_replays(void* h) { return static_cast<Plan*>(h)->replays; }
// -1: same structure; otherwise the index of the first node that differs (or the shorter length).
int oa_plan_first_mismatch(void* h, void* graph) {
  auto* p = static_cast<Plan*>(h);
  int n = oa_graph_num_nodes(graph), m = (int)p->node_hashes.size();
  for (int i = 0; i < std::min(n, m); ++i) if (oa_graph_node_hash(graph, i) != p->node_hashes[i]) return i;
  return n == m ? -1 : std::min(n, m);
}
uint64_t oa_plan_note_replay(void* h) { return ++static_cast<Plan*>(h)->replays; }

}  // extern "C"
