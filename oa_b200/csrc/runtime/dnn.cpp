// Fusion planner: validates a small operation graph (single assignment, producers before consumers) and partitions it
// into the engines the kernel library provides, with the values each partition must keep for the backward pass
// (reference: Source/Public/Oa/Runtime/Dnn.h:16-100, Source/Private/Oa/Runtime/Dnn.cpp; engines Portable /
// BlasLtEpilogue / PackedQkv / GatedFfn / ResidualNorm / FlashAttention / GroupedMoe).
// This planner works on use-def chains rather than on windows of adjacent ops, so unrelated ops may sit between the
// members of a pattern, and it knows two more engines: a matmul whose input is marked row-sharded becomes
// AllGatherGemm, a matmul whose output is marked row-sharded becomes GemmReduceScatter (the tensor-parallel kernels).
#include <algorithm>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace {

enum OpType : int { kMatmul, kBiasAdd, kRelu, kGelu, kSilu, kMultiply, kAdd, kRmsNorm, kFlashAttentionCausal, kGroupedGemm, kNumOps };
enum Engine : int { kPortable, kGemmEpilogue, kPackedQkv, kGatedFfn, kResidualNorm, kFlashAttention, kGroupedMoe, kAllGatherGemm, kGemmReduceScatter };

struct Matrix { uint32_t id; int rank; int64_t shape[4]; int dtype; bool external, is_virtual, row_sharded; };
struct Op { int type; std::vector<uint32_t> in, out; bool training; };
struct Partition { int engine; std::vector<uint32_t> ops; std::vector<uint32_t> saved; };

struct DnnGraph {
  std::vector<Matrix> mats;
  std::vector<Op> ops;
  std::vector<Partition> plan;
  uint64_t hash = 0;
  std::string error;
};

const Matrix* find(const DnnGraph& g, uint32_t id) {
  for (const auto& m : g.mats) if (m.id == id) return &m;
  return nullptr;
}

bool validate(DnnGraph& g) {
  if (g.mats.empty() || g.ops.empty()) { g.error = "graph is empty"; return false; }
  std::vector<uint32_t> produced;
  for (const Op& op : g.ops) {
    for (uint32_t id : op.in) {
      const Matrix* m = find(g, id);
      if (!m) { g.error = "operation has a dangling input"; return false; }
      if (!m->external && std::find(produced.begin(), produced.end(), id) == produced.end()) { g.error = "value consumed before its producer"; return false; }
    }
    for (uint32_t id : op.out) {
      if (!find(g, id)) { g.error = "operation has a dangling output"; return false; }
      if (std::find(produced.begin(), produced.end(), id) != produced.end()) { g.error = "a value is assigned twice"; return false; }
      produced.push_back(id);
    }
  }
  return true;
}

void mix(uint64_t& h, uint64_t v) { h ^= v; h *= 0x100000001b3ull; }

bool plan(DnnGraph& g, bool allow_recompute) {
  g.plan.clear();
  if (!validate(g)) return false;
  uint64_t h = 0xcbf29ce484222325ull;
  for (const Matrix& m : g.mats) {
    mix(h, m.id); mix(h, (uint64_t)m.dtype); mix(h, (uint64_t)m.rank);
    for (int d = 0; d < m.rank; ++d) mix(h, (uint64_t)m.shape[d]);
    mix(h, m.external); mix(h, m.is_virtual); mix(h, m.row_sharded);
  }
  const int n = (int)g.ops.size();
  for (const Op& op : g.ops) mix(h, (uint64_t)op.type);
  g.hash = h;
  // use-def: the consumers of every value
  std::map<uint32_t, std::vector<int>> users;
  for (int i = 0; i < n; ++i) for (uint32_t id : g.ops[i].in) users[id].push_back(i);
  std::vector<char> taken(n, 0);
  auto sole_user = [&](int i) -> int {          // the single consumer of op i's single output, or -1
    if (g.ops[i].out.size() != 1) return -1;
    auto it = users.find(g.ops[i].out[0]);
    if (it == users.end() || it->second.size() != 1) return -1;
    return taken[it->second[0]] ? -1 : it->second[0];
  };
  auto is_act = [](int t) { return t == kRelu || t == kGelu || t == kSilu; };
  auto emit = [&](int engine, std::vector<int> ops, std::vector<uint32_t> saved) {
    std::sort(ops.begin(), ops.end());
    Partition p; p.engine = engine; p.saved = std::move(saved);
    for (int o : ops) { p.ops.push_back((uint32_t)o); taken[o] = 1; }
    g.plan.push_back(std::move(p));
  };
  for (int i = 0; i < n; ++i) {
    if (taken[i]) continue;
    const Op& op = g.ops[i];
    if (op.type == kMatmul && !op.in.empty()) {
      const uint32_t x = op.in[0];
      std::vector<int> sib;                       // untaken matmuls reading the same activation, in program order
      for (int u : users[x]) if (!taken[u] && g.ops[u].type == kMatmul && g.ops[u].in[0] == x) sib.push_back(u);
      // gated FFN: two sibling matmuls, silu on one, multiply joining both
      bool done = false;
      for (size_t a = 0; a < sib.size() && !done; ++a) for (size_t b = 0; b < sib.size() && !done; ++b) {
        if (a == b) continue;
        const int act = sole_user(sib[a]);
        if (act < 0 || g.ops[act].type != kSilu) continue;
        const int mul = sole_user(act), mul2 = sole_user(sib[b]);
        if (mul >= 0 && mul == mul2 && g.ops[mul].type == kMultiply) {
          emit(kGatedFfn, {sib[a], sib[b], act, mul}, op.training ? std::vector<uint32_t>{x} : std::vector<uint32_t>{});
          done = true;
        }
      }
      if (done) { --i; continue; }                 // op i may have been one of the pair or not: look at it again
      if (sib.size() >= 3) {
        emit(kPackedQkv, {sib[0], sib[1], sib[2]}, op.training ? std::vector<uint32_t>{x} : std::vector<uint32_t>{});
        --i; continue;
      }
      const Matrix* mx = find(g, x);
      const Matrix* my = op.out.empty() ? nullptr : find(g, op.out[0]);
      if (mx && mx->row_sharded) { emit(kAllGatherGemm, {i}, op.training ? std::vector<uint32_t>{x} : std::vector<uint32_t>{}); continue; }
      if (my && my->row_sharded) { emit(kGemmReduceScatter, {i}, op.training ? std::vector<uint32_t>{x} : std::vector<uint32_t>{}); continue; }
      const int bias = sole_user(i);
      if (bias >= 0 && g.ops[bias].type == kBiasAdd) {
        std::vector<int> members{i, bias};
        std::vector<uint32_t> saved;
        const int act = sole_user(bias);
        if (act >= 0 && is_act(g.ops[act].type)) {
          members.push_back(act);
          if (op.training && !allow_recompute) saved.push_back(g.ops[bias].out[0]);
        }
        emit(kGemmEpilogue, members, saved);
        continue;
      }
    }
    if (op.type == kFlashAttentionCausal) { emit(kFlashAttention, {i}, op.training ? op.out : std::vector<uint32_t>{}); continue; }
    if (op.type == kGroupedGemm) { emit(kGroupedMoe, {i}, (op.training && !op.in.empty()) ? std::vector<uint32_t>{op.in[0]} : std::vector<uint32_t>{}); continue; }
    if (op.type == kAdd) {
      const int norm = sole_user(i);
      // a residual stream usually has two readers (the norm and the next add): accept any norm among the users
      int found = norm >= 0 && g.ops[norm].type == kRmsNorm ? norm : -1;
      if (found < 0 && op.out.size() == 1)
        for (int u : users[op.out[0]]) if (!taken[u] && g.ops[u].type == kRmsNorm) { found = u; break; }
      if (found >= 0) { emit(kResidualNorm, {i, found}, {}); continue; }
    }
    emit(kPortable, {i}, {});
  }
  return true;
}

}  // namespace

extern "C" {

void* oa_dnn_create() { return new DnnGraph(); }
void oa_dnn_destroy(void* g) { delete static_cast<DnnGraph*>(g); }
const char* oa_dnn_error(void* g) { return static_cast<DnnGraph*>(g)->error.c_str(); }

int oa_dnn_add_matrix(void* g, uint32_t id, int rank, const int64_t* shape, int dtype, int external, int is_virtual, int row_sharded) {
  auto* G = static_cast<DnnGraph*>(g);
  int64_t ne = 1;
  for (int d = 0; d < rank && d < 4; ++d) ne *= shape[d];
  if (id == 0xffffffffu || rank <= 0 || rank > 4 || ne <= 0) { G->error = "matrix has an invalid id or shape"; return 1; }
  if (find(*G, id)) { G->error = "matrix ids must be unique"; return 1; }
  Matrix m{id, rank, {0, 0, 0, 0}, dtype, external != 0, is_virtual != 0, row_sharded != 0};
  for (int d = 0; d < rank; ++d) m.shape[d] = shape[d];
  G->mats.push_back(m);
  return 0;
}

int oa_dnn_add_op(void* g, int type, const uint32_t* inputs, int n_in, const uint32_t* outputs, int n_out, int training) {
  auto* G = static_cast<DnnGraph*>(g);
  if (type < 0 || type >= kNumOps || n_in <= 0 || n_out <= 0) { G->error = "operation needs a known type, inputs and outputs"; return 1; }
  Op op; op.type = type; op.in.assign(inputs, inputs + n_in); op.out.assign(outputs, outputs + n_out); op.training = training != 0;
  G->ops.push_back(std::move(op));
  return 0;
}

int oa_dnn_plan(void* g, int allow_recompute) { return plan(*static_cast<DnnGraph*>(g), allow_recompute != 0) ? 0 : 1; }
uint64_t oa_dnn_hash(void* g) { return static_cast<DnnGraph*>(g)->hash; }
int oa_dnn_num_partitions(void* g) { return (int)static_cast<DnnGraph*>(g)->plan.size(); }
int oa_dnn_partition_engine(void* g, int p) { return static_cast<DnnGraph*>(g)->plan[p].engine; }

int oa_dnn_partition_ops(void* g, int p, uint32_t* out, int cap) {
  const auto& v = static_cast<DnnGraph*>(g)->plan[p].ops;
  for (int i = 0; i < (int)v.size() && i < cap; ++i) out[i] = v[i];
  return (int)v.size();
}

int oa_dnn_partition_saved(void* g, int p, uint32_t* out, int cap) {
  const auto& v = static_cast<DnnGraph*>(g)->plan[p].saved;
  for (int i = 0; i < (int)v.size() && i < cap; ++i) out[i] = v[i];
  return (int)v.size();
}

}  // extern "C"
