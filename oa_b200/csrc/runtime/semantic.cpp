// Semantic graph: the handle-free operation / value IR that records WHAT a step computes (operations with their
// contracts, attributes, accesses, aliases and autograd provenance), beside the executable graph that records HOW
// (kernel launches).  The lowering analysis relates the two: an operation is lowered directly (one launch of its
// own), decomposed (several launches) or fused (shares a launch with other operations).
//
// Parity: Source/Public/Oa/Runtime/SemanticGraph.h:10-198, Source/Private/Oa/Runtime/SemanticGraph.cpp.
// Here it drives the reports, the replay-safety checks of a captured step and the placement of tensor- and
// expert-parallel variants, so it stays a small native library without any device dependency.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <sstream>
#include <string>
#include <vector>

namespace {

constexpr uint32_t kInvalid = 0xffffffffu;

struct Value {
  std::string name;
  int kind = 0;            // 0 matrix, 1 scalar, 2 state
  std::vector<int64_t> shape;
  int dtype = 0;
  bool external = false, is_virtual = false;
  uint32_t producer = kInvalid;
};

struct Access { uint32_t value; int mode; };   // mode: 1 read, 2 write, 3 read-write
struct Alias { uint32_t output, input; };

struct Operation {
  std::string name;
  uint64_t contract = 0;
  int differentiation = 0;   // 0 none, 1 explicit backward, 2 composite
  int lowering = 0;          // 0 dispatch, 1 GEMM
  std::vector<uint32_t> inputs, outputs, control;
  std::vector<std::pair<std::string, std::string>> attrs;
  std::vector<Access> accesses;
  std::vector<uint32_t> mutated;
  std::vector<Alias> aliases;
  uint32_t backward_of = kInvalid;
  uint64_t backward_seq = 0;
};

struct Autograd {
  uint32_t forward, output, output_index;
  uint64_t sequence;
  uint32_t backward_first = kInvalid, backward_count = 0;
  bool expanded = false;
};

struct Semantic {
  std::vector<Value> values;
  std::vector<Operation> ops;
  std::vector<Autograd> autograd;
  std::string error, report;
};

static int fail(Semantic* g, const std::string& msg) { g->error = msg; return -1; }

static std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += c; }
    else if ((unsigned char)c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o += b; }
    else o += c;
  }
  return o;
}

static int validate(Semantic* g) {
  const uint32_t nv = (uint32_t)g->values.size(), no = (uint32_t)g->ops.size();
  std::vector<int> writers(nv, 0);
  for (uint32_t i = 0; i < no; ++i) {
    const Operation& op = g->ops[i];
    if (op.name.empty()) return fail(g, "operation " + std::to_string(i) + " has no name");
    for (uint32_t v : op.inputs) {
      if (v >= nv) return fail(g, op.name + ": input value out of range");
      const Value& val = g->values[v];
      if (!val.external && (val.producer == kInvalid || val.producer >= i))
        return fail(g, op.name + ": input '" + val.name + "' is read before it is produced");
    }
    for (uint32_t v : op.outputs) {
      if (v >= nv) return fail(g, op.name + ": output value out of range");
      if (g->values[v].producer != i) return fail(g, op.name + ": output '" + g->values[v].name + "' has another producer");
      if (++writers[v] > 1) return fail(g, op.name + ": value '" + g->values[v].name + "' is produced twice");
    }
    for (uint32_t c : op.control) if (c >= i) return fail(g, op.name + ": control dependency on a later operation");
    for (uint32_t m : op.mutated)
      if (std::find(op.inputs.begin(), op.inputs.end(), m) == op.inputs.end()) return fail(g, op.name + ": mutated value is not an input");
    for (const Alias& a : op.aliases) {
      if (std::find(op.outputs.begin(), op.outputs.end(), a.output) == op.outputs.end() ||
          std::find(op.inputs.begin(), op.inputs.end(), a.input) == op.inputs.end())
        return fail(g, op.name + ": alias does not join an output to an input");
    }
    if (op.backward_of != kInvalid && op.backward_of >= no) return fail(g, op.name + ": backward of an unknown operation");
  }
  for (const Autograd& a : g->autograd) {
    if (a.forward >= no) return fail(g, "autograd record names an unknown operation");
    if (a.expanded) {
      if (a.backward_first == kInvalid || (uint64_t)a.backward_first + a.backward_count > no || a.backward_first <= a.forward)
        return fail(g, "autograd record of '" + g->ops[a.forward].name + "' has a bad backward range");
    }
  }
  g->error.clear();
  return 0;
}

}  // namespace

extern "C" {

void* oa_sem_create() { return new Semantic(); }
void oa_sem_destroy(void* h) { delete static_cast<Semantic*>(h); }
void oa_sem_reset(void* h) { auto* g = static_cast<Semantic*>(h); g->values.clear(); g->ops.clear(); g->autograd.clear(); g->error.clear(); }
const char* oa_sem_error(void* h) { return static_cast<Semantic*>(h)->error.c_str(); }
int oa_sem_num_values(void* h) { return (int)static_cast<Semantic*>(h)->values.size(); }
int oa_sem_num_ops(void* h) { return (int)static_cast<Semantic*>(h)->ops.size(); }
int oa_sem_num_autograd(void* h) { return (int)static_cast<Semantic*>(h)->autograd.size(); }

int oa_sem_add_value(void* h, const char* name, int kind, int rank, const int64_t* shape, int dtype, int external, int is_virtual) {
  auto* g = static_cast<Semantic*>(h);
  if (rank < 0 || rank > 8) return fail(g, "rank out of range");
  for (int i = 0; i < rank; ++i) if (shape[i] < 0) return fail(g, "negative extent");
  Value v;
  v.name = name ? name : "";
  v.kind = kind; v.dtype = dtype; v.external = external != 0; v.is_virtual = is_virtual != 0;
  v.shape.assign(shape, shape + rank);
  g->values.push_back(std::move(v));
  return (int)g->values.size() - 1;
}

// mutated_mask: bit i set = input i is written in place.  Outputs must not have a producer yet.
int oa_sem_add_op(void* h, const char* name, uint64_t contract, int differentiation, int lowering, const uint32_t* inputs, int n_in,
                  const uint32_t* outputs, int n_out, const uint32_t* control, int n_ctrl, uint64_t mutated_mask) {
  auto* g = static_cast<Semantic*>(h);
  const uint32_t nv = (uint32_t)g->values.size(), id = (uint32_t)g->ops.size();
  for (int i = 0; i < n_in; ++i) if (inputs[i] >= nv) return fail(g, "input value out of range");
  for (int i = 0; i < n_out; ++i) {
    if (outputs[i] >= nv) return fail(g, "output value out of range");
    if (g->values[outputs[i]].producer != kInvalid) return fail(g, "value '" + g->values[outputs[i]].name + "' already has a producer");
    if (g->values[outputs[i]].external) return fail(g, "external value '" + g->values[outputs[i]].name + "' cannot be an output");
  }
  for (int i = 0; i < n_ctrl; ++i) if (control[i] >= id) return fail(g, "control dependency on a later operation");
  Operation op;
  op.name = name ? name : "";
  op.contract = contract; op.differentiation = differentiation; op.lowering = lowering;
  op.inputs.assign(inputs, inputs + n_in);
  op.outputs.assign(outputs, outputs + n_out);
  op.control.assign(control, control + n_ctrl);
  for (int i = 0; i < n_in; ++i) {
    bool mut = i < 64 && ((mutated_mask >> i) & 1);
    op.accesses.push_back({inputs[i], mut ? 3 : 1});
    if (mut) op.mutated.push_back(inputs[i]);
  }
  for (int i = 0; i < n_out; ++i) { op.accesses.push_back({outputs[i], 2}); g->values[outputs[i]].producer = id; }
  g->ops.push_back(std::move(op));
  return (int)id;
}

int oa_sem_op_set_attr(void* h, uint32_t op, const char* key, const char* value) {
  auto* g = static_cast<Semantic*>(h);
  if (op >= g->ops.size()) return fail(g, "unknown operation");
  for (auto& kv : g->ops[op].attrs) if (kv.first == key) { kv.second = value; return 0; }
  g->ops[op].attrs.emplace_back(key, value);
  return 0;
}
int oa_sem_op_add_alias(void* h, uint32_t op, uint32_t output, uint32_t input) {
  auto* g = static_cast<Semantic*>(h);
  if (op >= g->ops.size()) return fail(g, "unknown operation");
  g->ops[op].aliases.push_back({output, input});
  return 0;
}
int oa_sem_op_set_backward_of(void* h, uint32_t op, uint32_t forward, uint64_t sequence) {
  auto* g = static_cast<Semantic*>(h);
  if (op >= g->ops.size() || forward >= g->ops.size()) return fail(g, "unknown operation");
  g->ops[op].backward_of = forward; g->ops[op].backward_seq = sequence;
  return 0;
}

int oa_sem_attach_autograd(void* h, uint32_t forward, uint32_t output_index, uint64_t sequence) {
  auto* g = static_cast<Semantic*>(h);
  if (forward >= g->ops.size()) return fail(g, "unknown operation");
  const Operation& op = g->ops[forward];
  if (output_index >= op.outputs.size()) return fail(g, op.name + ": output index out of range");
  if (op.differentiation == 0) return fail(g, op.name + ": operation is not differentiable");
  for (const Autograd& a : g->autograd) if (a.sequence == sequence) return fail(g, "autograd sequence number used twice");
  g->autograd.push_back({forward, op.outputs[output_index], output_index, sequence});
  return 0;
}
int oa_sem_complete_autograd(void* h, uint32_t forward, uint64_t sequence, uint32_t backward_first, uint32_t backward_count) {
  auto* g = static_cast<Semantic*>(h);
  for (Autograd& a : g->autograd) {
    if (a.forward != forward || a.sequence != sequence) continue;
    if (a.expanded) return fail(g, "autograd record completed twice");
    if ((uint64_t)backward_first + backward_count > g->ops.size() || backward_first <= forward) return fail(g, "bad backward range");
    a.backward_first = backward_first; a.backward_count = backward_count; a.expanded = true;
    for (uint32_t i = 0; i < backward_count; ++i) { g->ops[backward_first + i].backward_of = forward; g->ops[backward_first + i].backward_seq = sequence; }
    return 0;
  }
  return fail(g, "no autograd record for that operation and sequence");
}

int oa_sem_validate(void* h) { return validate(static_cast<Semantic*>(h)); }

int oa_sem_copy_from(void* dst, void* src) {
  auto* d = static_cast<Semantic*>(dst); auto* s = static_cast<Semantic*>(src);
  if (validate(s) != 0) { d->error = s->error; return -1; }
  d->values = s->values; d->ops = s->ops; d->autograd = s->autograd; d->error.clear();
  return 0;
}

// out = {producer, kind, dtype, rank, external, virtual}
int oa_sem_value_info(void* h, uint32_t v, int64_t* out, int64_t* shape) {
  auto* g = static_cast<Semantic*>(h);
  if (v >= g->values.size()) return -1;
  const Value& x = g->values[v];
  out[0] = x.producer == kInvalid ? -1 : (int64_t)x.producer; out[1] = x.kind; out[2] = x.dtype; out[3] = (int64_t)x.shape.size();
  out[4] = x.external; out[5] = x.is_virtual;
  for (size_t i = 0; i < x.shape.size(); ++i) shape[i] = x.shape[i];
  return 0;
}
const char* oa_sem_value_name(void* h, uint32_t v) { auto* g = static_cast<Semantic*>(h); return v < g->values.size() ? g->values[v].name.c_str() : ""; }
const char* oa_sem_op_name(void* h, uint32_t op) { auto* g = static_cast<Semantic*>(h); return op < g->ops.size() ? g->ops[op].name.c_str() : ""; }
// out = {contract, differentiation, lowering, n_in, n_out, backward_of (-1 none), backward_seq, n_mutated}
int oa_sem_op_info(void* h, uint32_t op, int64_t* out) {
  auto* g = static_cast<Semantic*>(h);
  if (op >= g->ops.size()) return -1;
  const Operation& o = g->ops[op];
  out[0] = (int64_t)o.contract; out[1] = o.differentiation; out[2] = o.lowering; out[3] = (int64_t)o.inputs.size(); out[4] = (int64_t)o.outputs.size();
  out[5] = o.backward_of == kInvalid ? -1 : (int64_t)o.backward_of; out[6] = (int64_t)o.backward_seq; out[7] = (int64_t)o.mutated.size();
  return 0;
}

// Lowering analysis.  The executable graph is given as, per node, the list of semantic operations the launch
// implements (CSR: node_offsets[n_nodes + 1] into node_ops); a node that names no operation is a compatibility
// node (a launch recorded outside any contract).  out = {schema-owned nodes, compatibility nodes, direct ops,
// decomposed ops, fused ops, fused nodes, max nodes per op, max ops per node}; per_op (may be null) receives the
// launch count of every operation.  Returns -1 when a node names an unknown operation or an operation has no
// launch although it produces a value that is not virtual.
int oa_sem_analyze_lowering(void* h, const uint32_t* node_ops, const uint32_t* node_offsets, int n_nodes, uint32_t* out, uint32_t* per_op) {
  auto* g = static_cast<Semantic*>(h);
  const uint32_t no = (uint32_t)g->ops.size();
  std::vector<uint32_t> count(no, 0);
  std::vector<bool> shares(no, false);
  uint32_t owned = 0, compat = 0, fused_nodes = 0, max_ops_per_node = 0;
  for (int n = 0; n < n_nodes; ++n) {
    uint32_t lo = node_offsets[n], hi = node_offsets[n + 1];
    if (hi == lo) { ++compat; continue; }
    ++owned;
    std::set<uint32_t> distinct(node_ops + lo, node_ops + hi);
    for (uint32_t op : distinct) {
      if (op >= no) return fail(g, "executable node " + std::to_string(n) + " names an unknown operation");
      ++count[op];
      if (distinct.size() > 1) shares[op] = true;
    }
    if (distinct.size() > 1) ++fused_nodes;
    max_ops_per_node = std::max<uint32_t>(max_ops_per_node, (uint32_t)distinct.size());
  }
  uint32_t direct = 0, decomposed = 0, fused = 0, max_nodes = 0;
  for (uint32_t i = 0; i < no; ++i) {
    if (count[i] == 0) {
      bool real_output = false;
      for (uint32_t v : g->ops[i].outputs) real_output |= !g->values[v].is_virtual;
      if (real_output || !g->ops[i].mutated.empty()) return fail(g, "operation '" + g->ops[i].name + "' has no executable node");
      continue;
    }
    if (shares[i]) ++fused; else if (count[i] == 1) ++direct; else ++decomposed;
    max_nodes = std::max(max_nodes, count[i]);
  }
  out[0] = owned; out[1] = compat; out[2] = direct; out[3] = decomposed; out[4] = fused; out[5] = fused_nodes; out[6] = max_nodes; out[7] = max_ops_per_node;
  if (per_op) std::copy(count.begin(), count.end(), per_op);
  g->error.clear();
  return 0;
}

const char* oa_sem_report_json(void* h, const char* name) {
  auto* g = static_cast<Semantic*>(h);
  std::ostringstream o;
  o << "{\"name\":\"" << json_escape(name ? name : "") << "\",\"values\":[";
  for (size_t i = 0; i < g->values.size(); ++i) {
    const Value& v = g->values[i];
    o << (i ? "," : "") << "{\"id\":" << i << ",\"name\":\"" << json_escape(v.name) << "\",\"kind\":" << v.kind << ",\"dtype\":" << v.dtype << ",\"shape\":[";
    for (size_t k = 0; k < v.shape.size(); ++k) o << (k ? "," : "") << v.shape[k];
    o << "],\"external\":" << (v.external ? "true" : "false") << ",\"virtual\":" << (v.is_virtual ? "true" : "false") << ",\"producer\":";
    if (v.producer == kInvalid) o << "null"; else o << v.producer;
    o << "}";
  }
  o << "],\"operations\":[";
  for (size_t i = 0; i < g->ops.size(); ++i) {
    const Operation& op = g->ops[i];
    o << (i ? "," : "") << "{\"id\":" << i << ",\"name\":\"" << json_escape(op.name) << "\",\"contract\":\"" << std::hex << op.contract << std::dec
      << "\",\"differentiation\":" << op.differentiation << ",\"lowering\":" << op.lowering << ",\"inputs\":[";
    for (size_t k = 0; k < op.inputs.size(); ++k) o << (k ? "," : "") << op.inputs[k];
    o << "],\"outputs\":[";
    for (size_t k = 0; k < op.outputs.size(); ++k) o << (k ? "," : "") << op.outputs[k];
    o << "],\"mutated\":[";
    for (size_t k = 0; k < op.mutated.size(); ++k) o << (k ? "," : "") << op.mutated[k];
    o << "],\"attributes\":{";
    for (size_t k = 0; k < op.attrs.size(); ++k) o << (k ? "," : "") << "\"" << json_escape(op.attrs[k].first) << "\":\"" << json_escape(op.attrs[k].second) << "\"";
    o << "},\"backward_of\":";
    if (op.backward_of == kInvalid) o << "null"; else o << op.backward_of;
    o << "}";
  }
  o << "],\"autograd\":[";
  for (size_t i = 0; i < g->autograd.size(); ++i) {
    const Autograd& a = g->autograd[i];
    o << (i ? "," : "") << "{\"forward\":" << a.forward << ",\"output\":" << a.output << ",\"sequence\":" << a.sequence << ",\"expanded\":"
      << (a.expanded ? "true" : "false") << ",\"backward_count\":" << a.backward_count << "}";
  }
  o << "]}";
  g->report = o.str();
  return g->report.c_str();
}

}  // extern "C"
