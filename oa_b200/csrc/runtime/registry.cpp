// Kernel registry and operation contracts (native).
// The reference keeps an authoritative kernel list - name, stable id (category prefix + ordinal), category, provider
// (Source/Public/Oa/Core/KernelRegistry.h:1-521) - and a registry of operation contracts - name, FNV-1a hash, kind,
// differentiation, lowering, effects, mutated-input mask (Source/Public/Oa/Core/Operation.h:12-166,
// Source/Private/Oa/Core/OperationRegistry.gen.h).  Here the same two tables live in the runtime library: the kernel
// table is filled from the exported C entry points of the kernel library (one row per entry, grouped by source file), the
// operation table from the matrix-function namespace; graph reports, the semantic graph and the fusion planner look
// names up here, and a stable id survives rebuilds as long as the entry keeps its position inside its category.
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace {

constexpr uint64_t kFnvOffset = 0xCBF29CE484222325ull, kFnvPrime = 0x100000001B3ull;

uint64_t fnv1a(const char* s) {
  uint64_t h = kFnvOffset;
  for (; *s; ++s) { h ^= (uint8_t)*s; h *= kFnvPrime; }
  return h;
}

struct Kernel { std::string name, category, provider; uint32_t id; };
struct Operation {
  std::string name;
  uint64_t hash;
  int kind, differentiation, lowering, effects;
  uint32_t mutated_mask;
  std::vector<std::string> kernels;
};

struct Registry {
  std::mutex mu;
  std::vector<Kernel> kernels;
  std::map<std::string, int> kernel_by_name;
  std::map<uint32_t, int> kernel_by_id;
  std::map<std::string, uint32_t> category_prefix, category_count;
  std::vector<Operation> ops;
  std::map<std::string, int> op_by_name;
  std::map<uint64_t, int> op_by_hash;
};

Registry& reg() { static Registry r; return r; }

}  // namespace

extern "C" {

uint64_t oa_registry_fnv1a(const char* s) { return fnv1a(s ? s : ""); }

// Registers a kernel entry; returns its stable id (category prefix in the high 16 bits, ordinal inside the category in
// the low 16).  Registering the same name again returns the existing id.
uint32_t oa_registry_add_kernel(const char* name, const char* category, const char* provider) {
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  auto it = r.kernel_by_name.find(name);
  if (it != r.kernel_by_name.end()) return r.kernels[it->second].id;
  auto pit = r.category_prefix.find(category);
  if (pit == r.category_prefix.end()) pit = r.category_prefix.emplace(category, (uint32_t)r.category_prefix.size() + 1).first;
  const uint32_t ordinal = r.category_count[category]++;
  Kernel k{name, category, provider ? provider : "", (pit->second << 16) | (ordinal & 0xFFFFu)};
  r.kernel_by_name[k.name] = (int)r.kernels.size();
  r.kernel_by_id[k.id] = (int)r.kernels.size();
  r.kernels.push_back(k);
  return k.id;
}

int oa_registry_num_kernels() { return (int)reg().kernels.size(); }
int oa_registry_find_kernel(const char* name) { auto& r = reg(); auto it = r.kernel_by_name.find(name); return it == r.kernel_by_name.end() ? -1 : it->second; }
int oa_registry_find_kernel_id(uint32_t id) { auto& r = reg(); auto it = r.kernel_by_id.find(id); return it == r.kernel_by_id.end() ? -1 : it->second; }
const char* oa_registry_kernel_name(int i) { return reg().kernels[i].name.c_str(); }
const char* oa_registry_kernel_category(int i) { return reg().kernels[i].category.c_str(); }
const char* oa_registry_kernel_provider(int i) { return reg().kernels[i].provider.c_str(); }
uint32_t oa_registry_kernel_id(int i) { return reg().kernels[i].id; }

// kind: 0 elementwise, 1 reduction, 2 gemm, 3 indexing, 4 normalisation, 5 attention, 6 loss, 7 shape, 8 factory, 9 other
// differentiation: 0 none, 1 analytic backward; lowering: 0 dispatch, 1 gemm, 2 composite; effects: 0 pure, 1 mutates input,
// 2 random.  Returns the operation index; the hash is FNV-1a of the name (stable across builds).
int oa_registry_add_operation(const char* name, int kind, int differentiation, int lowering, int effects, uint32_t mutated_mask) {
  Registry& r = reg();
  std::lock_guard<std::mutex> lock(r.mu);
  auto it = r.op_by_name.find(name);
  if (it != r.op_by_name.end()) return it->second;
  Operation o{name, fnv1a(name), kind, differentiation, lowering, effects, mutated_mask, {}};
  const int idx = (int)r.ops.size();
  r.op_by_name[o.name] = idx;
  r.op_by_hash[o.hash] = idx;
  r.ops.push_back(o);
  return idx;
}

void oa_registry_operation_add_kernel(int op, const char* kernel) { reg().ops[op].kernels.emplace_back(kernel); }
int oa_registry_num_operations() { return (int)reg().ops.size(); }
int oa_registry_find_operation(const char* name) { auto& r = reg(); auto it = r.op_by_name.find(name); return it == r.op_by_name.end() ? -1 : it->second; }
int oa_registry_find_operation_hash(uint64_t hash) { auto& r = reg(); auto it = r.op_by_hash.find(hash); return it == r.op_by_hash.end() ? -1 : it->second; }
const char* oa_registry_operation_name(int i) { return reg().ops[i].name.c_str(); }
uint64_t oa_registry_operation_hash(int i) { return reg().ops[i].hash; }
void oa_registry_operation_fields(int i, int* kind, int* differentiation, int* lowering, int* effects, uint32_t* mutated_mask) {
  const Operation& o = reg().ops[i];
  *kind = o.kind; *differentiation = o.differentiation; *lowering = o.lowering; *effects = o.effects; *mutated_mask = o.mutated_mask;
}
int oa_registry_operation_num_kernels(int i) { return (int)reg().ops[i].kernels.size(); }
const char* oa_registry_operation_kernel(int i, int k) { return reg().ops[i].kernels[k].c_str(); }

}  // extern "C"
