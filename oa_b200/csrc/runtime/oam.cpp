// .oam model file reader / writer (host only, C ABI).
//
// On-disk layout (little endian, packed), as written by the reference
// (Source/Public/Oa/Ml/Oam.h:22-136, Source/Private/Oa/Ml/Oam.cpp):
//   file header 64 B {magic "OAM\0", version 2, section count, flags, total size, manifest checksum}
//   section table, 64 B per section {type, compression 0, flags, offset, size, compressed size, checksum}
//   zero padding to 4096, then the payloads in the order Config(1) Weights(2) State(3) Optimizer(4)
//   Progress(5) Spirv(6); Weights and State payloads are padded to 4096.
//   Tensor section = u32 count, u32 reserved(0), count x 216 B entries {name[128], blob offset, bytes,
//   dtype u8, rank u8, reserved[6], shape u64[8]}, blob.
//   Optimizer section = 68 B header {type[16], lr, beta1, beta2, eps, weight decay, step i64,
//   param count u64, reserved[16]} + AdamM f32[] + AdamV f32[] + MuonM f32[].
//   Checksums: FNV-1a 64 per payload; manifest = FNV-1a over (header with checksum 0 || section table);
//   version 1 files carry the XOR of the section checksums instead.
// Writing is atomic: temp file -> flush -> fsync -> rename -> fsync of the directory.
// Loading validates everything (bounds, overlap, duplicates, checksums, shape/byte agreement)
// before any tensor is handed out.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>
#include <algorithm>
#include <atomic>
#include <chrono>
#include <fcntl.h>
#include <unistd.h>
#include <libgen.h>
#include <sys/stat.h>

namespace {

constexpr uint32_t kMagic = 0x004D414F, kVersion = 2, kMinVersion = 1;
constexpr size_t kPage = 4096, kMaxRank = 8, kMaxName = 128, kMaxSections = 32;

#pragma pack(push, 1)
struct FileHeader {
  uint32_t magic = kMagic, version = kVersion, num_sections = 0, flags = 0;
  uint64_t total_size = 0, checksum = 0;
  uint8_t reserved[32] = {};
};
struct SectionHeader {
  uint32_t type = 0;
  uint8_t compression = 0, reserved0[3] = {};
  uint32_t flags = 0;
  uint64_t offset = 0, size = 0, compressed_size = 0, checksum = 0;
  uint8_t reserved1[20] = {};
};
struct Config {
  char architecture[32] = {};
  uint32_t config_version = 1, flags = 0, d_model = 0, n_layers = 0, d_vocab = 256, arch_config_size = 0;
  uint8_t weight_dtype = 0, state_dtype = 0, compute_dtype = 0, reserved0 = 0;
  uint8_t reserved1[48] = {};
};
struct TensorEntry {
  char name[kMaxName] = {};
  uint64_t blob_offset = 0, num_bytes = 0;
  uint8_t dtype = 0, rank = 0, reserved[6] = {};
  uint64_t shape[kMaxRank] = {};
};
struct OptimizerHeader {
  char type[16] = "AdamW";
  float lr = 3e-4f, beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f, weight_decay = 0.1f;
  int64_t step = 0;
  uint64_t num_params = 0;
  uint8_t reserved[16] = {};
};
struct Progress {
  uint8_t phase = 0, reserved0[3] = {};
  int64_t step = 0;
  uint64_t bytes_seen = 0, env_steps = 0;
  float lr = 3e-4f, best_metric = 0.0f;
  uint8_t lower_is_better = 1, reserved1[3] = {};
  char metric_name[32] = "loss";
  uint8_t reserved2[32] = {};
};
#pragma pack(pop)
static_assert(sizeof(FileHeader) == 64, "file header");
static_assert(sizeof(SectionHeader) == 64, "section header");
static_assert(sizeof(TensorEntry) == 216, "tensor entry");
static_assert(sizeof(OptimizerHeader) == 68, "optimizer header");

uint64_t fnv1a(const uint8_t* d, size_t n, uint64_t h = 0xcbf29ce484222325ULL) {
  for (size_t i = 0; i < n; ++i) { h ^= d[i]; h *= 0x100000001b3ULL; }
  return h;
}
size_t page_align(size_t n) { return (n + kPage - 1) & ~(kPage - 1); }

size_t dtype_bytes(uint8_t d) {
  switch (d) {
    case 0: return 4; case 1: return 2; case 2: return 2; case 3: return 1; case 4: return 4; case 5: return 1;
    case 6: return 8; case 7: return 2; case 8: return 8; case 9: return 2; case 10: return 4; case 11: return 8;
    case 12: return 1; default: return 0;  // quantised block types: byte count is not checked against the shape
  }
}

struct Model {
  uint32_t format_version = kVersion;
  Config config;
  std::vector<uint8_t> arch_config;
  std::vector<TensorEntry> weight_index, state_index;
  std::vector<uint8_t> weight_blob, state_blob;
  OptimizerHeader optimizer;
  std::vector<float> adam_m, adam_v, muon_m;
  bool optimizer_present = false;
  Progress progress;
  std::string error;
};

bool known_optimizer(const OptimizerHeader& h) {
  static const char* names[] = {"SGD", "Adam", "AdamW", "Muon", "MuonAdamW"};
  for (auto n : names) if (std::strncmp(h.type, n, sizeof(h.type)) == 0) return true;
  return false;
}

std::vector<uint8_t> serialize_tensors(const std::vector<TensorEntry>& idx, const std::vector<uint8_t>& blob) {
  uint32_t count = (uint32_t)idx.size(), reserved = 0;
  std::vector<uint8_t> raw(8 + sizeof(TensorEntry) * count + blob.size());
  uint8_t* p = raw.data();
  std::memcpy(p, &count, 4); p += 4;
  std::memcpy(p, &reserved, 4); p += 4;
  for (auto& e : idx) { std::memcpy(p, &e, sizeof(e)); p += sizeof(e); }
  if (!blob.empty()) std::memcpy(p, blob.data(), blob.size());
  return raw;
}

uint64_t manifest_hash(FileHeader h, const std::vector<SectionHeader>& s) {
  h.checksum = 0;
  uint64_t x = fnv1a(reinterpret_cast<const uint8_t*>(&h), sizeof(h));
  if (!s.empty()) x = fnv1a(reinterpret_cast<const uint8_t*>(s.data()), s.size() * sizeof(SectionHeader), x);
  return x;
}

std::atomic<uint64_t> g_seq{0};

int write_all(int fd, const void* data, size_t n) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  while (n > 0) {
    ssize_t w = ::write(fd, p, n);
    if (w <= 0) return -1;
    p += w; n -= (size_t)w;
  }
  return 0;
}

// A writer never produces a file that the loader refuses: an entry whose byte count disagrees with its shape and data
// type is caught here, not at the next load.
bool entries_consistent(const std::vector<TensorEntry>& idx, std::string& err) {
  for (const TensorEntry& e : idx) {
    if (e.rank > kMaxRank) { err = std::string("tensor rank above the format's limit: ") + e.name; return false; }
    const size_t eb = dtype_bytes(e.dtype);
    if (!eb) continue;
    uint64_t n = 1;
    for (int r = 0; r < e.rank; ++r) {
      if (e.shape[r] != 0 && n > UINT64_MAX / e.shape[r]) { err = std::string("tensor element count overflow: ") + e.name; return false; }
      n *= e.shape[r];
    }
    if (n * eb != e.num_bytes) { err = std::string("tensor byte count does not match shape/dtype: ") + e.name; return false; }
  }
  return true;
}

int save_model(const Model& m, const char* path, std::string& err) {
  struct Payload { uint32_t type; std::vector<uint8_t> data; };
  std::vector<Payload> pl;
  if (!entries_consistent(m.weight_index, err) || !entries_consistent(m.state_index, err)) return 4;
  {
    std::vector<uint8_t> raw(sizeof(Config) + m.arch_config.size());
    Config c = m.config;
    c.arch_config_size = (uint32_t)m.arch_config.size();
    std::memcpy(raw.data(), &c, sizeof(c));
    if (!m.arch_config.empty()) std::memcpy(raw.data() + sizeof(c), m.arch_config.data(), m.arch_config.size());
    pl.push_back({1, std::move(raw)});
  }
  if (!m.weight_blob.empty()) pl.push_back({2, serialize_tensors(m.weight_index, m.weight_blob)});
  if (!m.state_blob.empty()) pl.push_back({3, serialize_tensors(m.state_index, m.state_blob)});
  if (m.optimizer_present || !m.adam_m.empty() || !m.adam_v.empty() || !m.muon_m.empty()) {
    if (!known_optimizer(m.optimizer)) { err = "cannot save .oam with an unknown optimizer type"; return 3; }
    OptimizerHeader h = m.optimizer;
    h.num_params = m.adam_m.size();
    if (std::strncmp(h.type, "MuonAdamW", 16) == 0) { uint64_t n = m.muon_m.size(); std::memcpy(h.reserved, &n, 8); }
    std::vector<uint8_t> raw(sizeof(h) + 4 * (m.adam_m.size() + m.adam_v.size() + m.muon_m.size()));
    uint8_t* p = raw.data();
    std::memcpy(p, &h, sizeof(h)); p += sizeof(h);
    if (!m.adam_m.empty()) { std::memcpy(p, m.adam_m.data(), 4 * m.adam_m.size()); p += 4 * m.adam_m.size(); }
    if (!m.adam_v.empty()) { std::memcpy(p, m.adam_v.data(), 4 * m.adam_v.size()); p += 4 * m.adam_v.size(); }
    if (!m.muon_m.empty()) std::memcpy(p, m.muon_m.data(), 4 * m.muon_m.size());
    pl.push_back({4, std::move(raw)});
  }
  {
    std::vector<uint8_t> raw(sizeof(Progress));
    std::memcpy(raw.data(), &m.progress, sizeof(Progress));
    pl.push_back({5, std::move(raw)});
  }
  uint32_t ns = (uint32_t)pl.size();
  size_t data_start = page_align(sizeof(FileHeader) + ns * sizeof(SectionHeader));
  std::vector<SectionHeader> sh(ns);
  uint64_t off = data_start;
  for (uint32_t i = 0; i < ns; ++i) {
    sh[i].type = pl[i].type;
    sh[i].offset = off;
    sh[i].size = pl[i].data.size();
    sh[i].checksum = fnv1a(pl[i].data.data(), pl[i].data.size());
    bool align = pl[i].type == 2 || pl[i].type == 3;
    off += align ? page_align(pl[i].data.size()) : pl[i].data.size();
  }
  FileHeader fh;
  fh.num_sections = ns;
  fh.total_size = off;
  fh.checksum = manifest_hash(fh, sh);

  std::string p(path);
  {
    std::string dir = p;
    size_t slash = dir.find_last_of('/');
    if (slash != std::string::npos) {
      dir = dir.substr(0, slash);
      std::string cur;
      for (size_t i = 0; i <= dir.size(); ++i) {
        if (i == dir.size() || dir[i] == '/') { if (!cur.empty()) ::mkdir(cur.c_str(), 0777); }
        if (i < dir.size()) cur += dir[i];
      }
    }
  }
  auto ticks = std::chrono::steady_clock::now().time_since_epoch().count();
  std::string tmp = p + ".tmp." + std::to_string((long long)ticks) + "." + std::to_string(g_seq.fetch_add(1));
  int fd = ::open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
  if (fd < 0) { err = "failed to open for write: " + tmp; return 14; }
  int rc = 0;
  rc |= write_all(fd, &fh, sizeof(fh));
  rc |= write_all(fd, sh.data(), sh.size() * sizeof(SectionHeader));
  {
    std::vector<uint8_t> z(data_start - (sizeof(fh) + sh.size() * sizeof(SectionHeader)), 0);
    rc |= write_all(fd, z.data(), z.size());
  }
  for (uint32_t i = 0; i < ns && rc == 0; ++i) {
    rc |= write_all(fd, pl[i].data.data(), pl[i].data.size());
    if (pl[i].type == 2 || pl[i].type == 3) {
      std::vector<uint8_t> z(page_align(pl[i].data.size()) - pl[i].data.size(), 0);
      if (!z.empty()) rc |= write_all(fd, z.data(), z.size());
    }
  }
  if (rc != 0 || ::fsync(fd) != 0) {
    ::close(fd);
    ::unlink(tmp.c_str());
    err = "failed to write complete .oam: " + p;
    return 8;
  }
  ::close(fd);
  if (::rename(tmp.c_str(), p.c_str()) != 0) { ::unlink(tmp.c_str()); err = "failed to replace " + p; return 14; }
  {
    std::string dir = ".";
    size_t slash = p.find_last_of('/');
    if (slash != std::string::npos) dir = slash == 0 ? "/" : p.substr(0, slash);
    int dfd = ::open(dir.c_str(), O_RDONLY | O_DIRECTORY);
    if (dfd >= 0) { ::fsync(dfd); ::close(dfd); }
  }
  return 0;
}

bool parse_tensors(const std::vector<uint8_t>& file, const SectionHeader& sh, std::vector<TensorEntry>& idx,
                   std::vector<uint8_t>& blob, std::string& err) {
  if (sh.size < 8) { err = "truncated tensor index"; return false; }
  const uint8_t* p = file.data() + sh.offset;
  uint32_t count, reserved;
  std::memcpy(&count, p, 4);
  std::memcpy(&reserved, p + 4, 4);
  if (reserved != 0) { err = "tensor index reserved field is nonzero"; return false; }
  uint64_t index_bytes = 8 + (uint64_t)count * sizeof(TensorEntry);
  if (index_bytes > sh.size) { err = "truncated tensor index entries"; return false; }
  uint64_t blob_bytes = sh.size - index_bytes;
  idx.resize(count);
  for (uint32_t i = 0; i < count; ++i) {
    std::memcpy(&idx[i], p + 8 + (size_t)i * sizeof(TensorEntry), sizeof(TensorEntry));
    const TensorEntry& e = idx[i];
    if (e.rank > kMaxRank || e.name[kMaxName - 1] != 0 || e.name[0] == 0) { err = "invalid tensor metadata"; return false; }
    if (e.blob_offset > blob_bytes || e.num_bytes > blob_bytes - e.blob_offset) {
      err = "tensor payload range is outside its section"; return false;
    }
    for (uint32_t j = 0; j < i; ++j)
      if (std::strncmp(idx[j].name, e.name, kMaxName) == 0) { err = "duplicate tensor name"; return false; }
    size_t eb = dtype_bytes(e.dtype);
    if (eb) {
      uint64_t n = 1;
      for (int r = 0; r < e.rank; ++r) {
        if (e.shape[r] != 0 && n > UINT64_MAX / e.shape[r]) { err = "tensor element count overflow"; return false; }
        n *= e.shape[r];
      }
      if (n * eb != e.num_bytes) { err = "tensor byte count does not match shape/dtype"; return false; }
    }
  }
  blob.assign(p + index_bytes, p + index_bytes + blob_bytes);
  return true;
}

Model* load_model(const char* path, std::string& err) {
  FILE* f = std::fopen(path, "rb");
  if (!f) { err = std::string("cannot open: ") + path; return nullptr; }
  std::fseek(f, 0, SEEK_END);
  long end = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  if (end < 0) { std::fclose(f); err = "corrupt .oam: cannot determine file size"; return nullptr; }
  std::vector<uint8_t> file((size_t)end);
  if (end > 0 && std::fread(file.data(), 1, (size_t)end, f) != (size_t)end) { std::fclose(f); err = "corrupt .oam: short read"; return nullptr; }
  std::fclose(f);
  auto corrupt = [&](const char* m) -> Model* { err = std::string("corrupt .oam: ") + m; return nullptr; };
  if (file.size() < sizeof(FileHeader)) return corrupt("truncated file header");
  FileHeader fh;
  std::memcpy(&fh, file.data(), sizeof(fh));
  if (fh.magic != kMagic) return corrupt("invalid magic");
  if (fh.version < kMinVersion || fh.version > kVersion) return corrupt("unsupported format version");
  if (fh.num_sections == 0 || fh.num_sections > kMaxSections) return corrupt("invalid section count");
  size_t table_end = sizeof(fh) + (size_t)fh.num_sections * sizeof(SectionHeader);
  if (table_end > file.size()) return corrupt("truncated section table");
  if (fh.total_size != file.size()) return corrupt("file size does not match header");
  std::vector<SectionHeader> sh(fh.num_sections);
  std::memcpy(sh.data(), file.data() + sizeof(fh), sh.size() * sizeof(SectionHeader));
  if (fh.version >= 2 && manifest_hash(fh, sh) != fh.checksum) return corrupt("file metadata checksum mismatch");
  bool seen[8] = {};
  uint64_t xor_sum = 0;
  for (auto& s : sh) {
    if (s.type < 1 || s.type > 6) return corrupt("unknown section type");
    if (seen[s.type]) return corrupt("duplicate section type");
    seen[s.type] = true;
    if (s.compression != 0) return corrupt("unsupported section compression");
    if (s.offset < table_end || s.offset > file.size() || s.size > file.size() - s.offset) return corrupt("section range is outside the file");
    if (fnv1a(file.data() + s.offset, s.size) != s.checksum) return corrupt("section payload checksum mismatch");
    xor_sum ^= s.checksum;
  }
  for (size_t i = 0; i < sh.size(); ++i)
    for (size_t j = i + 1; j < sh.size(); ++j) {
      uint64_t a0 = sh[i].offset, a1 = a0 + sh[i].size, b0 = sh[j].offset, b1 = b0 + sh[j].size;
      if (a0 < b1 && b0 < a1) return corrupt("overlapping section ranges");
    }
  if (fh.version == 1 && xor_sum != fh.checksum) return corrupt("legacy file checksum mismatch");
  if (!seen[1]) return corrupt("required section is missing");
  Model* m = new Model();
  m->format_version = fh.version;
  auto fail = [&](const std::string& msg) -> Model* { err = "corrupt .oam: " + msg; delete m; return nullptr; };
  for (auto& s : sh) {
    const uint8_t* p = file.data() + s.offset;
    if (s.type == 1) {
      if (s.size < sizeof(Config)) return fail("invalid config section");
      std::memcpy(&m->config, p, sizeof(Config));
      if (m->config.arch_config_size != s.size - sizeof(Config)) return fail("architecture config size mismatch");
      if (m->config.architecture[31] != 0) return fail("invalid config metadata");
      m->arch_config.assign(p + sizeof(Config), p + s.size);
    } else if (s.type == 2) {
      std::string e;
      if (!parse_tensors(file, s, m->weight_index, m->weight_blob, e)) return fail(e);
    } else if (s.type == 3) {
      std::string e;
      if (!parse_tensors(file, s, m->state_index, m->state_blob, e)) return fail(e);
    } else if (s.type == 4) {
      if (s.size < sizeof(OptimizerHeader)) return fail("invalid optimizer header");
      std::memcpy(&m->optimizer, p, sizeof(OptimizerHeader));
      if (!known_optimizer(m->optimizer)) return fail("unknown optimizer type");
      uint64_t n = m->optimizer.num_params, muon = 0;
      bool hybrid = std::strncmp(m->optimizer.type, "MuonAdamW", 16) == 0;
      bool muon_only = std::strncmp(m->optimizer.type, "Muon", 16) == 0;
      bool sgd = std::strncmp(m->optimizer.type, "SGD", 16) == 0;
      if (hybrid) std::memcpy(&muon, m->optimizer.reserved, 8);
      uint64_t body = s.size - sizeof(OptimizerHeader);
      uint64_t expect_m = n, expect_v = (muon_only || sgd) ? 0 : n;
      if (muon_only) { muon = n; expect_m = 0; }
      if ((expect_m + expect_v + muon) * 4 != body) {
        // SGD momentum is stored in the AdamM slot only
        if (!(sgd && n * 4 == body)) return fail("optimizer state size mismatch");
      }
      const float* fp = reinterpret_cast<const float*>(p + sizeof(OptimizerHeader));
      m->adam_m.assign(fp, fp + expect_m); fp += expect_m;
      m->adam_v.assign(fp, fp + expect_v); fp += expect_v;
      m->muon_m.assign(fp, fp + muon);
      m->optimizer_present = true;
    } else if (s.type == 5) {
      if (s.size < sizeof(Progress)) return fail("invalid progress section");
      std::memcpy(&m->progress, p, sizeof(Progress));
    }
  }
  return m;
}

void add_tensor(std::vector<TensorEntry>& idx, std::vector<uint8_t>& blob, const char* name, int dtype, int rank,
                const uint64_t* shape, const void* data, uint64_t bytes) {
  TensorEntry e;
  std::strncpy(e.name, name, kMaxName - 1);
  e.blob_offset = blob.size();
  e.num_bytes = bytes;
  e.dtype = (uint8_t)dtype;
  e.rank = (uint8_t)rank;
  for (int i = 0; i < rank && i < (int)kMaxRank; ++i) e.shape[i] = shape[i];
  idx.push_back(e);
  size_t old = blob.size();
  blob.resize(old + bytes);
  if (bytes) std::memcpy(blob.data() + old, data, bytes);
}

thread_local std::string g_last_error;

}  // namespace

extern "C" {

void* oam_create() { return new Model(); }
void oam_destroy(void* h) { delete static_cast<Model*>(h); }
const char* oam_last_error() { return g_last_error.c_str(); }
uint64_t oam_hash(const uint8_t* data, uint64_t n) { return fnv1a(data, n); }

void oam_set_config(void* h, const char* arch, uint32_t d_model, uint32_t n_layers, uint32_t d_vocab, int weight_dtype,
                    int state_dtype, int compute_dtype, uint32_t flags, const uint8_t* arch_cfg, uint64_t arch_cfg_bytes) {
  Model* m = static_cast<Model*>(h);
  std::memset(m->config.architecture, 0, 32);
  std::strncpy(m->config.architecture, arch, 31);
  m->config.d_model = d_model; m->config.n_layers = n_layers; m->config.d_vocab = d_vocab; m->config.flags = flags;
  m->config.weight_dtype = (uint8_t)weight_dtype; m->config.state_dtype = (uint8_t)state_dtype; m->config.compute_dtype = (uint8_t)compute_dtype;
  m->arch_config.assign(arch_cfg, arch_cfg + arch_cfg_bytes);
}
void oam_get_config(void* h, char* arch32, uint32_t* d_model, uint32_t* n_layers, uint32_t* d_vocab, int* dtypes3, uint32_t* flags) {
  Model* m = static_cast<Model*>(h);
  std::memcpy(arch32, m->config.architecture, 32);
  *d_model = m->config.d_model; *n_layers = m->config.n_layers; *d_vocab = m->config.d_vocab; *flags = m->config.flags;
  dtypes3[0] = m->config.weight_dtype; dtypes3[1] = m->config.state_dtype; dtypes3[2] = m->config.compute_dtype;
}
uint64_t oam_arch_config(void* h, const uint8_t** out) {
  Model* m = static_cast<Model*>(h);
  *out = m->arch_config.data();
  return m->arch_config.size();
}
uint32_t oam_format_version(void* h) { return static_cast<Model*>(h)->format_version; }

void oam_add_tensor(void* h, int is_state, const char* name, int dtype, int rank, const uint64_t* shape, const void* data, uint64_t bytes) {
  Model* m = static_cast<Model*>(h);
  if (is_state) add_tensor(m->state_index, m->state_blob, name, dtype, rank, shape, data, bytes);
  else add_tensor(m->weight_index, m->weight_blob, name, dtype, rank, shape, data, bytes);
}
uint32_t oam_num_tensors(void* h, int is_state) {
  Model* m = static_cast<Model*>(h);
  return (uint32_t)(is_state ? m->state_index.size() : m->weight_index.size());
}
// Fills name (128 B), dtype, rank, shape[8], bytes and returns the payload pointer.
const void* oam_tensor_at(void* h, int is_state, uint32_t i, char* name128, int* dtype, int* rank, uint64_t* shape8, uint64_t* bytes) {
  Model* m = static_cast<Model*>(h);
  auto& idx = is_state ? m->state_index : m->weight_index;
  auto& blob = is_state ? m->state_blob : m->weight_blob;
  if (i >= idx.size()) return nullptr;
  const TensorEntry& e = idx[i];
  std::memcpy(name128, e.name, kMaxName);
  *dtype = e.dtype; *rank = e.rank; *bytes = e.num_bytes;
  for (size_t k = 0; k < kMaxRank; ++k) shape8[k] = e.shape[k];
  return blob.data() + e.blob_offset;
}

void oam_set_optimizer(void* h, const char* type, float lr, float b1, float b2, float eps, float wd, int64_t step,
                       const float* m_, uint64_t nm, const float* v_, uint64_t nv, const float* mu, uint64_t nmu) {
  Model* m = static_cast<Model*>(h);
  std::memset(m->optimizer.type, 0, 16);
  std::strncpy(m->optimizer.type, type, 15);
  m->optimizer.lr = lr; m->optimizer.beta1 = b1; m->optimizer.beta2 = b2; m->optimizer.eps = eps; m->optimizer.weight_decay = wd;
  m->optimizer.step = step;
  m->adam_m.assign(m_, m_ + nm);
  m->adam_v.assign(v_, v_ + nv);
  m->muon_m.assign(mu, mu + nmu);
  m->optimizer.num_params = nm;
  m->optimizer_present = true;
}
int oam_has_optimizer(void* h) {
  Model* m = static_cast<Model*>(h);
  return m->optimizer_present || !m->adam_m.empty() || !m->adam_v.empty() || !m->muon_m.empty();
}
void oam_get_optimizer(void* h, char* type16, float* hyper5, int64_t* step, uint64_t* counts3, const float** m_, const float** v_, const float** mu) {
  Model* m = static_cast<Model*>(h);
  std::memcpy(type16, m->optimizer.type, 16);
  hyper5[0] = m->optimizer.lr; hyper5[1] = m->optimizer.beta1; hyper5[2] = m->optimizer.beta2; hyper5[3] = m->optimizer.eps; hyper5[4] = m->optimizer.weight_decay;
  *step = m->optimizer.step;
  counts3[0] = m->adam_m.size(); counts3[1] = m->adam_v.size(); counts3[2] = m->muon_m.size();
  *m_ = m->adam_m.data(); *v_ = m->adam_v.data(); *mu = m->muon_m.data();
}
void oam_set_progress(void* h, int phase, int64_t step, uint64_t bytes_seen, uint64_t env_steps, float lr, float best, int lower_is_better, const char* metric) {
  Model* m = static_cast<Model*>(h);
  m->progress.phase = (uint8_t)phase; m->progress.step = step; m->progress.bytes_seen = bytes_seen; m->progress.env_steps = env_steps;
  m->progress.lr = lr; m->progress.best_metric = best; m->progress.lower_is_better = (uint8_t)lower_is_better;
  std::memset(m->progress.metric_name, 0, 32);
  std::strncpy(m->progress.metric_name, metric, 31);
}
void oam_get_progress(void* h, int* phase, int64_t* step, uint64_t* bytes_seen, uint64_t* env_steps, float* lr, float* best, int* lower, char* metric32) {
  Model* m = static_cast<Model*>(h);
  *phase = m->progress.phase; *step = m->progress.step; *bytes_seen = m->progress.bytes_seen; *env_steps = m->progress.env_steps;
  *lr = m->progress.lr; *best = m->progress.best_metric; *lower = m->progress.lower_is_better;
  std::memcpy(metric32, m->progress.metric_name, 32);
}

int oam_save(void* h, const char* path) {
  std::string err;
  int rc = save_model(*static_cast<Model*>(h), path, err);
  g_last_error = err;
  return rc;
}
void* oam_load(const char* path) {
  std::string err;
  Model* m = load_model(path, err);
  g_last_error = err;
  return m;
}

}  // extern "C"
