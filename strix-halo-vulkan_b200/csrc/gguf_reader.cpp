// GGUF v2/v3 container reader (reference: gguf/gguf.go:265-403 parse, :501-518 value tags):
// mmaps the file, reads the hyper-parameters the way llm/model.go:66-96, 375-468 does, and
// uploads every tensor to the device.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "model.h"

namespace b200 {
namespace {

struct Cursor {
  const uint8_t* p; size_t n, o = 0; bool bad = false;
  template <class T> T get() {
    T v{};
    if (o + sizeof(T) > n) { bad = true; return v; }
    memcpy(&v, p + o, sizeof(T)); o += sizeof(T);
    return v;
  }
  std::string str() {
    uint64_t len = get<uint64_t>();
    if (bad || len > n - o) { bad = true; return ""; }
    std::string s((const char*)p + o, (size_t)len); o += (size_t)len;
    return s;
  }
};

struct Value { double num = 0; std::string s; std::vector<double> arr; };

bool read_value(Cursor& c, uint32_t tag, Value* v, int depth = 0) {
  switch (tag) {
    case 0: v->num = c.get<uint8_t>(); break;
    case 1: v->num = c.get<int8_t>(); break;
    case 2: v->num = c.get<uint16_t>(); break;
    case 3: v->num = c.get<int16_t>(); break;
    case 4: v->num = c.get<uint32_t>(); break;
    case 5: v->num = c.get<int32_t>(); break;
    case 6: v->num = c.get<float>(); break;
    case 7: v->num = c.get<uint8_t>(); break;
    case 8: v->s = c.str(); break;
    case 9: {
      if (depth > 2) return false;
      uint32_t et = c.get<uint32_t>(); uint64_t n = c.get<uint64_t>();
      for (uint64_t i = 0; i < n && !c.bad; i++) { Value e; if (!read_value(c, et, &e, depth + 1)) return false; v->arr.push_back(e.num); }
      break;
    }
    case 10: v->num = (double)c.get<uint64_t>(); break;
    case 11: v->num = (double)c.get<int64_t>(); break;
    case 12: v->num = c.get<double>(); break;
    default: return false;
  }
  return !c.bad;
}

}  // namespace

int load_gguf_into(const char* path, int device, Model* m) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) { set_error(std::string("cannot open ") + path); return EIO_; }
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size < 24) { close(fd); set_error(std::string(path) + ": too short for a GGUF file"); return EIO_; }
  void* map = mmap(nullptr, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) { set_error(std::string("cannot mmap ") + path); return EIO_; }
  struct Unmap { void* p; size_t n; ~Unmap() { munmap(p, n); } } unmap{map, (size_t)sb.st_size};
  Cursor c{(const uint8_t*)map, (size_t)sb.st_size};
  if (memcmp(c.p, "GGUF", 4) != 0) { set_error(std::string(path) + ": not a GGUF file"); return EINVAL_; }
  c.o = 4;
  uint32_t version = c.get<uint32_t>();
  if (version != 2 && version != 3) { set_error(std::string(path) + ": GGUF version " + std::to_string(version) + " is not 2 or 3"); return EINVAL_; }
  uint64_t nt = c.get<uint64_t>(), nkv = c.get<uint64_t>();
  std::map<std::string, Value> kv;
  for (uint64_t i = 0; i < nkv; i++) {
    std::string key = c.str();
    uint32_t tag = c.get<uint32_t>();
    Value v;
    if (c.bad || !read_value(c, tag, &v)) { set_error(std::string(path) + ": malformed metadata near key " + key); return EINVAL_; }
    kv[key] = v;
  }
  struct Info { std::string name; uint32_t nd, type; int64_t dims[4]; uint64_t off; };
  std::vector<Info> infos;
  for (uint64_t i = 0; i < nt; i++) {
    Info in{}; in.name = c.str(); in.nd = c.get<uint32_t>();
    if (c.bad || in.nd < 1 || in.nd > 4) { set_error(std::string(path) + ": malformed tensor table"); return EINVAL_; }
    for (uint32_t d = 0; d < in.nd; d++) in.dims[d] = (int64_t)c.get<uint64_t>();
    in.type = c.get<uint32_t>(); in.off = c.get<uint64_t>();
    if (c.bad) { set_error(std::string(path) + ": truncated tensor table"); return EINVAL_; }
    infos.push_back(in);
  }
  uint64_t align = kv.count("general.alignment") ? (uint64_t)kv["general.alignment"].num : 32;
  if (align == 0) align = 32;
  const uint64_t base = (c.o + align - 1) / align * align;
  const std::string arch = kv.count("general.architecture") ? kv["general.architecture"].s : "";
  if (arch.empty()) { set_error(std::string(path) + ": checkpoint states no general.architecture"); return EINVAL_; }
  auto num = [&](const std::string& k, double def = 0) { auto it = kv.find(arch + "." + k); return it == kv.end() ? def : it->second.num; };
  b200_config cfg{};
  const int draft = (int)num("nextn_predict_layers");
  cfg.n_layer = (int)num("block_count") - draft; cfg.n_embd = (int)num("embedding_length");
  cfg.n_head = (int)num("attention.head_count"); cfg.n_head_kv = (int)num("attention.head_count_kv");
  cfg.head_dim = (int)num("attention.key_length"); cfg.rope_dims = (int)num("rope.dimension_count");
  cfg.rope_base = (float)num("rope.freq_base", 10000.0); cfg.eps = (float)num("attention.layer_norm_rms_epsilon", 1e-6);
  cfg.n_expert = (int)num("expert_count"); cfg.n_expert_used = (int)num("expert_used_count");
  cfg.ffn_expert = (int)num("expert_feed_forward_length");
  cfg.ffn_shared = (int)num("expert_shared_feed_forward_length", cfg.ffn_expert);
  cfg.dn_head_dim = (int)num("ssm.state_size"); cfg.dn_heads_k = (int)num("ssm.group_count"); cfg.dn_heads_v = (int)num("ssm.time_step_rank");
  cfg.dn_conv = (int)num("ssm.conv_kernel"); cfg.has_draft = draft ? 1 : 0;
  for (const Info& in : infos) if (in.name == "token_embd.weight" && in.nd > 1) cfg.vocab = (int)in.dims[1];  // llm/model.go:91-93
  m->c = cfg; m->device = device;
  for (const Info& in : infos) {
    int64_t rows = 1;
    for (uint32_t d = 1; d < in.nd; d++) rows *= in.dims[d];
    const int64_t rb = gguf_row_bytes(in.type, in.dims[0]);
    if (rb < 0) { set_error(in.name + ": unsupported ggml type " + std::to_string(in.type)); return EINVAL_; }
    if (base + in.off + (uint64_t)(rb * rows) > (uint64_t)sb.st_size) { set_error(in.name + ": data runs past the end of the file"); return EINVAL_; }
    B200_TRY(m->add_host(in.name, in.type, in.nd, in.dims, c.p + base + in.off));
  }
  return m->finalize();
}

}  // namespace b200
