// GGUF v2/v3 container reader (reference: gguf/gguf.go:265-403 parse, :501-518 value tags):
// mmaps the file, reads the hyper-parameters the way llm/model.go:66-96, 375-468 does, and
// uploads every tensor to the device. A checkpoint split over several files
// (`<base>-00001-of-00004.gguf`, reference: gguf/gguf.go:726-886) is opened from any one of
// its shards: every shard is a whole GGUF with its own tensor table, the first carries the
// model's metadata, and `split.no` / `split.count` / `split.tensors.count` are checked so that
// an incomplete download is refused instead of surfacing later as a missing weight.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cctype>
#include <cstdio>
#include <cstdlib>
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


struct Info { std::string name; uint32_t nd, type; int64_t dims[4]; uint64_t off; };

// one shard, mapped
struct Shard {
  std::string path;
  void* map = MAP_FAILED; size_t size = 0;
  std::map<std::string, Value> kv;
  std::vector<Info> infos;
  uint64_t base = 0;   // offset of the data section
  Shard() = default;
  Shard(const Shard&) = delete;
  Shard& operator=(const Shard&) = delete;
  ~Shard() { if (map != MAP_FAILED) munmap(map, size); }
  const uint8_t* bytes() const { return (const uint8_t*)map; }
};

int open_shard(const std::string& path, Shard* sh) {
  sh->path = path;
  int fd = open(path.c_str(), O_RDONLY);
  if (fd < 0) { set_error("cannot open " + path); return EIO_; }
  struct stat sb;
  if (fstat(fd, &sb) != 0 || sb.st_size < 24) { close(fd); set_error(path + ": too short for a GGUF file"); return EIO_; }
  sh->map = mmap(nullptr, (size_t)sb.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (sh->map == MAP_FAILED) { set_error("cannot mmap " + path); return EIO_; }
  sh->size = (size_t)sb.st_size;
  Cursor c{sh->bytes(), sh->size};
  if (memcmp(c.p, "GGUF", 4) != 0) { set_error(path + ": not a GGUF file"); return EINVAL_; }
  c.o = 4;
  uint32_t version = c.get<uint32_t>();
  if (version != 2 && version != 3) { set_error(path + ": GGUF version " + std::to_string(version) + " is not 2 or 3"); return EINVAL_; }
  uint64_t nt = c.get<uint64_t>(), nkv = c.get<uint64_t>();
  for (uint64_t i = 0; i < nkv; i++) {
    std::string key = c.str();
    uint32_t tag = c.get<uint32_t>();
    Value v;
    if (c.bad || !read_value(c, tag, &v)) { set_error(path + ": malformed metadata near key " + key); return EINVAL_; }
    sh->kv[key] = v;
  }
  for (uint64_t i = 0; i < nt; i++) {
    Info in{}; in.name = c.str(); in.nd = c.get<uint32_t>();
    if (c.bad || in.nd < 1 || in.nd > 4) { set_error(path + ": malformed tensor table"); return EINVAL_; }
    for (uint32_t d = 0; d < in.nd; d++) in.dims[d] = (int64_t)c.get<uint64_t>();
    in.type = c.get<uint32_t>(); in.off = c.get<uint64_t>();
    if (c.bad) { set_error(path + ": truncated tensor table"); return EINVAL_; }
    sh->infos.push_back(in);
  }
  uint64_t align = sh->kv.count("general.alignment") ? (uint64_t)sh->kv["general.alignment"].num : 32;
  if (align == 0 || align > (1u << 20)) align = 32;
  sh->base = (c.o + align - 1) / align * align;
  if (sh->base > sh->size) { set_error(path + ": no data section"); return EINVAL_; }
  return OK;
}

// `<base>-NNNNN-of-MMMMM.gguf` -> every shard's path; any other name is a set of one
int shard_paths(const std::string& path, std::vector<std::string>* out) {
  out->clear();
  const size_t n = path.size();
  // suffix layout: '-' 5 digits "-of-" 5 digits ".gguf" = 20 characters
  bool split = n > 20 && path.compare(n - 5, 5, ".gguf") == 0 && path[n - 20] == '-' && path.compare(n - 14, 4, "-of-") == 0;
  for (size_t i = 0; split && i < 5; i++) split = isdigit((unsigned char)path[n - 19 + i]) && isdigit((unsigned char)path[n - 10 + i]);
  if (!split) { out->push_back(path); return OK; }
  const int count = atoi(path.substr(n - 10, 5).c_str());
  if (count < 1) { set_error(path + ": unreadable shard count"); return EINVAL_; }
  const std::string stem = path.substr(0, n - 20);
  for (int i = 1; i <= count; i++) {
    char suf[32];
    snprintf(suf, sizeof suf, "-%05d-of-%05d.gguf", i, count);
    std::string sp = stem + suf;
    struct stat sb;
    if (stat(sp.c_str(), &sb) != 0) { set_error(path + ": shard " + std::to_string(i) + " of " + std::to_string(count) + " is missing"); return EIO_; }
    out->push_back(sp);
  }
  return OK;
}

}  // namespace

int load_gguf_into(const char* path, int device, Model* m) {
  std::vector<std::string> paths;
  B200_TRY(shard_paths(path, &paths));
  std::vector<Shard> shards(paths.size());
  size_t n_tensors = 0;
  for (size_t i = 0; i < paths.size(); i++) { B200_TRY(open_shard(paths[i], &shards[i])); n_tensors += shards[i].infos.size(); }
  // the shards must form one whole checkpoint (gguf/gguf.go:795-818)
  std::map<std::string, Value>& kv = shards[0].kv;
  if (shards.size() == 1) {
    if (kv.count("split.count") && kv["split.count"].num > 1) { set_error(paths[0] + " is one shard of " + std::to_string((int)kv["split.count"].num) + " but is not named like one"); return EINVAL_; }
  } else {
    for (size_t i = 0; i < shards.size(); i++) {
      auto& k = shards[i].kv;
      if (!k.count("split.no")) { set_error(paths[i] + " has no split.no"); return EINVAL_; }
      if ((size_t)k["split.no"].num != i) { set_error(paths[i] + ": split.no is " + std::to_string((int)k["split.no"].num) + ", expected " + std::to_string(i)); return EINVAL_; }
      if (k.count("split.count") && (size_t)k["split.count"].num != shards.size()) { set_error(paths[i] + ": split.count disagrees with the number of shards opened"); return EINVAL_; }
    }
    if (kv.count("split.tensors.count") && (size_t)kv["split.tensors.count"].num != n_tensors) { set_error(paths[0] + ": split.tensors.count disagrees with the tensors read"); return EINVAL_; }
  }
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
  for (const Shard& sh : shards)
    for (const Info& in : sh.infos)
      if (in.name == "token_embd.weight" && in.nd > 1 && in.dims[1] > 0 && in.dims[1] < ((int64_t)1 << 31)) cfg.vocab = (int)in.dims[1];  // llm/model.go:91-93
  m->c = cfg; m->device = device;
  for (const Shard& sh : shards) {
    for (const Info& in : sh.infos) {
      // sizes come from the file: nothing is multiplied or added without an overflow check
      int64_t rows = 1, nbytes = 0;
      for (uint32_t d = 0; d < in.nd; d++) {
        if (in.dims[d] <= 0 || in.dims[d] > ((int64_t)1 << 40)) { set_error(in.name + ": dimension out of range"); return EINVAL_; }
        if (d > 0 && __builtin_mul_overflow(rows, in.dims[d], &rows)) { set_error(in.name + ": element count overflows"); return EINVAL_; }
      }
      const int64_t rb = gguf_row_bytes(in.type, in.dims[0]);
      if (rb < 0) { set_error(in.name + ": unsupported ggml type " + std::to_string(in.type)); return EINVAL_; }
      if (__builtin_mul_overflow(rb, rows, &nbytes)) { set_error(in.name + ": tensor size overflows"); return EINVAL_; }
      const uint64_t room = (uint64_t)sh.size - sh.base;
      if (in.off > room || (uint64_t)nbytes > room - in.off) { set_error(in.name + ": data runs past the end of " + sh.path); return EINVAL_; }
      if (m->tensors.count(in.name)) { set_error(in.name + " appears in more than one shard"); return EINVAL_; }
      B200_TRY(m->add_host(in.name, in.type, in.nd, in.dims, sh.bytes() + sh.base + in.off));
    }
  }
  return m->finalize();
}

}  // namespace b200
