// extern "C" surface of libb200llm.so (include/b200_llm.h).
#include <cstring>
#include <new>
#include <vector>

#include "graph.h"

using namespace b200;

struct b200_model { Model m; };
struct b200_graph { Graph g; };

namespace {
struct Scratch {   // device temporaries of one call
  std::vector<void*> ptrs;
  ~Scratch() { for (void* p : ptrs) cudaFree(p); }
  template <class T> int get(T** out, size_t bytes) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess) { set_error(std::string("device allocation of ") + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e)); return ENOMEM_; }
    ptrs.push_back(p);
    *out = (T*)p;
    return OK;
  }
};
}  // namespace

extern "C" {

const char* b200_last_error(void) { return last_error(); }

int32_t b200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

int32_t b200_model_new(const b200_config* cfg, int32_t device, b200_model** out) {
  if (!cfg || !out) { set_error("model_new: null argument"); return EINVAL_; }
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { set_error("no CUDA device: this library has no CPU path"); return ECUDA; }
  if (device < 0 || device >= n) { set_error("model_new: no such device"); return EINVAL_; }
  auto* m = new (std::nothrow) b200_model();
  if (!m) return ENOMEM_;
  m->m.c = *cfg; m->m.device = device;
  *out = m;
  return OK;
}
int32_t b200_model_add_tensor(b200_model* m, const char* name, uint32_t type, uint32_t n_dims, const int64_t* dims, const void* host) {
  if (!m || !name || !dims || !host) { set_error("add_tensor: null argument"); return EINVAL_; }
  return m->m.add_host(name, type, n_dims, dims, host);
}
int32_t b200_model_add_synthetic(b200_model* m, const char* name, uint32_t type, uint32_t n_dims, const int64_t* dims, uint64_t seed, int32_t rule, float p0, float p1) {
  if (!m || !name || !dims) { set_error("add_synthetic: null argument"); return EINVAL_; }
  return m->m.add_synthetic(name, type, n_dims, dims, seed, rule, p0, p1);
}
int32_t b200_model_finalize(b200_model* m) { if (!m) { set_error("null model"); return EINVAL_; } return m->m.finalize(); }
int32_t b200_model_open_gguf(const char* path, int32_t device, b200_model** out) {
  if (!path || !out) { set_error("open_gguf: null argument"); return EINVAL_; }
  auto* bm = new (std::nothrow) b200_model();
  if (!bm) return ENOMEM_;
  int s = load_gguf_into(path, device, &bm->m);
  if (s != OK) { delete bm; return s; }
  *out = bm;
  return OK;
}
int32_t b200_model_config(const b200_model* m, b200_config* out) { if (!m || !out) return EINVAL_; *out = m->m.c; return OK; }
int64_t b200_model_weight_bytes(const b200_model* m) { return m ? m->m.weight_bytes : 0; }
int64_t b200_model_tensor_bytes(const b200_model* m, const char* name) {
  if (!m || !name) return -1;
  auto it = m->m.tensors.find(name);
  if (it == m->m.tensors.end()) return -1;
  return gguf_row_bytes(it->second.type, it->second.k) * it->second.rows;
}
int32_t b200_model_read_tensor(const b200_model* m, const char* name, void* dst, int64_t nbytes) {
  if (!m || !name || !dst) { set_error("read_tensor: null argument"); return EINVAL_; }
  return m->m.read_tensor(name, dst, nbytes);
}
void b200_model_free(b200_model* m) { delete m; }

int32_t b200_graph_create(b200_model* m, const b200_graph_opts* opts, b200_graph** out) {
  if (!m || !opts || !out) { set_error("graph_create: null argument"); return EINVAL_; }
  auto* g = new (std::nothrow) b200_graph();
  if (!g) return ENOMEM_;
  int s = g->g.init(&m->m, *opts);
  if (s != OK) { delete g; return s; }
  *out = g;
  return OK;
}
void b200_graph_destroy(b200_graph* g) { delete g; }
int32_t b200_graph_slots(const b200_graph* g) { return g ? g->g.o.slots : 0; }
int32_t b200_graph_nkv(const b200_graph* g) { return g ? g->g.o.n_kv : 0; }
int32_t b200_graph_use_slot(b200_graph* g, int32_t slot) {
  if (!g) return EINVAL_;
  if (slot < 0 || slot >= g->g.o.slots) { set_error("use_slot: slot " + std::to_string(slot) + " does not exist"); return EINVAL_; }
  g->g.cur = slot; g->g.dcur = slot; g->g.spec_n = 0;
  return OK;
}
int32_t b200_graph_reset(b200_graph* g) { if (!g) return EINVAL_; return g->g.reset_slot(g->g.cur); }
int32_t b200_graph_set_past(b200_graph* g, int32_t past) {
  if (!g) return EINVAL_;
  if (past < 0 || past > g->g.o.n_kv) { set_error("set_past: position outside the slot's context"); return EINVAL_; }
  g->g.past[g->g.cur] = past; g->g.spec_n = 0;
  return OK;
}
int32_t b200_graph_past(const b200_graph* g) { return g ? g->g.past[g->g.cur] : 0; }

int32_t b200_graph_forward(b200_graph* g, const int32_t* ids, int32_t n, const float** logits, const float** hidden) {
  if (!g || !ids) { set_error("forward: null argument"); return EINVAL_; }
  B200_TRY(g->g.reset_slot(g->g.cur));
  PassFlags f;
  return g->g.extend(ids, n, f, logits, hidden);
}
int32_t b200_graph_extend(b200_graph* g, const int32_t* ids, int32_t n, const float** logits, const float** hidden) {
  if (!g || !ids) { set_error("extend: null argument"); return EINVAL_; }
  PassFlags f;
  return g->g.extend(ids, n, f, logits, hidden);
}
int32_t b200_graph_extend_input(b200_graph* g, const b200_input* in, const float** logits, const float** hidden) {
  if (!g || !in || !in->ids) { set_error("extend_input: null argument"); return EINVAL_; }
  if (in->n_images != 0) { set_error("extend_input: this library has no vision tower; inputs with images are refused"); return EINVAL_; }
  PassFlags f;
  return g->g.extend(in->ids, in->n, f, logits, hidden);
}
int32_t b200_graph_extend_rows(b200_graph* g, const int32_t* ids, int32_t n, const float** logits, const float** residual) {
  if (!g || !ids) { set_error("extend_rows: null argument"); return EINVAL_; }
  PassFlags f; f.want_all_logits = true; f.want_residual = true; f.spec = g->g.speculating;
  return g->g.extend(ids, n, f, logits, residual);
}
int32_t b200_graph_extend_residual(b200_graph* g, const int32_t* ids, int32_t n, const float** logits, const float** residual) {
  if (!g || !ids) { set_error("extend_residual: null argument"); return EINVAL_; }
  PassFlags f; f.want_residual = true;
  return g->g.extend(ids, n, f, logits, residual);
}
int32_t b200_graph_decode_rows(b200_graph* g, const int32_t* slots, const int32_t* ids, int32_t n, const float** logits) {
  if (!g || !slots || !ids) { set_error("decode_rows: null argument"); return EINVAL_; }
  return g->g.decode_rows(slots, ids, n, logits);
}
int32_t b200_graph_checkpoint(b200_graph* g, int32_t* handle) { if (!g || !handle) return EINVAL_; return g->g.checkpoint(handle); }
int32_t b200_graph_restore(b200_graph* g, int32_t handle) { if (!g) return EINVAL_; return g->g.restore(handle); }
int32_t b200_graph_checkpoint_free(b200_graph* g, int32_t handle) {
  if (!g) return EINVAL_;
  auto it = g->g.ckpts.find(handle);
  if (it == g->g.ckpts.end()) { set_error("checkpoint_free: unknown checkpoint"); return EINVAL_; }
  cudaSetDevice(g->g.m->device);
  for (float* p : it->second.state) cudaFree(p);
  for (float* p : it->second.ring) cudaFree(p);
  g->g.ckpts.erase(it);
  return OK;
}
int32_t b200_graph_speculate(b200_graph* g, int32_t on) {
  if (!g) return EINVAL_;
  if (on && !g->g.o.speculative) { set_error("speculate: the graph was created with speculative = 0"); return ESTATE; }
  g->g.speculating = on != 0;
  return OK;
}
int32_t b200_graph_speculating(const b200_graph* g) { return g && g->g.speculating ? 1 : 0; }
int32_t b200_graph_speculate_first(b200_graph* g, int32_t on) {
  if (!g) return EINVAL_;
  if (g->g.spec_n > 0) { set_error("speculate_first: a speculative pass is in flight; commit or rewind it first"); return ESTATE; }
  g->g.spec_first = on != 0;
  return OK;
}
int32_t b200_graph_keep(b200_graph* g, int32_t k) { if (!g) return EINVAL_; return g->g.keep(k); }
int32_t b200_graph_keep_first(b200_graph* g) { if (!g) return EINVAL_; return g->g.keep(1); }
int32_t b200_graph_commit(b200_graph* g) { if (!g) return EINVAL_; return g->g.keep(g->g.spec_n); }
int32_t b200_graph_rewind(b200_graph* g) {
  if (!g) return EINVAL_;
  // with SpeculateFirst on, row 0 of a pass is a token already emitted: the pass ends by Commit or KeepFirst (llm/graph.go:1166-1178)
  if (g->g.spec_first && g->g.spec_n > 0) { set_error("rewind: with speculate_first on a pass is ended by commit or keep_first"); return ESTATE; }
  return g->g.keep(0);
}
int32_t b200_graph_residual_row(b200_graph* g, int32_t r, float* dst) { if (!g || !dst) { set_error("residual_row: null argument"); return EINVAL_; } return g->g.residual_row(r, dst); }
int32_t b200_graph_pass_experts(b200_graph* g, int32_t* out) { if (!g || !out) { set_error("pass_experts: null argument"); return EINVAL_; } return g->g.pass_experts(out); }
uint32_t b200_graph_fp16_weight_mask(const b200_graph* g, int32_t rows, int32_t logit_rows) { return g ? g->g.fp16_weight_mask(rows, logit_rows) : 0; }
int32_t b200_graph_stats_get(const b200_graph* g, b200_graph_stats* out) {
  if (!g || !out) return EINVAL_;
  *out = g->g.stats;
  int64_t dev = 0;
  cudaSetDevice(g->g.m->device);
  if (cudaMemcpy(&dev, g->g.distinct_dev, sizeof(dev), cudaMemcpyDeviceToHost) != cudaSuccess) { set_error("stats: cannot read the device counter"); return ECUDA; }
  out->expert_streams = dev + g->g.single_row_layers * g->g.m->c.n_expert_used;
  return OK;
}
int32_t b200_graph_stats_reset(b200_graph* g) {
  if (!g) return EINVAL_;
  g->g.stats = b200_graph_stats{}; g->g.single_row_layers = 0;
  cudaSetDevice(g->g.m->device);
  if (cudaMemset(g->g.distinct_dev, 0, sizeof(int64_t)) != cudaSuccess) { set_error("stats: cannot clear the device counter"); return ECUDA; }
  return OK;
}
int32_t b200_graph_ep_export(b200_graph* g, int32_t rank, int32_t world, b200_ep_handle* out) { if (!g || !out) return EINVAL_; return g->g.ep_export(rank, world, out->bytes); }
int32_t b200_graph_ep_attach(b200_graph* g, const b200_ep_handle* handles) { if (!g || !handles) return EINVAL_; return g->g.ep_attach(handles); }
int32_t b200_graph_ep_prepare(b200_graph* g, int32_t rank, int32_t world) { if (!g) return EINVAL_; return g->g.ep_prepare(rank, world); }
int32_t b200_graph_ep_attach_local(b200_graph* g, b200_graph* const* graphs, int32_t world) {
  if (!g || !graphs || world < 1 || world > EP_MAX_RANKS) { set_error("ep_attach_local: bad argument"); return EINVAL_; }
  Graph* peers[EP_MAX_RANKS] = {};
  for (int i = 0; i < world; i++) peers[i] = graphs[i] ? &graphs[i]->g : nullptr;
  return g->g.ep_attach_local(peers, world);
}
int32_t b200_graph_ep_enable(b200_graph* g, int32_t on) {
  if (!g) return EINVAL_;
  if (on && !g->g.ep_ready) { set_error("ep_enable: attach the peers first"); return ESTATE; }
  g->g.ep_on = on != 0;
  return OK;
}
int32_t b200_graph_synth_context(b200_graph* g, int32_t cells, uint64_t seed) { if (!g) return EINVAL_; return g->g.synth_context(g->g.cur, cells, seed); }
int32_t b200_graph_inject_wait_timeout(b200_graph* g) { if (!g) return EINVAL_; return g->g.inject_wait_timeout(); }

int32_t b200_graph_generate_greedy(b200_graph* g, const int32_t* slots, const int32_t* first_ids, int32_t n, int32_t steps, int32_t* out_ids) {
  if (!g || !slots || !first_ids || !out_ids) { set_error("generate_greedy: null argument"); return EINVAL_; }
  return g->g.generate_greedy(slots, first_ids, n, steps, out_ids);
}
float b200_graph_last_device_ms(const b200_graph* g) { return g ? g->g.last_ms : 0.f; }
int32_t b200_graph_last_launches(const b200_graph* g) { return g ? g->g.last_launches : 0; }
int32_t b200_graph_timeline(b200_graph* g, int64_t* dst, int32_t max_launches) {
  if (!g || !dst) return -1;
  if (!g->g.timeline) return 0;
  cudaSetDevice(g->g.m->device);
  int n = g->g.last_launches < g->g.timeline_cap ? g->g.last_launches : g->g.timeline_cap;
  if (n > max_launches) n = max_launches;
  if (cudaMemcpy(dst, g->g.timeline, (size_t)n * 8 * sizeof(long long), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return n;
}
int64_t b200_graph_trace(b200_graph* g, int32_t what, void* dst, int64_t nbytes) { if (!g || !dst) return -EINVAL_; return g->g.trace(what, dst, nbytes); }

int32_t b200_draft_rows(b200_graph* g, const float* hs, const int32_t* ids, int32_t n, int32_t vocab_k, const float** residual, const float** logits) {
  if (!g || !hs || !ids) { set_error("draft_rows: null argument"); return EINVAL_; }
  return g->g.draft_rows(hs, ids, n, vocab_k, residual, logits);
}
int32_t b200_draft_past(const b200_graph* g) { return g ? g->g.draft_past[g->g.dcur] : 0; }
int32_t b200_draft_rewind(b200_graph* g, int32_t past) {
  if (!g) return EINVAL_;
  if (past < 0 || past > g->g.draft_past[g->g.dcur]) { set_error("draft_rewind: position outside the draft cache"); return EINVAL_; }
  g->g.draft_past[g->g.dcur] = past;
  return OK;
}
int32_t b200_draft_set_vocab(b200_graph* g, int32_t k) {
  if (!g) return EINVAL_;
  if (k < 0 || k % 16 || k > g->g.m->c.vocab) { set_error("draft_set_vocab: a multiple of 16 up to the vocabulary size, or 0 for all of it"); return EINVAL_; }
  g->g.draft_vocab_default = k == g->g.m->c.vocab ? 0 : k;
  return OK;
}
int32_t b200_draft_use_slot(b200_graph* g, int32_t slot) {
  if (!g) return EINVAL_;
  if (slot < 0 || slot >= g->g.o.slots) { set_error("draft_use_slot: draft cache slot " + std::to_string(slot) + " of " + std::to_string(g->g.o.slots)); return EINVAL_; }
  g->g.dcur = slot;
  return OK;
}
int32_t b200_draft_slots(const b200_graph* g) { return g && g->g.m->c.has_draft ? g->g.o.slots : 0; }
int32_t b200_draft_reset(b200_graph* g) { if (!g) return EINVAL_; g->g.draft_past[g->g.dcur] = 0; return OK; }
int32_t b200_draft_max_rows(const b200_graph* g) { return g ? g->g.LR : 0; }
int32_t b200_draft_wide(const b200_graph* g) { return g ? g->g.m->c.n_embd : 0; }

// ---- unit entry points --------------------------------------------------------------------
// They run on the device that is current in the calling thread and free what they allocate on
// every path out.
static int need_device() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { set_error("no CUDA device: this library has no CPU path"); return ECUDA; }
  return OK;
}


int32_t b200_dequantize(uint32_t type, const void* host_data, int64_t n, float* host_out) {
  B200_TRY(need_device());
  int e, nb;
  if (!host_data || !host_out || !block_geometry(type, &e, &nb) || n % e || n <= 0) { set_error("dequantize: bad type or element count"); return EINVAL_; }
  const int64_t bytes = gguf_row_bytes(type, n);
  DTensor t; t.type = type; t.k = n; t.rows = 1; t.stride = device_row_stride(type, n);
  Scratch sc;
  uint8_t* src = nullptr; float* out = nullptr;
  B200_TRY(sc.get(&src, (size_t)bytes)); B200_TRY(sc.get(&t.data, (size_t)t.stride + 256)); B200_TRY(sc.get(&out, (size_t)n * sizeof(float)));
  B200_CUDA(cudaMemcpy(src, host_data, (size_t)bytes, cudaMemcpyHostToDevice));
  B200_TRY(repack_rows(type, n, 1, src, t.data, 0));
  B200_TRY(dequant_rows(t, 0, 1, out, 0));
  B200_CUDA(cudaMemcpy(host_out, out, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
  return OK;
}

// weights in device layout, activations as fp16 rows, an error word: what both projection entry points stage
static int stage_projection(Scratch& sc, uint32_t type, const void* host_w, int64_t rows, int64_t k, const float* host_x, int32_t mrows,
                            DTensor* t, __half** x16, float** y, int** err) {
  const int64_t rb = gguf_row_bytes(type, k);
  if (rb < 0) { set_error("projection: bad type or row length"); return EINVAL_; }
  t->type = type; t->k = k; t->rows = rows; t->stride = device_row_stride(type, k);
  uint8_t* src = nullptr; float* xf = nullptr;
  B200_TRY(sc.get(&src, (size_t)(rb * rows))); B200_TRY(sc.get(&t->data, (size_t)(t->stride * rows) + 256));
  B200_TRY(sc.get(&xf, (size_t)mrows * k * sizeof(float))); B200_TRY(sc.get(x16, (size_t)mrows * k * sizeof(__half)));
  B200_TRY(sc.get(y, (size_t)mrows * rows * sizeof(float))); B200_TRY(sc.get(err, sizeof(int)));
  B200_CUDA(cudaMemset(*err, 0, sizeof(int)));
  B200_CUDA(cudaMemcpy(src, host_w, (size_t)(rb * rows), cudaMemcpyHostToDevice));
  B200_CUDA(cudaMemcpy(xf, host_x, (size_t)mrows * k * sizeof(float), cudaMemcpyHostToDevice));
  B200_TRY(repack_rows(type, k, rows, src, t->data, 0));
  B200_TRY(quantize_rows_device(T_F16, xf, mrows, k, (uint8_t*)*x16, 0));
  return OK;
}
static int finish_projection(const char* who, const float* y, const int* err, int64_t n, float* host_y) {
  int herr = 0;
  B200_CUDA(cudaMemcpy(&herr, err, sizeof(int), cudaMemcpyDeviceToHost));
  if (herr != 0) { set_error(std::string(who) + ": a bounded wait gave up"); return ETIMEOUT; }
  B200_CUDA(cudaMemcpy(host_y, y, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
  return OK;
}

int32_t b200_qgemv(uint32_t type, const void* host_w, int64_t rows, int64_t k, const float* host_x, int32_t mrows, float* host_y) {
  B200_TRY(need_device());
  if (!host_w || !host_x || !host_y || rows <= 0 || mrows <= 0) { set_error("qgemv: bad argument"); return EINVAL_; }
  Scratch sc; DTensor t; __half* x16 = nullptr; float* y = nullptr; int* err = nullptr;
  B200_TRY(stage_projection(sc, type, host_w, rows, k, host_x, mrows, &t, &x16, &y, &err));
  QGemvParams p{};
  p.w[0] = t.data; p.seg_end[0] = (int)rows; p.nseg = 1; p.stride = t.stride; p.K = (int)k; p.N = (int)rows; p.M = mrows; p.xcols = mrows < QG_MAXCOLS ? mrows : QG_MAXCOLS;
  p.x = x16; p.ldx = k; p.y = y; p.ldy = rows; p.x_div = 1; p.err = err;
  B200_TRY(launch_qgemv(type, PRO_F16, EPI_STORE, false, false, p, 0, false, 0));
  return finish_projection("qgemv", y, err, (int64_t)mrows * rows, host_y);
}

int32_t b200_qgemm(uint32_t type, const void* host_w, int64_t rows, int64_t k, const float* host_x, int32_t mrows, int32_t tile_rows, float* host_y) {
  B200_TRY(need_device());
  if (!host_w || !host_x || !host_y || rows <= 0 || mrows <= 0) { set_error("qgemm: bad argument"); return EINVAL_; }
  Scratch sc; DTensor t; __half* x16 = nullptr; float* y = nullptr; int* err = nullptr;
  B200_TRY(stage_projection(sc, type, host_w, rows, k, host_x, mrows, &t, &x16, &y, &err));
  alignas(64) unsigned char tmap[128];
  B200_TRY(make_x_tensor_map(x16, mrows, (int)k, tile_rows, tmap));
  QGemmParams p{};
  p.w = t.data; p.one.expert = 0; p.one.x_row0 = 0; p.one.count = mrows; p.one.y_row0 = 0; p.max_problems = 1; p.max_count = mrows;
  p.stride = t.stride; p.K = (int)k; p.N = (int)rows; p.y = y; p.ldy = rows; p.err = err;
  B200_TRY(launch_qgemm(type, GEMM_STORE, tile_rows, p, tmap, false, 0));
  return finish_projection("qgemm", y, err, (int64_t)mrows * rows, host_y);
}

int32_t b200_qgemv_static(uint32_t type, const void* dev_w, int64_t rows, int64_t k, const float* dev_x, int32_t m, float* dev_y) {
  B200_TRY(need_device());
  return qgemv_static(type, dev_w, rows, k, dev_x, m, dev_y);
}

int32_t b200_quantize(uint32_t type, const float* host_src, int64_t rows, int64_t k, void* host_dst) {
  B200_TRY(need_device());
  const int64_t rb = gguf_row_bytes(type, k);
  if (!host_src || !host_dst || rb < 0 || rows <= 0) { set_error("quantize: bad argument"); return EINVAL_; }
  Scratch sc; float* f = nullptr; uint8_t* q = nullptr;
  B200_TRY(sc.get(&f, (size_t)rows * k * sizeof(float))); B200_TRY(sc.get(&q, (size_t)(rb * rows)));
  B200_CUDA(cudaMemcpy(f, host_src, (size_t)rows * k * sizeof(float), cudaMemcpyHostToDevice));
  B200_TRY(quantize_rows_device(type, f, rows, k, q, 0));
  B200_CUDA(cudaMemcpy(host_dst, q, (size_t)(rb * rows), cudaMemcpyDeviceToHost));
  return OK;
}

}  // extern "C"
