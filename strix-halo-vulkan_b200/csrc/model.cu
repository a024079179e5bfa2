// Checkpoint container: uploads GGUF tensors (re-laying Q6_K / Q8_0 rows), resolves the
// per-layer view and validates shapes before anything is launched.
#include "model.h"

#include "kernels.cuh"

namespace b200 {

static thread_local std::string g_err;
void set_error(const std::string& s) { g_err = s; }
const char* last_error() { return g_err.c_str(); }

int sm_count_current() {
  static std::atomic<int> cache[MAX_DEVICES];
  const int slot = current_device_slot();
  int n = cache[slot].load(std::memory_order_acquire);
  if (n > 0) return n;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || n <= 0) { set_error(std::string("cannot read the SM count: ") + cudaGetErrorString(e)); return 0; }
  cache[slot].store(n, std::memory_order_release);
  return n;
}

Model::~Model() {
  cudaSetDevice(device);
  for (void* p : allocs) cudaFree(p);
}

int Model::alloc_tensor(const std::string& name, uint32_t type, uint32_t n_dims, const int64_t* d, DTensor* out) {
  if (finalized) { set_error("model already finalized"); return ESTATE; }
  if (n_dims < 1 || n_dims > 4) { set_error(name + ": 1..4 dims expected"); return EINVAL_; }
  if (tensors.count(name)) { set_error(name + ": tensor added twice"); return EINVAL_; }
  // dims come from an untrusted file: every product is checked before it is used as a size
  int64_t k = d[0], rows = 1;
  for (uint32_t i = 0; i < n_dims; i++) {
    if (d[i] <= 0 || d[i] > ((int64_t)1 << 40)) { set_error(name + ": dimension out of range"); return EINVAL_; }
    if (i > 0 && __builtin_mul_overflow(rows, d[i], &rows)) { set_error(name + ": element count overflows"); return EINVAL_; }
  }
  int64_t stride = device_row_stride(type, k), total = 0;
  if (stride < 0 || k <= 0 || rows <= 0) { set_error(name + ": unsupported type or row length"); return EINVAL_; }
  if (__builtin_mul_overflow(stride, rows, &total) || total > ((int64_t)1 << 46)) { set_error(name + ": tensor size overflows"); return EINVAL_; }
  B200_CUDA(cudaSetDevice(device));
  void* p = nullptr;
  B200_CUDA(cudaMalloc(&p, (size_t)(stride * rows) + 256));
  allocs.push_back(p);
  DTensor t; t.type = type; t.k = k; t.rows = rows; t.stride = stride; t.data = (uint8_t*)p;
  tensors[name] = t;
  dims[name] = std::vector<int64_t>(d, d + n_dims);
  weight_bytes += gguf_row_bytes(type, k) * rows;
  *out = t;
  return OK;
}

int Model::add_host(const std::string& name, uint32_t type, uint32_t n_dims, const int64_t* d, const void* host) {
  DTensor t;
  B200_TRY(alloc_tensor(name, type, n_dims, d, &t));
  const int64_t nbytes = gguf_row_bytes(type, t.k) * t.rows;
  if (type == T_Q6_K || type == T_Q8_0) {
    void* tmp = nullptr;
    B200_CUDA(cudaMalloc(&tmp, (size_t)nbytes));
    cudaError_t e = cudaMemcpy(tmp, host, (size_t)nbytes, cudaMemcpyHostToDevice);
    int s = e == cudaSuccess ? repack_rows(type, t.k, t.rows, (const uint8_t*)tmp, t.data, 0) : ECUDA;
    if (s == OK) e = cudaDeviceSynchronize();
    cudaFree(tmp);
    if (e != cudaSuccess) { set_error(name + ": upload failed: " + cudaGetErrorString(e)); return ECUDA; }
    return s;
  }
  B200_CUDA(cudaMemcpy(t.data, host, (size_t)nbytes, cudaMemcpyHostToDevice));
  return OK;
}

int Model::add_synthetic(const std::string& name, uint32_t type, uint32_t n_dims, const int64_t* d, uint64_t seed, int rule, float p0, float p1) {
  DTensor t;
  B200_TRY(alloc_tensor(name, type, n_dims, d, &t));
  // generate and quantise in slabs of rows so the f32 staging stays small
  const int64_t slab_rows = std::max<int64_t>(1, (int64_t)(64 << 20) / t.k);
  float* f = nullptr; uint8_t* q = nullptr;
  const int64_t rb = gguf_row_bytes(type, t.k);
  B200_CUDA(cudaMalloc(&f, (size_t)(slab_rows * t.k) * sizeof(float)));
  cudaError_t e = cudaMalloc(&q, (size_t)(slab_rows * rb));
  if (e != cudaSuccess) { cudaFree(f); set_error("synthetic: out of memory"); return ENOMEM_; }
  int s = OK;
  for (int64_t r0 = 0; r0 < t.rows && s == OK; r0 += slab_rows) {
    const int64_t nr = std::min(slab_rows, t.rows - r0);
    s = synth_fill(f, nr * t.k, seed + (uint64_t)r0 * 0x9E3779B97F4A7C15ull, rule, p0, p1, 0);
    if (s == OK) s = quantize_rows_device(type, f, nr, t.k, q, 0);
    if (s == OK) s = repack_rows(type, t.k, nr, q, t.data + r0 * t.stride, 0);
  }
  e = cudaDeviceSynchronize();
  cudaFree(f); cudaFree(q);
  if (s == OK && e != cudaSuccess) { set_error(name + ": synthetic generation failed: " + cudaGetErrorString(e)); return ECUDA; }
  return s;
}

int Model::read_tensor(const std::string& name, void* dst, int64_t nbytes) const {
  auto it = tensors.find(name);
  if (it == tensors.end()) { set_error(name + ": no such tensor"); return EINVAL_; }
  const DTensor& t = it->second;
  const int64_t want = gguf_row_bytes(t.type, t.k) * t.rows;
  if (nbytes != want) { set_error(name + ": buffer size does not match the tensor"); return EINVAL_; }
  B200_CUDA(cudaSetDevice(device));
  void* tmp = nullptr;
  B200_CUDA(cudaMalloc(&tmp, (size_t)want));
  int s = unpack_rows(t.type, t.k, t.rows, t.data, (uint8_t*)tmp, 0);
  cudaError_t e = cudaMemcpy(dst, tmp, (size_t)want, cudaMemcpyDeviceToHost);
  cudaFree(tmp);
  if (s == OK && e != cudaSuccess) { set_error(std::string("read_tensor: ") + cudaGetErrorString(e)); return ECUDA; }
  return s;
}

static bool fused_type(uint32_t t) { return t == T_Q4_K || t == T_Q5_K || t == T_Q6_K; }

int Model::finalize() {
  if (finalized) return OK;
  std::string missing, bad;
  auto get = [&](const std::string& n, DTensor* t, bool required = true) {
    auto it = tensors.find(n + ".weight");
    if (it == tensors.end()) it = tensors.find(n);
    if (it == tensors.end()) { if (required) missing += " " + n; return false; }
    *t = it->second;
    return true;
  };
  auto want = [&](const std::string& n, const DTensor& t, int64_t k, int64_t rows, int kind) {
    // kind 0: F32 vector/matrix, 1: fused projection (K-quant), 2: any dequantisable matrix
    if (!t.ok()) return;
    if (t.k != k || t.rows != rows) bad += " " + n + "[" + std::to_string(t.k) + "x" + std::to_string(t.rows) + " want " + std::to_string(k) + "x" + std::to_string(rows) + "]";
    else if (kind == 0 && t.type != T_F32) bad += " " + n + "(must be F32)";
    else if (kind == 1 && !fused_type(t.type)) bad += " " + n + "(must be Q4_K, Q5_K or Q6_K)";
    else if (kind == 1 && rows % 16) bad += " " + n + "(rows must be a multiple of 16)";
  };
  const int H = c.n_embd;
  get("token_embd", &token_embd);
  if (!get("output", &output, false)) output = token_embd;
  get("output_norm", &output_norm);
  want("token_embd", token_embd, H, c.vocab, 2);
  want("output", output, H, c.vocab, 1);
  want("output_norm", output_norm, H, 1, 0);
  const int nl = c.n_layer + (c.has_draft ? 1 : 0);
  layers.assign(nl, LayerW());
  const int D = c.dn_head_dim, qk = c.dn_heads_k * D, vw = c.dn_heads_v * D, cw = 2 * qk + vw;
  const int hd = c.head_dim, qw = c.n_head * hd, kvw = c.n_head_kv * hd;
  for (int l = 0; l < nl; l++) {
    LayerW& L = layers[l];
    const std::string p = "blk." + std::to_string(l) + ".";
    L.is_attn = tensors.count(p + "attn_q.weight") > 0;  // reference: llm/model.go:377, :443
    get(p + "attn_norm", &L.attn_norm); get(p + "ffn_norm", &L.ffn_norm);
    want(p + "attn_norm", L.attn_norm, H, 1, 0); want(p + "ffn_norm", L.ffn_norm, H, 1, 0);
    if (L.is_attn) {
      get(p + "attn_q", &L.q); get(p + "attn_k", &L.k); get(p + "attn_v", &L.v); get(p + "attn_output", &L.o);
      get(p + "attn_q_norm", &L.q_norm); get(p + "attn_k_norm", &L.k_norm);
      want(p + "attn_q", L.q, H, 2 * qw, 1); want(p + "attn_k", L.k, H, kvw, 1); want(p + "attn_v", L.v, H, kvw, 1);
      want(p + "attn_output", L.o, qw, H, 1);
      want(p + "attn_q_norm", L.q_norm, hd, 1, 0); want(p + "attn_k_norm", L.k_norm, hd, 1, 0);
    } else {
      get(p + "attn_qkv", &L.qkv); get(p + "attn_gate", &L.z); get(p + "ssm_alpha", &L.alpha); get(p + "ssm_beta", &L.beta);
      get(p + "ssm_conv1d", &L.conv1d); get(p + "ssm_a", &L.ssm_a); get(p + "ssm_dt.bias", &L.dt_bias);
      get(p + "ssm_norm", &L.ssm_norm); get(p + "ssm_out", &L.ssm_out);
      want(p + "attn_qkv", L.qkv, H, cw, 1); want(p + "attn_gate", L.z, H, vw, 1);
      want(p + "ssm_alpha", L.alpha, H, c.dn_heads_v, 0); want(p + "ssm_beta", L.beta, H, c.dn_heads_v, 0);
      want(p + "ssm_conv1d", L.conv1d, c.dn_conv, cw, 0); want(p + "ssm_a", L.ssm_a, c.dn_heads_v, 1, 0);
      want(p + "ssm_dt.bias", L.dt_bias, c.dn_heads_v, 1, 0); want(p + "ssm_norm", L.ssm_norm, D, 1, 0);
      want(p + "ssm_out", L.ssm_out, vw, H, 1);
      if (L.qkv.ok() && L.z.ok() && L.qkv.type != L.z.type) bad += " " + p + "attn_gate(type must match attn_qkv)";
    }
    get(p + "ffn_gate_inp", &L.router); get(p + "ffn_gate_inp_shexp", &L.sh_gate_inp);
    get(p + "ffn_gate_exps", &L.gate_exps); get(p + "ffn_up_exps", &L.up_exps); get(p + "ffn_down_exps", &L.down_exps);
    get(p + "ffn_gate_shexp", &L.gate_sh); get(p + "ffn_up_shexp", &L.up_sh); get(p + "ffn_down_shexp", &L.down_sh);
    want(p + "ffn_gate_inp", L.router, H, c.n_expert, 2); want(p + "ffn_gate_inp_shexp", L.sh_gate_inp, H, 1, 0);
    want(p + "ffn_gate_exps", L.gate_exps, H, (int64_t)c.ffn_expert * c.n_expert, 1);
    want(p + "ffn_up_exps", L.up_exps, H, (int64_t)c.ffn_expert * c.n_expert, 1);
    want(p + "ffn_down_exps", L.down_exps, c.ffn_expert, (int64_t)H * c.n_expert, 1);
    want(p + "ffn_gate_shexp", L.gate_sh, H, c.ffn_shared, 1); want(p + "ffn_up_shexp", L.up_sh, H, c.ffn_shared, 1);
    want(p + "ffn_down_shexp", L.down_sh, c.ffn_shared, H, 1);
    if (L.gate_exps.ok() && L.up_exps.ok() && L.gate_sh.ok() && L.up_sh.ok() &&
        (L.gate_exps.type != L.up_exps.type || L.gate_sh.type != L.gate_exps.type || L.up_sh.type != L.gate_exps.type))
      bad += " " + p + "ffn_{gate,up}_{exps,shexp}(must share one type)";
    if (L.down_exps.ok() && L.down_sh.ok() && L.down_exps.type != L.down_sh.type) bad += " " + p + "ffn_down_shexp(type must match ffn_down_exps)";
    if (l == c.n_layer) {
      get(p + "nextn.enorm", &L.enorm); get(p + "nextn.hnorm", &L.hnorm); get(p + "nextn.eh_proj", &L.eh_proj);
      get(p + "nextn.shared_head_norm", &L.head_norm);
      want(p + "nextn.enorm", L.enorm, H, 1, 0); want(p + "nextn.hnorm", L.hnorm, H, 1, 0);
      want(p + "nextn.eh_proj", L.eh_proj, 2 * H, H, 1); want(p + "nextn.shared_head_norm", L.head_norm, H, 1, 0);
      if (!L.is_attn) bad += " " + p + "(the draft layer must be an attention layer)";
    }
  }
  if (c.ffn_shared != c.ffn_expert) bad += " ffn_shared(must equal ffn_expert: the shared expert runs as one more tile of the expert kernel)";
  if (c.dn_head_dim != 128 || c.dn_conv != 4) bad += " ssm(state_size must be 128 and conv_kernel 4)";
  if (c.dn_heads_k <= 0 || c.dn_heads_v % c.dn_heads_k) bad += " ssm(time_step_rank must be a multiple of group_count: V head h reads K head h % group_count, llm/deltanet.go:405-418)";
  if (c.n_head_kv <= 0 || c.n_head % c.n_head_kv) bad += " attention(head_count must be a multiple of head_count_kv)";
  if (H % 256) bad += " embedding_length(must be a multiple of 256)";
  if (c.n_expert > 1024 || c.n_expert_used > 32 || c.n_expert_used > c.n_expert) bad += " experts(at most 1024 experts, 32 used)";
  if (!missing.empty()) { set_error("checkpoint is missing tensors:" + missing); return EINVAL_; }
  if (!bad.empty()) { set_error("checkpoint tensors refused:" + bad); return EINVAL_; }
  finalized = true;
  return OK;
}

}  // namespace b200
