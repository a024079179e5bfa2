// Pass scheduling of the token loop (see graph.h). Layer order follows the reference's
// layers() loop (llm/graph.go:2330-2466) with a plain pre-norm residual stream in place of
// its hyper-connection mixers.
#include "graph.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <set>
#include <cstdlib>
#include <cstring>

namespace b200 {

template <class T>
int Graph::dalloc(T** p, size_t n, bool zero) {
  void* q = nullptr;
  size_t bytes = std::max<size_t>(n, 1) * sizeof(T);
  cudaError_t e = cudaMalloc(&q, bytes);
  if (e != cudaSuccess) { set_error(std::string("graph: device allocation of ") + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e)); return ENOMEM_; }
  if (zero) B200_CUDA(cudaMemset(q, 0, bytes));
  allocs.push_back(q);
  *p = (T*)q;
  return OK;
}

Graph::~Graph() {
  if (m) cudaSetDevice(m->device);
  if (st) cudaStreamSynchronize(st);
  for (auto& kv : decode_graphs) cudaGraphExecDestroy(kv.second);
  for (auto& kv : greedy_graphs) cudaGraphExecDestroy(kv.second);
  for (auto& kv : ckpts) { for (float* p : kv.second.state) cudaFree(p); for (float* p : kv.second.ring) cudaFree(p); }
  for (void* p : ep_mapped) cudaIpcCloseMemHandle(p);
  for (void* p : allocs) cudaFree(p);
  if (stage) cudaFreeHost(stage);
  if (logits_host) cudaFreeHost(logits_host);
  if (resid_host) cudaFreeHost(resid_host);
  if (hidden_host) cudaFreeHost(hidden_host);
  if (err_host) cudaFreeHost(err_host);
  if (ids_host) cudaFreeHost(ids_host);
  if (ev0) cudaEventDestroy(ev0);
  if (ev1) cudaEventDestroy(ev1);
  if (st) cudaStreamDestroy(st);
}

int Graph::init(Model* model, const b200_graph_opts& opts) {
  m = model; o = opts;
  if (!m->finalized) { set_error("graph: model is not finalized"); return ESTATE; }
  const b200_config& c = m->c;
  if (o.max_tokens <= 0) o.max_tokens = 64;
  if (o.slots <= 0) o.slots = 1;
  if (o.n_kv <= 0) { set_error("graph: n_kv must be positive"); return EINVAL_; }
  if (o.speculative && o.spec_rows <= 0) o.spec_rows = 3;
  if (o.spec_rows > DN_RING - 3) { set_error("graph: spec_rows is limited to 5 (the conv ring keeps 8 positions)"); return ECAPACITY; }
  // Rows per pass. Many-row passes of one sequence run the tiled causal attention kernel, which keeps nothing per
  // row; where the head layout has no such kernel, every row goes through the split-KV kernel, whose per-row
  // partial results cap the pass at 2048 rows.
  const int grp = c.n_head_kv > 0 ? c.n_head / c.n_head_kv : 0;
  const bool tiled_attn = (grp == 8 && c.head_dim == 256) || (grp == 4 && c.head_dim == 128);
  MR = std::min(o.max_tokens, tiled_attn ? 4096 : 2048);
  LR = std::min(MR, 512);              // rows whose logits a pass can return
  attn_rows = tiled_attn ? std::min(MR, std::max(std::max(o.slots, 16), o.spec_rows)) : MR;   // rows the split-KV kernel may see
  // a CTA's four warps take 16 cells each per round; longer contexts get longer splits so the merge stays short
  split_cells = o.attn_split_cells > 0 ? (o.attn_split_cells + 15) / 16 * 16 : (o.n_kv <= 4096 ? 64 : o.n_kv <= 8192 ? 128 : o.n_kv <= 16384 ? 256 : 512);
  nsplit = (o.n_kv + split_cells - 1) / split_cells;
  B200_CUDA(cudaSetDevice(m->device));
  B200_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  B200_CUDA(cudaEventCreate(&ev0));
  B200_CUDA(cudaEventCreate(&ev1));
  const int H = c.n_embd, D = c.dn_head_dim, qk = c.dn_heads_k * D, vw = c.dn_heads_v * D, cw = 2 * qk + vw;
  const int hd = c.head_dim, qw = c.n_head * hd, kvw = c.n_head_kv * hd, used = c.n_expert_used, slots1 = used + 1;
  proj_ld = std::max(cw + vw, 2 * qw + 2 * kvw);
  const int nl = (int)m->layers.size();
  dn_index.assign(nl, -1); attn_index.assign(nl, -1);
  for (int l = 0; l < nl; l++) {
    if (m->layers[l].is_attn) attn_index[l] = n_attn++;
    else dn_index[l] = n_dn++;
  }
  max_entries = std::max(max_entries_for(MR), max_entries_for(std::min(MR, 128)));
  B200_TRY(dalloc(&hbuf[0], (size_t)MR * H)); B200_TRY(dalloc(&hbuf[1], (size_t)MR * H)); h = hbuf[0]; B200_TRY(dalloc(&proj, (size_t)MR * proj_ld));
  B200_TRY(dalloc(&xn16, (size_t)MR * H)); B200_TRY(dalloc(&q16, (size_t)MR * qw)); B200_TRY(dalloc(&ctx16, (size_t)MR * qw));
  B200_TRY(dalloc(&attn_partial, (size_t)attn_rows * c.n_head * nsplit * (hd + 2)));
  B200_TRY(dalloc(&r_logits, (size_t)MR * c.n_expert));
  B200_TRY(dalloc(&topk, (size_t)MR * used)); B200_TRY(dalloc(&topk_w, (size_t)MR * slots1)); B200_TRY(dalloc(&margin, (size_t)MR));
  B200_TRY(dalloc(&entries, (size_t)max_entries)); B200_TRY(dalloc(&n_entries, 1)); B200_TRY(dalloc(&cols, (size_t)MR * slots1));
  B200_TRY(dalloc(&r_ticket, (size_t)2 + MR / 8)); B200_TRY(dalloc(&err_flag, 1)); B200_TRY(dalloc(&ss_part, (size_t)MR * SS_LD)); B200_TRY(dalloc(&y16, (size_t)MR * vw));
  B200_TRY(dalloc(&act16, (size_t)MR * slots1 * c.ffn_expert)); B200_TRY(dalloc(&down, (size_t)MR * slots1 * H));
  B200_TRY(dalloc(&logits, (size_t)LR * c.vocab));
  { B200_TRY(dalloc(&dn_pre, (size_t)MR * ((size_t)c.dn_heads_k * 256 + (size_t)c.dn_heads_v * 130))); B200_TRY(dalloc(&dn_oraw, (size_t)MR * vw)); B200_TRY(dalloc(&dn_ab, (size_t)MR * 2 * c.dn_heads_v)); }
  { std::vector<float> one(64, 1.f); B200_TRY(dalloc(&ones, one.size())); B200_CUDA(cudaMemcpy(ones, one.data(), one.size() * sizeof(float), cudaMemcpyHostToDevice)); }
  B200_TRY(dalloc(&xperm16, (size_t)MR * used * H)); B200_TRY(dalloc(&gprob, (size_t)c.n_expert)); B200_TRY(dalloc(&n_expert_dev, 1));
  B200_CUDA(cudaMemcpy(n_expert_dev, &c.n_expert, sizeof(int), cudaMemcpyHostToDevice));
  for (int i = 0; i < 3; i++) {
    const int tn = 64 << i;
    B200_TRY(make_x_tensor_map(xperm16, (int64_t)MR * used, H, tn, tm_xperm[i]));
    B200_TRY(make_x_tensor_map(act16, (int64_t)MR * slots1, c.ffn_expert, tn, tm_act[i]));
    B200_TRY(make_x_tensor_map(xn16, MR, H, tn, tm_xn[i]));
    B200_TRY(make_x_tensor_map(y16, MR, vw, tn, tm_y16[i]));
    B200_TRY(make_x_tensor_map(ctx16, MR, qw, tn, tm_ctx[i]));
  }
  B200_TRY(dalloc(&ids_dev, (size_t)MR)); B200_TRY(dalloc(&next_ids, (size_t)MR)); B200_TRY(dalloc(&row_slot, (size_t)MR));
  B200_TRY(dalloc(&row_pos, (size_t)MR)); B200_TRY(dalloc(&logit_rows, (size_t)MR)); B200_TRY(dalloc(&seqs, (size_t)MR));
  B200_TRY(dalloc(&hist_len, 1));
  B200_TRY(dalloc(&distinct_dev, 1));
  if (c.has_draft) { B200_TRY(dalloc(&e_buf, (size_t)MR * H)); B200_TRY(dalloc(&hs_buf, (size_t)MR * H)); B200_TRY(dalloc(&xcat16, (size_t)MR * 2 * H)); }
  // rotary table, angle walked in f64 like the reference (llm/attn.go:554-584, llm/gpu_attn.go:1440-1477)
  {
    const int rot = std::min(c.rope_dims, c.head_dim), half = rot / 2, npos = o.n_kv + 2;
    std::vector<float> tab((size_t)npos * half * 2);
    const double scale = std::pow((double)c.rope_base, -2.0 / (double)rot);
    for (int p = 0; p < npos; p++) {
      double theta = (double)p;
      for (int i = 0; i < half; i++) {
        tab[((size_t)p * half + i) * 2] = (float)std::cos(theta);
        tab[((size_t)p * half + i) * 2 + 1] = (float)std::sin(theta);
        theta *= scale;
      }
    }
    B200_TRY(dalloc(&rope, tab.size(), false));
    B200_CUDA(cudaMemcpy(rope, tab.data(), tab.size() * sizeof(float), cudaMemcpyHostToDevice));
  }
  // sequence state
  state_slot_stride = (int64_t)c.dn_heads_v * D * D;
  ring_slot_stride = (int64_t)c.dn_heads_v * 4 * DN_RING * DN_RING_W;
  kv_slot_stride = (int64_t)o.n_kv * kvw;
  mid_seq_stride = (int64_t)std::max(o.spec_rows, 1) * state_slot_stride;
  dn_state.resize(n_dn); dn_ring.resize(n_dn); dn_mid.assign(n_dn, nullptr);
  for (int i = 0; i < n_dn; i++) {
    B200_TRY(dalloc(&dn_state[i], (size_t)o.slots * state_slot_stride));
    B200_TRY(dalloc(&dn_ring[i], (size_t)o.slots * ring_slot_stride));
    if (o.speculative) B200_TRY(dalloc(&dn_mid[i], (size_t)mid_seq_stride));
  }
  kcache.resize(n_attn); vcache.resize(n_attn);
  for (int i = 0; i < n_attn; i++) {
    B200_TRY(dalloc(&kcache[i], (size_t)o.slots * kv_slot_stride));
    B200_TRY(dalloc(&vcache[i], (size_t)o.slots * kv_slot_stride));
  }
  past.assign(o.slots, 0); draft_past.assign(o.slots, 0);
  // host staging
  stage_bytes = (size_t)MR * (4 * sizeof(int32_t) + sizeof(SeqDesc));
  B200_CUDA(cudaMallocHost((void**)&stage, stage_bytes));
  B200_CUDA(cudaMallocHost((void**)&logits_host, (size_t)LR * c.vocab * sizeof(float)));
  B200_CUDA(cudaMallocHost((void**)&resid_host, (size_t)MR * H * sizeof(float)));
  B200_CUDA(cudaMallocHost((void**)&hidden_host, (size_t)H * sizeof(float)));
  B200_CUDA(cudaMallocHost((void**)&err_host, sizeof(int)));
  *err_host = 0;
  B200_CUDA(cudaMallocHost((void**)&ids_host, (size_t)MR * 4096 * sizeof(int32_t)));
  B200_TRY(dalloc(&history, (size_t)MR * 4096));
  if (o.trace) {
    B200_TRY(dalloc(&tr_mid, (size_t)nl * MR * H)); B200_TRY(dalloc(&tr_out, (size_t)nl * MR * H));
    B200_TRY(dalloc(&tr_topk, (size_t)nl * MR * used)); B200_TRY(dalloc(&tr_w, (size_t)nl * MR * slots1)); B200_TRY(dalloc(&tr_margin, (size_t)nl * MR));
  }
  if (getenv("B200_TIMELINE") != nullptr) { timeline_cap = 1024; B200_TRY(dalloc(&timeline, (size_t)timeline_cap * 8)); }
  B200_CUDA(cudaDeviceSynchronize());
  return OK;
}

// Columns per work-list entry. A pass of some tens of rows leaves one or two rows per touched expert: entries of
// four columns halve the activation staging of the expert kernels, which then fit three to an SM.
int Graph::entry_cols(int M) { return M >= 16 && M <= 128 ? 4 : 8; }

int Graph::max_entries_for(int M) const {
  const int used = m->c.n_expert_used, ec = entry_cols(M);
  return std::min(M * used, m->c.n_expert + (M * used + ec - 1) / ec) + (M + ec - 1) / ec;
}

// Tile height of a many-row projection of N weight rows over M activation rows: as tall as the pass allows,
// shrunk while the launch would leave SMs idle. 0: its tiles would cover under a third of the SMs and the
// projection stays on the column-tiled kernel (exact weights).
static int gemm_tile_rows(int M, int N) {
  int tn = M <= 64 ? 64 : M <= 128 ? 128 : 256;
  while (tn > 64 && ((N + 127) / 128) * ((M + tn - 1) / tn) < 120) tn /= 2;
  if (((N + 127) / 128) * ((M + tn - 1) / tn) < 48) return 0;
  return tn;
}
// Router logits of passes of this many rows and more come from the column-tiled mma kernel (Q8_0 weights as
// fp16(d * q), the reference's many-row router arithmetic: llm_gemm MODE 2), below it from per-row dot products
constexpr int ROUTER_MMA_FROM = 16;
// Fused passes (at most 8 rows) of this many rows and more finish the MoE block's rows in one row kernel; with fewer
// rows every CTA of the next projection forms them while it stages (each staged row costs every CTA a trip to L2)
constexpr int COMBINE_ROWS_FROM = 4;
static bool pass_uses_gemm(int M, int H) { return !(M <= QG_FUSED_ROWS && H <= QG_COMBINE_MAX_K) && M >= 16; }
static bool pass_moe_gemm(const b200_config& c, const LayerW& L, int M, int H) {
  return pass_uses_gemm(M, H) && (int64_t)M * c.n_expert_used >= 32 * (int64_t)c.n_expert && L.gate_exps.type == L.gate_sh.type && L.down_exps.type == L.down_sh.type;
}

// Which weight matrices a pass of M rows multiplies as fp16-rounded values (the tensor-core kernels, the
// reference's prefill arithmetic: shaders/llm_gemm.comp MODE 2, shaders/llm_moe_gemm.comp:260-261) and
// which as exact dequantised values (the column-tiled kernels). The same predicates drive enqueue_pass.
uint32_t Graph::fp16_weight_mask(int M, int n_logit_rows) const {
  const b200_config& c = m->c;
  const int H = c.n_embd, D = c.dn_head_dim, qk = c.dn_heads_k * D, vw = c.dn_heads_v * D, cw = 2 * qk + vw;
  const int hd = c.head_dim, qw = c.n_head * hd, kvw = c.n_head_kv * hd;
  if (!pass_uses_gemm(M, H)) return 0;
  uint32_t mask = 0;
  if (gemm_tile_rows(M, cw)) mask |= B200_W16_DN_QKV;
  if (gemm_tile_rows(M, vw)) mask |= B200_W16_DN_GATE;
  if (gemm_tile_rows(M, H)) mask |= B200_W16_DN_OUT | B200_W16_ATTN_OUT;
  if (gemm_tile_rows(M, 2 * qw)) mask |= B200_W16_ATTN_Q;
  if (gemm_tile_rows(M, kvw)) mask |= B200_W16_ATTN_K | B200_W16_ATTN_V;
  for (const LayerW& L : m->layers) {
    if (M >= ROUTER_MMA_FROM && L.router.type == T_Q8_0) mask |= B200_W16_ROUTER;
    if (pass_moe_gemm(c, L, M, H)) mask |= B200_W16_EXPERTS | B200_W16_SHARED;
  }
  if (n_logit_rows == M && gemm_tile_rows(M, c.vocab)) mask |= B200_W16_HEAD;
  return mask;
}

// ---- one pass over M rows --------------------------------------------------------------
// Per layer: [in-proj] [DeltaNet step | attention pre-pass + split-KV attention] [out-proj + residual]
// [router + top-k + work list] [experts gate/up + SwiGLU] [experts down + weighted combine + residual].
// Passes of at most 8 rows never materialise a norm: the kernel that writes the residual leaves per-CTA
// partial sums of squares, and each consumer normalises the rows while it stages them. Larger passes
// finish their rows in stand-alone row kernels and read fp16 rows.
int Graph::enqueue_pass(int M, int n_seq, int n_logit_rows, const PassFlags& f) {
  const b200_config& c = m->c;
  const int H = c.n_embd, D = c.dn_head_dim, qk = c.dn_heads_k * D, vw = c.dn_heads_v * D, cw = 2 * qk + vw;
  const int hd = c.head_dim, qw = c.n_head * hd, kvw = c.n_head_kv * hd, used = c.n_expert_used, slots1 = used + 1;
  const int xcols = std::min(M, QG_MAXCOLS);
  const bool fused = M <= QG_FUSED_ROWS && H <= QG_COMBINE_MAX_K;
  // expert-parallel MoE block: plain decode passes only (every rank runs the same number of rows at the same time)
  const bool epx = ep_on && ep_ready && !f.draft && !f.spec && n_seq == M;
  const int Mg = epx ? M * ep.world : M;   // rows of all ranks
  float* hc = hbuf[0];      // residual rows of this pass
  bool pending = false;     // fused passes: the MoE output of the last layer is not in hc yet; the next
                            // projection of the residual folds it in while staging and writes the other buffer
  int trace_layer = -1;     // layer whose post-MoE residual is still to be traced
  bool xn_valid = false;    // fused passes of 2..8 rows: a row kernel finished the MoE block and left the next
                            // layer's normalised fp16 rows in xn16 (reading (used + 1) x M expert rows in every
                            // CTA's staging costs more than that one launch)
  int comb_used = used;     // what the pending combine adds: comb_used + 1 rows of `down` with weights comb_w
  const float* comb_w = topk_w;
  launches = 0;
  bool first = true;
  int ss_n = 1;  // partial sums of squares the current residual rows carry
  auto pdl = [&]() { bool p = !first; first = false; launches++; return p; };
  // timestamps slot of the NEXT launch (launches counts the ones already issued)
  auto tl = [&]() { Timeline t{timeline, launches < timeline_cap ? launches : 0}; if (launches >= timeline_cap) t.buf = nullptr; return t; };
  auto base = [&](const DTensor& w, int K, int N, const __half* x, int ldx) {
    QGemvParams p{};
    p.w[0] = w.data; p.seg_end[0] = N; p.nseg = 1; p.stride = w.stride; p.K = K; p.N = N; p.M = M; p.xcols = xcols; p.x_div = 1;
    p.x = x; p.ldx = ldx; p.err = err_flag; p.tl = tl(); p.eps = c.eps;
    return p;
  };
  // a projection of the normalised residual: fused passes normalise while staging, others read xn16
  auto normed = [&](QGemvParams& p, const DTensor& gamma, __half* xn_copy) {
    if (!fused || xn_valid) return (int)PRO_F16;
    p.hsrc = hc; p.gamma = (const float*)gamma.data; p.xn_out = xn_copy;
    if (!pending) { p.ss_in = ss_part; p.ss_n = ss_n; return (int)PRO_NORM; }
    p.down = down; p.topk_w = comb_w; p.used = comb_used; p.h_out = hc == hbuf[0] ? hbuf[1] : hbuf[0];
    return (int)PRO_COMBINE;
  };
  // after a PRO_COMBINE launch the rows live in the other buffer
  auto combined = [&](int pro) {
    if (pro != PRO_COMBINE) return OK;
    hc = hc == hbuf[0] ? hbuf[1] : hbuf[0]; pending = false;
    if (o.trace && trace_layer >= 0) {
      B200_CUDA(cudaMemcpyAsync(tr_out + (size_t)trace_layer * MR * H, hc, (size_t)M * H * sizeof(float), cudaMemcpyDeviceToDevice, st));
      first = true; trace_layer = -1;
    }
    return OK;
  };
  auto row_tail = [&](int mode, const DTensor& gamma) {
    TailParams t{};
    t.mode = mode; t.h = hc; t.gamma = (const float*)gamma.data; t.xn = xn16; t.down = down; t.topk_w = fused ? comb_w : topk_w;
    t.used = fused ? comb_used : used; t.H = H; t.M = M; t.eps = c.eps;
    return t;
  };
  // passes of 16 rows and more run their dense projections on the tensor cores
  const bool use_gemm = pass_uses_gemm(M, H);
  // tile height per projection: as tall as the pass allows, shrunk while the launch would leave SMs idle
  // a projection whose tiles would cover under a third of the SMs stays on the column-tiled kernel
  auto gemm = [&](const DTensor& w, int K, int N, const __half* x, const unsigned char (*tmaps)[128], float* y, int64_t ldy, int epi) {
    const int tn = gemm_tile_rows(M, N);
    if (tn == 0) {
      QGemvParams q = base(w, K, N, x, K);
      q.y = y; q.ldy = ldy;
      return launch_qgemv(w.type, PRO_F16, epi == GEMM_RESID ? EPI_RESID : EPI_STORE, false, false, q, 0, pdl(), st);
    }
    const unsigned char* tmap = tmaps[tn == 64 ? 0 : tn == 128 ? 1 : 2];
    QGemmParams g{};
    g.w = w.data; g.one = GemmProblem{0, 0, M, 0}; g.max_problems = 1; g.max_count = M; g.stride = w.stride; g.K = K; g.N = N; g.y = y; g.ldy = ldy; g.err = err_flag;
    return launch_qgemm(w.type, epi, tn, g, tmap, pdl(), st);
  };
  const int l0 = f.draft ? c.n_layer : 0, l1 = f.draft ? c.n_layer + 1 : c.n_layer;
  if (f.draft) {
    // nextn seed, embedding first: h = eh_proj . concat(rms(embd, enorm), rms(h_prev, hnorm))  (llm/mtp.go:352-384)
    const LayerW& L = m->layers[c.n_layer];
    EmbedParams ep{m->token_embd, ids_dev, e_buf, M, H, nullptr, nullptr, c.eps, nullptr};
    B200_TRY(launch_embed(ep, st)); pdl();
    B200_TRY(launch_concat_norm(e_buf, hs_buf, (const float*)L.enorm.data, (const float*)L.hnorm.data, c.eps, H, M, xcat16, pdl(), st));
    QGemvParams p = base(L.eh_proj, 2 * H, H, xcat16, 2 * H);
    p.y = hc; p.ldy = H;
    if (fused) { p.ss_out = ss_part; ss_n = qgemv_groups(2 * H, H); }
    B200_TRY(launch_qgemv(L.eh_proj.type, PRO_F16, EPI_STORE, false, false, p, 0, pdl(), st));
    if (!fused) B200_TRY(launch_row_tail(row_tail(1, L.attn_norm), pdl(), st));
  } else {
    const LayerW& L0 = m->layers[0];
    EmbedParams ep{m->token_embd, ids_dev, hc, M, H, fused ? nullptr : (const float*)L0.attn_norm.data, xn16, c.eps, fused ? ss_part : nullptr};
    B200_TRY(launch_embed(ep, st)); pdl();
    ss_n = 1;
  }
  for (int l = l0; l < l1; l++) {
    const LayerW& L = m->layers[l];
    if (!L.is_attn) {
      const int di = dn_index[l];
      QGemvParams p = base(L.qkv, H, cw + vw, xn16, H);
      p.w[1] = L.z.data; p.seg_end[0] = cw; p.seg_end[1] = cw + vw; p.nseg = 2;
      p.y = proj; p.ldy = proj_ld;
      if (use_gemm) {
        B200_TRY(gemm(L.qkv, H, cw, xn16, tm_xn, proj, proj_ld, GEMM_STORE));
        B200_TRY(gemm(L.z, H, vw, xn16, tm_xn, proj + cw, proj_ld, GEMM_STORE));
      } else {
        const int pro = normed(p, L.attn_norm, xn16);  // the DeltaNet step reads the fp16 rows for alpha / beta
        B200_TRY(launch_qgemv(L.qkv.type, pro, EPI_STORE, false, false, p, 0, pdl(), st));
        B200_TRY(combined(pro));
      }
      DnStepParams d{};
      d.proj = proj; d.ldp = proj_ld; d.xn = xn16; d.alpha_w = (const float*)L.alpha.data; d.beta_w = (const float*)L.beta.data;
      d.conv_w = (const float*)L.conv1d.data; d.ssm_a = (const float*)L.ssm_a.data; d.dt_bias = (const float*)L.dt_bias.data;
      d.state = dn_state[di]; d.state_slot_stride = state_slot_stride; d.ring = dn_ring[di]; d.ring_slot_stride = ring_slot_stride;
      d.seqs = seqs; d.n_seq = n_seq; d.norm_w = (const float*)L.ssm_norm.data; d.y16 = y16;
      d.mid = f.spec ? dn_mid[di] : nullptr; d.mid_stride = state_slot_stride; d.mid_seq_stride = mid_seq_stride;
      d.H = H; d.Hk = c.dn_heads_k; d.Hv = c.dn_heads_v; d.D = D; d.conv = c.dn_conv; d.eps = c.eps; d.tl = tl();
      if (!fused && !f.spec && M > n_seq) {  // some sequence is long: state-independent part in parallel, then the scan
        d.pre = dn_pre; d.pre_rows = MR; d.o_raw = dn_oraw; d.ab = dn_ab;
        B200_TRY(launch_dn_scan(d, M, pass_max_n, pdl(), st)); launches += 3;
      } else {
        B200_TRY(launch_dn_step(d, pdl(), st));
      }
      QGemvParams q = base(L.ssm_out, vw, H, y16, vw);
      q.y = hc; q.ldy = H;
      if (fused) { q.ss_out = ss_part; ss_n = qgemv_groups(vw, H); }
      if (use_gemm) B200_TRY(gemm(L.ssm_out, vw, H, y16, tm_y16, hc, H, GEMM_RESID));
      else B200_TRY(launch_qgemv(L.ssm_out.type, PRO_F16, EPI_RESID, false, false, q, 0, pdl(), st));
    } else {
      const int ai = attn_index[l];
      // fused q|k|v projection; tensors of one type share a launch
      const DTensor* seg[3] = {&L.q, &L.k, &L.v};
      const int rows[3] = {2 * qw, kvw, kvw};
      int off = 0;
      bool xn_ready = false;
      for (int s = 0; s < 3 && use_gemm; s++) { B200_TRY(gemm(*seg[s], H, rows[s], xn16, tm_xn, proj + off, proj_ld, GEMM_STORE)); off += rows[s]; }
      for (int s = 0; s < 3 && !use_gemm;) {
        int e = s + 1;
        while (e < 3 && seg[e]->type == seg[s]->type) e++;
        int n = 0;
        QGemvParams p = base(*seg[s], H, 0, xn16, H);
        for (int i = s; i < e; i++) { p.w[i - s] = seg[i]->data; n += rows[i]; p.seg_end[i - s] = n; }
        p.nseg = e - s; p.N = n;
        p.y = proj + off; p.ldy = proj_ld;
        // the launch that folds the MoE output in also leaves the fp16 rows for the launches after it
        const int pro = normed(p, L.attn_norm, pending ? xn16 : nullptr);
        if (xn_ready) { B200_TRY(launch_qgemv(seg[s]->type, PRO_F16, EPI_STORE, false, false, p, 0, pdl(), st)); }
        else { B200_TRY(launch_qgemv(seg[s]->type, pro, EPI_STORE, false, false, p, 0, pdl(), st)); xn_ready = pro == PRO_COMBINE; B200_TRY(combined(pro)); }
        off += n; s = e;
      }
      AttnParams a{};
      a.proj = proj; a.ldp = proj_ld; a.q_norm = (const float*)L.q_norm.data; a.k_norm = (const float*)L.k_norm.data; a.rope = rope;
      a.kcache = kcache[ai]; a.vcache = vcache[ai]; a.slot_stride = kv_slot_stride; a.row_slot = row_slot; a.row_pos = row_pos;
      a.q16 = q16; a.partial = attn_partial; a.ctx16 = ctx16;
      a.M = M; a.Hq = c.n_head; a.Hkv = c.n_head_kv; a.hd = hd; a.rope_dims = std::min(c.rope_dims, hd); a.n_kv = o.n_kv;
      // many rows: longer splits while the grid still fills the device several times over (fewer partial
      // results to write and merge); the buffer is sized for the shortest split
      int sc = split_cells;
      if (o.attn_split_cells <= 0) while (sc < 2048 && (int64_t)M * c.n_head_kv * ((o.n_kv + sc - 1) / sc) >= 4096) sc *= 2;
      a.split_cells = sc; a.nsplit = (o.n_kv + sc - 1) / sc; a.eps = c.eps; a.rope_off = f.draft ? 1 : 0;
      a.one_row_per_seq = M == n_seq && !f.spec; a.err = err_flag; a.tl = tl();
      B200_TRY(launch_attn_pack(a, pdl(), st));
      a.tl = tl();
      if (n_seq == 1 && !f.spec && attn_prefill_fits(a)) {
        // many rows of one sequence: query tiles x key tiles, straight to the gated context rows
        B200_TRY(launch_attn_prefill(a, pdl(), st));
      } else {
        if (M > attn_rows) { set_error("pass of " + std::to_string(M) + " rows: the split attention buffers hold " + std::to_string(attn_rows)); return ECAPACITY; }
        B200_TRY(launch_attn_decode(a, pdl(), st));
        a.tl = tl();
        B200_TRY(launch_attn_merge(a, pdl(), st));
      }
      QGemvParams q = base(L.o, qw, H, ctx16, qw);
      q.y = hc; q.ldy = H;
      if (fused) { q.ss_out = ss_part; ss_n = qgemv_groups(qw, H); }
      if (use_gemm) B200_TRY(gemm(L.o, qw, H, ctx16, tm_ctx, hc, H, GEMM_RESID));
      else B200_TRY(launch_qgemv(L.o.type, PRO_F16, EPI_RESID, false, false, q, 0, pdl(), st));
    }
    if (!fused) B200_TRY(launch_row_tail(row_tail(1, L.ffn_norm), pdl(), st));
    if (o.trace) { B200_CUDA(cudaMemcpyAsync(tr_mid + (size_t)l * MR * H, hc, (size_t)M * H * sizeof(float), cudaMemcpyDeviceToDevice, st)); first = true; }
    // MoE block
    xn_valid = false;  // the router leaves its own normalised rows in xn16
    RouterParams r{};
    r.xn = xn16; r.router = L.router; r.sh_gate = (const float*)L.sh_gate_inp.data;
    if (fused) { r.h = hc; r.gamma = (const float*)L.ffn_norm.data; r.ss_in = ss_part; r.ss_n = ss_n; r.eps = c.eps; r.xn_out = xn16; }
    r.M = M; r.H = H; r.nE = c.n_expert; r.used = used; r.logits = r_logits; r.probs = nullptr; r.topk = topk; r.topk_w = topk_w;
    r.tl = tl(); r.margin = margin; r.entries = entries; r.n_entries = n_entries; r.cols = cols; r.ticket = r_ticket; r.max_entries = max_entries;
    // passes of at most 8 rows: the router stops after its logits and every row is routed, computed and combined on
    // the single-row schedule, so each row's result is the single-row pass's, bit for bit (the reference's batched
    // decode and verify passes equal their rows stepped alone: llm/graph_batch_test.go:36, llm/spec_slots_test.go:199)
    r.defer = fused && !epx; r.ecols = entry_cols(M); r.distinct = r.defer ? nullptr : distinct_dev;
    if (epx) { r.entries = nullptr; r.gprob = nullptr; }   // routing only: the work list comes from the gathered routing
    // 32 rows per expert on average and more: the experts run as grouped tensor-core GEMMs over expert-sorted
    // rows (below that the column-tiled kernel, which streams each expert's weights in whole tiles, is faster)
    const bool moe_gemm = pass_moe_gemm(c, L, M, H) && !epx;
    r.gprob = moe_gemm ? gprob : nullptr;
    if (use_gemm && M >= ROUTER_MMA_FROM && L.router.type == T_Q8_0) {
      // many rows: the router logits are one more tensor-core GEMM (the reference's prefill router is an fp16
      // GEMM too: llm_gemm MODE 2 + llm_moe_route), selection and work list in a kernel of their own
      QGemmParams g{};
      g.w = L.router.data; g.one = GemmProblem{0, 0, M, 0}; g.max_problems = 1; g.max_count = M; g.stride = L.router.stride;
      g.K = H; g.N = c.n_expert; g.y = r_logits; g.ldy = c.n_expert; g.err = err_flag;
      // up to a few hundred rows the four 128-expert tiles leave the device idle: column-tiled mma instead
      if (M < 256 && router_mma_fits(r)) { B200_TRY(launch_router_mma(r, pdl(), st)); }
      else B200_TRY(launch_qgemm(T_Q8_0, GEMM_STORE, 64, g, tm_xn[0], pdl(), st));
      B200_TRY(launch_route_rows(r, pdl(), st));
    } else {
      B200_TRY(launch_router(r, pdl(), st));
    }
    const int ne = max_entries_for(Mg);
    comb_used = used; comb_w = topk_w;
    float* down_rows = down;   // where the pairs of this rank's rows land
    if (epx) {
      // dispatch -> work list over my experts -> gate/up -> down (stores to the rows' owners) -> barrier
      EpParams e = ep;
      e.rows = M; e.xn = xn16; e.topk = topk;
      B200_TRY(launch_ep_dispatch(e, pdl(), st));
      RouterParams w = r;
      w.M = Mg; w.topk = reinterpret_cast<int32_t*>(ep_arena + ep.off_topk); w.entries = entries; w.ecols = entry_cols(Mg);
      w.e_lo = ep.rank * (c.n_expert / ep.world); w.e_hi = w.e_lo + c.n_expert / ep.world; w.sh_lo = ep.rank * M; w.sh_hi = w.sh_lo + M;
      w.n_pairs = ep_epoch + 2;
      B200_TRY(launch_ep_worklist(w, pdl(), st));
      const int ecx = std::min(std::min(Mg, QG_MAXCOLS), entry_cols(Mg));
      QGemvParams p = base(L.gate_exps, H, c.ffn_expert, reinterpret_cast<const __half*>(ep_arena + ep.off_xg), H);
      p.w2[0] = L.up_exps.data; p.ws = L.gate_sh.data; p.ws2 = L.up_sh.data; p.expert_stride = (int64_t)c.ffn_expert * L.gate_exps.stride;
      p.entries = entries; p.n_entries = n_entries; p.cols = cols; p.x_div = slots1; p.xcols = ecx; p.M = Mg;
      p.y16 = act16; p.ldy = c.ffn_expert;
      B200_TRY(launch_qgemv(L.gate_exps.type, PRO_F16, EPI_SWIGLU, true, true, p, ne, pdl(), st));
      QGemvParams q = base(L.down_exps, c.ffn_expert, H, act16, c.ffn_expert);
      q.ws = L.down_sh.data; q.expert_stride = (int64_t)H * L.down_exps.stride;
      q.entries = entries; q.n_entries = n_entries; q.cols = cols; q.x_div = 1; q.xcols = ecx; q.M = Mg;
      q.y = down; q.ldy = H;     // local: rows by pair id; the combine kernel carries them to the rows' owners
      B200_TRY(launch_qgemv(L.down_exps.type, PRO_F16, EPI_STORE, false, true, q, ne, pdl(), st));
      e.y_local = down; e.cols = cols; e.n_pairs = ep_epoch + 2; e.pairs_per_rank = M * slots1;
      B200_TRY(launch_ep_combine(e, M * slots1 + (Mg - M) * used, pdl(), st));
      down_rows = reinterpret_cast<float*>(ep_arena + ep.off_down);
    } else if (moe_gemm) {
      const int avg = M * used / c.n_expert, tne = avg <= 40 ? 64 : 128, tie = tne == 64 ? 0 : 1;
      B200_TRY(launch_moe_gather(xn16, cols, M * used, slots1, H, xperm16, pdl(), st));
      QGemmParams g{};
      g.problems = reinterpret_cast<const GemmProblem*>(gprob); g.n_problems = n_expert_dev; g.max_problems = c.n_expert; g.max_count = M;
      g.w = L.gate_exps.data; g.w2 = L.up_exps.data; g.expert_stride = (int64_t)c.ffn_expert * L.gate_exps.stride; g.stride = L.gate_exps.stride;
      g.K = H; g.N = c.ffn_expert; g.y16 = act16; g.ldy = c.ffn_expert; g.err = err_flag;
      B200_TRY(launch_qgemm(L.gate_exps.type, GEMM_SWIGLU, tne, g, tm_xperm[tie], pdl(), st));
      QGemmParams sh{};  // the shared expert: every row, outputs after the routed pairs
      sh.one = GemmProblem{0, 0, M, M * used}; sh.max_problems = 1; sh.max_count = M; sh.w = L.gate_sh.data; sh.w2 = L.up_sh.data; sh.stride = L.gate_sh.stride;
      sh.K = H; sh.N = c.ffn_expert; sh.y16 = act16; sh.ldy = c.ffn_expert; sh.err = err_flag;
      B200_TRY(launch_qgemm(L.gate_sh.type, GEMM_SWIGLU, 64, sh, tm_xn[0], pdl(), st));  // few weight tiles: short activation tiles fill more SMs
      QGemmParams d{};   // down projections: sorted rows in, pair rows out (cols maps sorted row -> pair)
      d.problems = g.problems; d.n_problems = n_expert_dev; d.max_problems = c.n_expert; d.max_count = M;
      d.w = L.down_exps.data; d.expert_stride = (int64_t)H * L.down_exps.stride; d.stride = L.down_exps.stride;
      d.K = c.ffn_expert; d.N = H; d.y = down; d.ldy = H; d.y_rows = cols; d.err = err_flag;
      B200_TRY(launch_qgemm(L.down_exps.type, GEMM_STORE, tne, d, tm_act[tie], pdl(), st));
      QGemmParams ds{};
      ds.one = GemmProblem{0, M * used, M, M * used}; ds.max_problems = 1; ds.max_count = M; ds.w = L.down_sh.data; ds.stride = L.down_sh.stride;
      ds.K = c.ffn_expert; ds.N = H; ds.y = down; ds.ldy = H; ds.y_rows = cols; ds.err = err_flag;
      B200_TRY(launch_qgemm(L.down_sh.type, GEMM_STORE, 64, ds, tm_act[0], pdl(), st));
    } else {
    QGemvParams p = base(L.gate_exps, H, c.ffn_expert, xn16, H);
    p.w2[0] = L.up_exps.data; p.ws = L.gate_sh.data; p.ws2 = L.up_sh.data; p.expert_stride = (int64_t)c.ffn_expert * L.gate_exps.stride;
    p.entries = entries; p.n_entries = n_entries; p.cols = cols; p.x_div = slots1; p.xcols = r.defer ? 1 : std::min(xcols, entry_cols(M));
    p.y16 = act16; p.ldy = c.ffn_expert;
    p.route_here = r.defer; p.route = r;
    B200_TRY(launch_qgemv(L.gate_exps.type, PRO_F16, EPI_SWIGLU, true, true, p, r.defer ? M * slots1 : ne, pdl(), st));
    QGemvParams q = base(L.down_exps, c.ffn_expert, H, act16, c.ffn_expert);
    q.ws = L.down_sh.data; q.expert_stride = (int64_t)H * L.down_exps.stride;
    q.entries = entries; q.n_entries = n_entries; q.cols = cols; q.x_div = 1; q.xcols = std::min(xcols, entry_cols(M));
    q.y = down; q.ldy = H;
    if (r.defer && L.down_exps.type == L.down_sh.type && slots1 <= 16) {
      // per row: the routing weights are applied inside the down projection, which leaves a few partial rows
      // (one per CTA of a tile) for the next projection to add, instead of used + 1 expert rows
      MoeDown1Params d1{};
      d1.w = L.down_exps.data; d1.ws = L.down_sh.data; d1.expert_stride = (int64_t)H * L.down_exps.stride; d1.stride = L.down_exps.stride;
      d1.K = c.ffn_expert; d1.N = H; d1.used = used; d1.topk = topk; d1.topk_w = topk_w; d1.act = act16; d1.part = down;
      d1.split = moe_down1_split(used, c.ffn_expert); d1.err = err_flag; d1.tl = tl();
      B200_TRY(launch_moe_down1(L.down_exps.type, d1, M, pdl(), st));
      comb_used = d1.split - 1; comb_w = ones;
    } else {
      B200_TRY(launch_qgemv(L.down_exps.type, PRO_F16, EPI_STORE, false, true, q, ne, pdl(), st));
    }
    }
    if (r.defer && M >= COMBINE_ROWS_FROM) {
      // the rows are finished once, by the arithmetic the next projection's staging would use (same sums in the
      // same order, so the rows are the single-row pass's bit for bit), and the consumers read fp16 rows
      const DTensor& next_norm = f.draft ? L.head_norm : (l + 1 < c.n_layer ? m->layers[l + 1].attn_norm : m->output_norm);
      QGemvParams cp{};
      cp.K = H; cp.M = M; cp.xcols = 1; cp.hsrc = hc; cp.gamma = (const float*)next_norm.data; cp.xn_out = xn16; cp.eps = c.eps;
      cp.down = down; cp.topk_w = comb_w; cp.used = comb_used; cp.h_out = hc == hbuf[0] ? hbuf[1] : hbuf[0];
      B200_TRY(launch_combine_rows(cp, pdl(), st));
      hc = cp.h_out;
      xn_valid = true;
    } else if (r.defer) pending = true;
    else {
      const DTensor& next_norm = f.draft ? L.head_norm : (l + 1 < c.n_layer ? m->layers[l + 1].attn_norm : m->output_norm);
      TailParams tp = row_tail(2, next_norm);
      tp.down = down_rows;
      B200_TRY(launch_row_tail(tp, pdl(), st));
      xn_valid = fused;
    }
    if (o.trace) {
      if (pending) trace_layer = l;
      else B200_CUDA(cudaMemcpyAsync(tr_out + (size_t)l * MR * H, hc, (size_t)M * H * sizeof(float), cudaMemcpyDeviceToDevice, st));
      B200_CUDA(cudaMemcpyAsync(tr_topk + (size_t)l * MR * used, topk, (size_t)M * used * sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
      B200_CUDA(cudaMemcpyAsync(tr_w + (size_t)l * MR * slots1, topk_w, (size_t)M * slots1 * sizeof(float), cudaMemcpyDeviceToDevice, st));
      B200_CUDA(cudaMemcpyAsync(tr_margin + (size_t)l * MR, margin, (size_t)M * sizeof(float), cudaMemcpyDeviceToDevice, st));
      first = true;  // copies sit between this kernel and the next: no programmatic edge
    }
  }
  const DTensor& nrm = f.draft ? m->layers[c.n_layer].head_norm : m->output_norm;
  bool head_reads_xn = false;
  if (pending && n_logit_rows != M) {
    // the head stages only some of the rows (or none): finish every row in place first
    B200_TRY(launch_row_tail(row_tail(2, nrm), pdl(), st));
    pending = false; head_reads_xn = true;
    if (o.trace && trace_layer >= 0) { B200_CUDA(cudaMemcpyAsync(tr_out + (size_t)trace_layer * MR * H, hc, (size_t)M * H * sizeof(float), cudaMemcpyDeviceToDevice, st)); first = true; trace_layer = -1; }
  }
  if (n_logit_rows > 0) {
    const int N = f.draft && draft_vocab > 0 ? draft_vocab : c.vocab;
    QGemvParams p = base(m->output, H, N, xn16, H);
    p.M = n_logit_rows; p.xcols = std::min(n_logit_rows, QG_MAXCOLS); p.row_ids = logit_rows;
    p.y = logits; p.ldy = N;
    if (use_gemm && n_logit_rows == M) {
      B200_TRY(gemm(m->output, H, N, xn16, tm_xn, logits, N, GEMM_STORE));
    } else {
      const int pro = head_reads_xn ? (int)PRO_F16 : normed(p, nrm, nullptr);
      B200_TRY(launch_qgemv(m->output.type, pro, EPI_STORE, false, false, p, 0, pdl(), st));
      B200_TRY(combined(pro));
    }
    if (f.greedy) {
      B200_TRY(launch_argmax(logits, n_logit_rows, N, next_ids, pdl(), st));
      B200_TRY(launch_advance(ids_dev, next_ids, row_pos, seqs, M, history, hist_len, st)); launches++;
    }
  }
  h = hc;
  last_launches = launches;
  return OK;
}

static void fill_stage(uint8_t* stage, int MR, const int32_t* ids, const int* slots, const int* pos, int M, const std::vector<SeqDesc>& sq, const std::vector<int>& lrows) {
  int32_t* s_ids = (int32_t*)stage; int* s_slot = (int*)stage + MR; int* s_pos = (int*)stage + 2 * MR; int* s_lr = (int*)stage + 3 * MR;
  SeqDesc* s_sq = (SeqDesc*)((int*)stage + 4 * MR);
  for (int i = 0; i < M; i++) { s_ids[i] = ids[i]; s_slot[i] = slots[i]; s_pos[i] = pos[i]; }
  for (size_t i = 0; i < lrows.size(); i++) s_lr[i] = lrows[i];
  for (size_t i = 0; i < sq.size(); i++) s_sq[i] = sq[i];
}

static int upload_stage(Graph* g, int M, int n_seq, int n_lr) {
  const int MR = g->MR;
  uint8_t* s = g->stage;
  B200_CUDA(cudaMemcpyAsync(g->ids_dev, s, M * sizeof(int32_t), cudaMemcpyHostToDevice, g->st));
  B200_CUDA(cudaMemcpyAsync(g->row_slot, (int*)s + MR, M * sizeof(int), cudaMemcpyHostToDevice, g->st));
  B200_CUDA(cudaMemcpyAsync(g->row_pos, (int*)s + 2 * MR, M * sizeof(int), cudaMemcpyHostToDevice, g->st));
  if (n_lr > 0) B200_CUDA(cudaMemcpyAsync(g->logit_rows, (int*)s + 3 * MR, n_lr * sizeof(int), cudaMemcpyHostToDevice, g->st));
  B200_CUDA(cudaMemcpyAsync(g->seqs, (int*)s + 4 * MR, n_seq * sizeof(SeqDesc), cudaMemcpyHostToDevice, g->st));
  return OK;
}

int Graph::run_rows(const int32_t* ids, const int* slots, const int* pos, int M, const std::vector<SeqDesc>& sq, const std::vector<int>& lrows, const PassFlags& f) {
  const b200_config& c = m->c;
  for (int i = 0; i < M; i++) {
    if (ids[i] < 0 || ids[i] >= c.vocab) { set_error("token id " + std::to_string(ids[i]) + " is outside the vocabulary"); return EINVAL_; }
  }
  B200_CUDA(cudaSetDevice(m->device));
  const auto host_t0 = std::chrono::steady_clock::now();
  fill_stage(stage, MR, ids, slots, pos, M, sq, lrows);
  pass_max_n = 1;
  for (const SeqDesc& s : sq) pass_max_n = std::max(pass_max_n, s.n);
  const int n_lr = (int)lrows.size(), n_seq = (int)sq.size();
  const int NV = f.draft && draft_vocab > 0 ? draft_vocab : c.vocab;
  bool single = !f.spec && !f.draft && !o.trace && o.use_cuda_graph && n_seq == M && n_lr == M && !f.want_residual;
  B200_CUDA(cudaEventRecord(ev0, st));
  if (single) {
    const int gkey = M * 2 + (ep_on ? 1 : 0);
    auto it = decode_graphs.find(gkey);
    if (it == decode_graphs.end()) {
      // the decode step is captured once and replayed, positions living in device memory
      // (the reference's pre-recorded command buffer: llm/graph.go:238-258)
      cudaGraph_t graph = nullptr;
      B200_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
      int s = upload_stage(this, M, n_seq, n_lr);
      if (s == OK) s = enqueue_pass(M, n_seq, n_lr, f);
      if (s == OK && cudaMemcpyAsync(logits_host, logits, (size_t)n_lr * NV * sizeof(float), cudaMemcpyDeviceToHost, st) != cudaSuccess) s = ECUDA;
      cudaError_t e = cudaStreamEndCapture(st, &graph);
      if (s != OK || e != cudaSuccess) { if (graph) cudaGraphDestroy(graph); if (s == OK) { set_error(std::string("graph capture: ") + cudaGetErrorString(e)); s = ECUDA; } return s; }
      cudaGraphExec_t exec = nullptr;
      e = cudaGraphInstantiate(&exec, graph, 0);
      cudaGraphDestroy(graph);
      if (e != cudaSuccess) { set_error(std::string("graph instantiate: ") + cudaGetErrorString(e)); return ECUDA; }
      it = decode_graphs.emplace(gkey, exec).first;
      decode_h[gkey] = h;
    }
    B200_CUDA(cudaGraphLaunch(it->second, st));
    h = decode_h[gkey];
  } else {
    B200_TRY(upload_stage(this, M, n_seq, n_lr));
    B200_TRY(enqueue_pass(M, n_seq, n_lr, f));
    if (n_lr > 0) B200_CUDA(cudaMemcpyAsync(logits_host, logits, (size_t)n_lr * NV * sizeof(float), cudaMemcpyDeviceToHost, st));
  }
  if (f.want_residual) B200_CUDA(cudaMemcpyAsync(resid_host + (size_t)resid_off * c.n_embd, h, (size_t)M * c.n_embd * sizeof(float), cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaMemcpyAsync(hidden_host, h + (size_t)(M - 1) * c.n_embd, (size_t)c.n_embd * sizeof(float), cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaEventRecord(ev1, st));
  B200_TRY(finish_pass());
  last_rows = M;
  float ms = 0.f;
  B200_CUDA(cudaEventElapsedTime(&ms, ev0, ev1));
  stats.passes++; stats.rows += M; stats.launches += last_launches; stats.device_ms += ms;
  stats.host_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - host_t0).count();
  stats.last_rows = M; stats.last_launches = last_launches; stats.last_device_ms = ms;
  // rows of fused passes select their experts inside the expert kernel: one stream per row and slot
  if (M <= QG_FUSED_ROWS && m->c.n_embd <= QG_COMBINE_MAX_K && !f.draft && !(ep_on && ep_ready && n_seq == M)) single_row_layers += (int64_t)M * m->c.n_layer;
  return OK;
}

// Reads the error word back with the pass's results. A bounded wait that gave up is reported once:
// the word is cleared so that the graph stays usable (what the slot held is the caller's to forget,
// as the reference's scheduler does after a failed unit, backend/llm_sched.go:713-717).
int Graph::finish_pass() {
  B200_CUDA(cudaMemcpyAsync(err_host, err_flag, sizeof(int), cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaStreamSynchronize(st));
  if (*err_host != 0) {
    *err_host = 0;
    B200_CUDA(cudaMemsetAsync(err_flag, 0, sizeof(int), st));
    B200_CUDA(cudaStreamSynchronize(st));
    set_error("a kernel gave up a bounded wait (a copy or a peer that never arrived); the pass's results are not valid");
    return ETIMEOUT;
  }
  return OK;
}

int Graph::extend(const int32_t* ids, int n, const PassFlags& f, const float** logits_out, const float** hidden_out) {
  if (n <= 0) { set_error("extend: no tokens"); return EINVAL_; }
  if (f.spec) {
    if (!o.speculative) { set_error("extend: the graph was not created with speculative = 1"); return ESTATE; }
    if (n > o.spec_rows) { set_error("extend: a speculative pass holds at most spec_rows rows"); return ECAPACITY; }
  }
  if (f.want_all_logits && n > LR) { set_error("extend_rows: more rows than max_tokens (logits of at most 512 rows per pass)"); return ECAPACITY; }
  if (f.want_residual && n > MR) { set_error("extend_residual: more rows than max_tokens"); return ECAPACITY; }
  if (past[cur] + n > o.n_kv) { set_error("extend: the slot's context is full (" + std::to_string(past[cur]) + " + " + std::to_string(n) + " > " + std::to_string(o.n_kv) + ")"); return ECAPACITY; }
  resid_off = 0;
  for (int off = 0; off < n; off += MR) {
    const int M = std::min(MR, n - off);
    std::vector<int> slots(M, cur), pos(M);
    for (int i = 0; i < M; i++) pos[i] = past[cur] + i;
    std::vector<SeqDesc> sq{SeqDesc{cur, 0, M, past[cur]}};
    std::vector<int> lrows;
    if (f.want_all_logits) for (int i = 0; i < M; i++) lrows.push_back(i);
    else if (off + M == n) lrows.push_back(M - 1);
    B200_TRY(run_rows(ids + off, slots.data(), pos.data(), M, sq, lrows, f));
    if (f.spec) { spec_pos0 = past[cur]; spec_n = M; }
    else { past[cur] += M; spec_n = 0; }
    resid_off += M;
  }
  if (logits_out) *logits_out = logits_host;
  if (hidden_out) *hidden_out = f.want_residual ? resid_host : hidden_host;
  return OK;
}

int Graph::decode_rows(const int32_t* slots_in, const int32_t* ids, int n, const float** logits_out) {
  // one token for each of n distinct slots (reference: llm/batch.go:45-63)
  if (n <= 0 || n > LR) { set_error("decode_rows: 1.." + std::to_string(LR) + " rows"); return ECAPACITY; }
  std::vector<int> slots(n), pos(n), lrows(n);
  std::vector<SeqDesc> sq(n);
  std::vector<char> seen(o.slots, 0);
  for (int i = 0; i < n; i++) {
    const int s = slots_in[i];
    if (s < 0 || s >= o.slots) { set_error("decode_rows: slot " + std::to_string(s) + " does not exist"); return EINVAL_; }
    if (seen[s]) { set_error("decode_rows: slot " + std::to_string(s) + " appears twice"); return EINVAL_; }
    if (past[s] + 1 > o.n_kv) { set_error("decode_rows: slot " + std::to_string(s) + " is full"); return ECAPACITY; }
    seen[s] = 1; slots[i] = s; pos[i] = past[s]; lrows[i] = i; sq[i] = SeqDesc{s, i, 1, past[s]};
  }
  if (ep_on && (int64_t)n * ep.world > MR) { set_error("decode_rows: with expert parallelism the rows of all ranks (" + std::to_string(n) + " x " + std::to_string(ep.world) + ") must fit max_tokens"); return ECAPACITY; }
  PassFlags f; f.want_all_logits = true;
  B200_TRY(run_rows(ids, slots.data(), pos.data(), n, sq, lrows, f));
  for (int i = 0; i < n; i++) past[slots[i]] += 1;
  spec_n = 0;
  if (logits_out) *logits_out = logits_host;
  return OK;
}

int Graph::generate_greedy(const int32_t* slots_in, const int32_t* first, int n, int steps, int32_t* out) {
  const b200_config& c = m->c;
  if (n <= 0 || n > LR) { set_error("generate_greedy: 1.." + std::to_string(LR) + " rows"); return ECAPACITY; }
  if (steps <= 0 || steps > 4096) { set_error("generate_greedy: 1..4096 steps per call"); return ECAPACITY; }
  std::vector<int> slots(n), pos(n), lrows(n);
  std::vector<SeqDesc> sq(n);
  std::vector<char> seen(o.slots, 0);
  for (int i = 0; i < n; i++) {
    const int s = slots_in[i];
    if (s < 0 || s >= o.slots || seen[s]) { set_error("generate_greedy: bad or repeated slot"); return EINVAL_; }
    if (first[i] < 0 || first[i] >= c.vocab) { set_error("generate_greedy: token id outside the vocabulary"); return EINVAL_; }
    if (past[s] + steps > o.n_kv) { set_error("generate_greedy: slot " + std::to_string(s) + " would overflow its context"); return ECAPACITY; }
    seen[s] = 1; slots[i] = s; pos[i] = past[s]; lrows[i] = i; sq[i] = SeqDesc{s, i, 1, past[s]};
  }
  if (ep_on && (int64_t)n * ep.world > MR) { set_error("generate_greedy: with expert parallelism the rows of all ranks must fit max_tokens"); return ECAPACITY; }
  B200_CUDA(cudaSetDevice(m->device));
  fill_stage(stage, MR, first, slots.data(), pos.data(), n, sq, lrows);
  B200_TRY(upload_stage(this, n, n, n));
  B200_CUDA(cudaMemsetAsync(hist_len, 0, sizeof(int), st));
  PassFlags f; f.want_all_logits = true; f.greedy = true;
  cudaGraphExec_t exec = nullptr;
  if (o.use_cuda_graph && !o.trace) {
    const int gkey = n * 2 + (ep_on ? 1 : 0);
    auto it = greedy_graphs.find(gkey);
    if (it == greedy_graphs.end()) {
      cudaGraph_t graph = nullptr;
      B200_CUDA(cudaStreamSynchronize(st));
      B200_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
      int s = enqueue_pass(n, n, n, f);
      cudaError_t e = cudaStreamEndCapture(st, &graph);
      if (s != OK || e != cudaSuccess) { if (graph) cudaGraphDestroy(graph); if (s == OK) { set_error(std::string("graph capture: ") + cudaGetErrorString(e)); s = ECUDA; } return s; }
      e = cudaGraphInstantiate(&exec, graph, 0);
      cudaGraphDestroy(graph);
      if (e != cudaSuccess) { set_error(std::string("graph instantiate: ") + cudaGetErrorString(e)); return ECUDA; }
      greedy_graphs.emplace(gkey, exec);
    } else exec = it->second;
  }
  B200_CUDA(cudaEventRecord(ev0, st));
  for (int s = 0; s < steps; s++) {
    if (exec) B200_CUDA(cudaGraphLaunch(exec, st));
    else B200_TRY(enqueue_pass(n, n, n, f));
  }
  B200_CUDA(cudaEventRecord(ev1, st));
  B200_CUDA(cudaMemcpyAsync(ids_host, history, (size_t)steps * n * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  B200_TRY(finish_pass());
  B200_CUDA(cudaEventElapsedTime(&last_ms, ev0, ev1));
  stats.passes += steps; stats.rows += (int64_t)steps * n; stats.launches += (int64_t)steps * last_launches; stats.device_ms += last_ms;
  stats.last_rows = n; stats.last_launches = last_launches; stats.last_device_ms = last_ms / steps;
  if (n <= QG_FUSED_ROWS && m->c.n_embd <= QG_COMBINE_MAX_K && !(ep_on && ep_ready)) single_row_layers += (int64_t)steps * n * m->c.n_layer;
  memcpy(out, ids_host, (size_t)steps * n * sizeof(int32_t));
  for (int i = 0; i < n; i++) past[slots[i]] += steps;
  spec_n = 0;
  return OK;
}

int Graph::draft_rows(const float* hs, const int32_t* ids, int n, int vocab_k, const float** resid, const float** logits_out) {
  const b200_config& c = m->c;
  if (!c.has_draft) { set_error("draft_rows: the checkpoint has no draft layer"); return ESTATE; }
  if (n <= 0 || n > LR) { set_error("draft_rows: row count out of range"); return ECAPACITY; }
  if (vocab_k <= 0 && draft_vocab_default > 0) vocab_k = draft_vocab_default;
  if (vocab_k <= 0 || vocab_k > c.vocab) vocab_k = c.vocab;
  if (vocab_k % 16) { set_error("draft_rows: vocab_k must be a multiple of 16"); return EINVAL_; }
  if (draft_past[dcur] + n + 1 > o.n_kv) { set_error("draft_rows: the draft cache is full"); return ECAPACITY; }
  B200_CUDA(cudaSetDevice(m->device));
  B200_CUDA(cudaMemcpyAsync(hs_buf, hs, (size_t)n * c.n_embd * sizeof(float), cudaMemcpyHostToDevice, st));
  draft_vocab = vocab_k;
  std::vector<int> slots(n, dcur), pos(n), lrows(n);
  for (int i = 0; i < n; i++) { pos[i] = draft_past[dcur] + i; lrows[i] = i; }
  std::vector<SeqDesc> sq{SeqDesc{dcur, 0, n, draft_past[dcur]}};
  PassFlags f; f.draft = true; f.want_all_logits = true; f.want_residual = true;
  resid_off = 0;
  B200_TRY(run_rows(ids, slots.data(), pos.data(), n, sq, lrows, f));
  draft_past[dcur] += n;
  if (resid) *resid = resid_host;
  if (logits_out) *logits_out = logits_host;
  return OK;
}

int Graph::reset_slot(int slot) {
  // a fresh sequence: zero recurrent state; rings and KV cells are masked by position
  B200_CUDA(cudaSetDevice(m->device));
  for (int i = 0; i < n_dn; i++)
    B200_CUDA(cudaMemsetAsync(dn_state[i] + (size_t)slot * state_slot_stride, 0, (size_t)state_slot_stride * sizeof(float), st));
  B200_CUDA(cudaStreamSynchronize(st));
  past[slot] = 0; draft_past[slot] = 0;
  if (slot == cur) spec_n = 0;
  return OK;
}

int Graph::keep(int k) {
  // keep the first k rows of the last speculative pass (reference: llm/graph.go:1189-1233)
  if (spec_n <= 0) { set_error("keep: no speculative pass is pending"); return ESTATE; }
  if (k < 0 || k > spec_n) { set_error("keep: k is outside the pass"); return EINVAL_; }
  B200_CUDA(cudaSetDevice(m->device));
  if (k > 0) {
    for (int i = 0; i < n_dn; i++)
      B200_CUDA(cudaMemcpyAsync(dn_state[i] + (size_t)cur * state_slot_stride, dn_mid[i] + (size_t)(k - 1) * state_slot_stride,
                                (size_t)state_slot_stride * sizeof(float), cudaMemcpyDeviceToDevice, st));
    B200_CUDA(cudaStreamSynchronize(st));
  }
  past[cur] = spec_pos0 + k;
  spec_n = 0;
  return OK;
}

int Graph::checkpoint(int* handle) {
  B200_CUDA(cudaSetDevice(m->device));
  Ckpt ck; ck.slot = cur; ck.past = past[cur];
  for (int i = 0; i < n_dn; i++) {
    float *s = nullptr, *r = nullptr;
    if (cudaMalloc((void**)&s, (size_t)state_slot_stride * sizeof(float)) != cudaSuccess || cudaMalloc((void**)&r, (size_t)ring_slot_stride * sizeof(float)) != cudaSuccess) {
      if (s) cudaFree(s);
      for (float* p : ck.state) cudaFree(p);
      for (float* p : ck.ring) cudaFree(p);
      set_error("checkpoint: out of device memory"); return ENOMEM_;
    }
    ck.state.push_back(s); ck.ring.push_back(r);
    B200_CUDA(cudaMemcpyAsync(s, dn_state[i] + (size_t)cur * state_slot_stride, (size_t)state_slot_stride * sizeof(float), cudaMemcpyDeviceToDevice, st));
    B200_CUDA(cudaMemcpyAsync(r, dn_ring[i] + (size_t)cur * ring_slot_stride, (size_t)ring_slot_stride * sizeof(float), cudaMemcpyDeviceToDevice, st));
  }
  B200_CUDA(cudaStreamSynchronize(st));
  *handle = next_ckpt++;
  ckpts[*handle] = ck;
  return OK;
}

int Graph::restore(int handle) {
  auto it = ckpts.find(handle);
  if (it == ckpts.end()) { set_error("restore: unknown checkpoint"); return EINVAL_; }
  const Ckpt& ck = it->second;
  // KV cells below the mark are not copied: they must still be this slot's (llm/graph.go:1037-1062)
  if (ck.slot != cur) { set_error("restore: the checkpoint was taken in another slot"); return ESTATE; }
  if (past[cur] < ck.past) { set_error("restore: the slot no longer holds the checkpoint's tokens"); return ESTATE; }
  B200_CUDA(cudaSetDevice(m->device));
  for (int i = 0; i < n_dn; i++) {
    B200_CUDA(cudaMemcpyAsync(dn_state[i] + (size_t)cur * state_slot_stride, ck.state[i], (size_t)state_slot_stride * sizeof(float), cudaMemcpyDeviceToDevice, st));
    B200_CUDA(cudaMemcpyAsync(dn_ring[i] + (size_t)cur * ring_slot_stride, ck.ring[i], (size_t)ring_slot_stride * sizeof(float), cudaMemcpyDeviceToDevice, st));
  }
  B200_CUDA(cudaStreamSynchronize(st));
  past[cur] = ck.past;
  spec_n = 0;
  return OK;
}

int Graph::synth_context(int slot, int cells, uint64_t seed) {
  const b200_config& c = m->c;
  if (cells < 0 || cells > o.n_kv) { set_error("synth_context: more cells than the slot holds"); return ECAPACITY; }
  B200_CUDA(cudaSetDevice(m->device));
  const int64_t kvw = (int64_t)c.n_head_kv * c.head_dim, n = (int64_t)cells * kvw;
  if (n > 0) {
    float* tmp = nullptr;   // f32 staging of one layer's cells, rounded to fp16 into the cache
    B200_CUDA(cudaMalloc((void**)&tmp, (size_t)n * sizeof(float)));
    int s = OK;
    for (int i = 0; i < n_attn && s == OK; i++) {
      for (int kv = 0; kv < 2 && s == OK; kv++) {
        __half* dst = (kv ? vcache[i] : kcache[i]) + (size_t)slot * kv_slot_stride;
        s = synth_fill(tmp, n, seed * 7919 + (uint64_t)(i * 2 + kv) * 104729 + (uint64_t)slot * 1299709, 0, 0.f, kv ? 0.5f : 1.0f, st);
        if (s == OK) s = quantize_rows_device(T_F16, tmp, cells, kvw, (uint8_t*)dst, st);
      }
    }
    cudaStreamSynchronize(st);
    cudaFree(tmp);
    B200_TRY(s);
  }
  for (int i = 0; i < n_dn; i++)
    B200_TRY(synth_fill(dn_state[i] + (size_t)slot * state_slot_stride, state_slot_stride, seed * 15485863 + (uint64_t)i * 32452843 + (uint64_t)slot, 0, 0.f, 0.05f, st));
  B200_CUDA(cudaStreamSynchronize(st));
  past[slot] = cells;
  if (slot == cur) spec_n = 0;
  return OK;
}

int Graph::inject_wait_timeout() {
  B200_CUDA(cudaSetDevice(m->device));
  return launch_wait_timeout_probe(err_flag, st);
}

int Graph::residual_row(int r, float* dst) {
  if (r < 0 || r >= last_rows) { set_error("residual_row: the last pass had " + std::to_string(last_rows) + " rows"); return EINVAL_; }
  B200_CUDA(cudaSetDevice(m->device));
  B200_CUDA(cudaMemcpyAsync(dst, h + (size_t)r * m->c.n_embd, (size_t)m->c.n_embd * sizeof(float), cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaStreamSynchronize(st));
  return OK;
}

int Graph::pass_experts(int* out) {
  // the routing buffers are shared by all layers: what is readable after a pass is the last layer's selection
  const int used = m->c.n_expert_used;
  if (last_rows <= 0) { *out = 0; return OK; }
  std::vector<int32_t> tk((size_t)last_rows * used);
  B200_CUDA(cudaSetDevice(m->device));
  B200_CUDA(cudaMemcpyAsync(tk.data(), topk, tk.size() * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaStreamSynchronize(st));
  std::set<int32_t> seen(tk.begin(), tk.end());
  *out = (int)seen.size();
  return OK;
}

int64_t Graph::trace(int what, void* dst, int64_t nbytes) {
  if (!o.trace) { set_error("trace: the graph was created without trace = 1"); return -ESTATE; }
  const b200_config& c = m->c;
  const int nl = c.n_layer, M = last_rows, used = c.n_expert_used;
  const void* src; size_t row_bytes, ld_bytes;
  switch (what) {
    case 0: src = tr_mid; row_bytes = (size_t)M * c.n_embd * 4; ld_bytes = (size_t)MR * c.n_embd * 4; break;
    case 1: src = tr_out; row_bytes = (size_t)M * c.n_embd * 4; ld_bytes = (size_t)MR * c.n_embd * 4; break;
    case 2: src = tr_topk; row_bytes = (size_t)M * used * 4; ld_bytes = (size_t)MR * used * 4; break;
    case 3: src = tr_w; row_bytes = (size_t)M * (used + 1) * 4; ld_bytes = (size_t)MR * (used + 1) * 4; break;
    case 4: src = tr_margin; row_bytes = (size_t)M * 4; ld_bytes = (size_t)MR * 4; break;
    default: set_error("trace: unknown selector"); return -EINVAL_;
  }
  if ((int64_t)(row_bytes * nl) > nbytes) { set_error("trace: buffer too small"); return -EINVAL_; }
  cudaSetDevice(m->device);
  if (cudaMemcpy2D(dst, row_bytes, src, ld_bytes, row_bytes, nl, cudaMemcpyDeviceToHost) != cudaSuccess) { set_error("trace: copy failed"); return -ECUDA; }
  return (int64_t)(row_bytes * nl);
}

}  // namespace b200
