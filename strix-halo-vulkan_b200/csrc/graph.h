// The token-loop graph: per-slot sequence state, pass scheduling, CUDA-graph replay.
// Host half of the reference's llm.Graph (llm/graph.go:184-289), re-designed for one
// device arena and one captured CUDA graph per decode step.
#pragma once
#include <map>
#include <vector>

#include "ep.cuh"
#include "kernels.cuh"
#include "model.h"

namespace b200 {

struct PassFlags {
  bool want_all_logits = false;   // logits for every row, else the last row only
  bool want_residual = false;     // copy every row's residual to the host
  bool spec = false;              // speculative: write per-row state planes, leave the state untouched
  bool greedy = false;            // argmax + advance on the device (no host traffic)
  bool draft = false;             // the pass runs the draft layer only
};

struct Graph {
  Model* m = nullptr;
  b200_graph_opts o{};
  cudaStream_t st = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  int MR = 0;           // rows per pass
  int LR = 0;           // rows whose logits one pass can return
  int attn_rows = 0;    // rows a pass may send through the split-KV attention kernel (its partial results are per row)
  int n_dn = 0, n_attn = 0;
  std::vector<int> dn_index, attn_index;  // layer -> index among its kind (draft layer = last attention)
  // activations
  // the residual stream alternates between two buffers: the kernel that folds the MoE output into it
  // reads one and writes the other. h is the one the last pass finished in.
  float *hbuf[2] = {nullptr, nullptr}, *h = nullptr, *proj = nullptr, *attn_partial = nullptr, *down = nullptr, *logits = nullptr, *e_buf = nullptr, *hs_buf = nullptr;
  __half *xn16 = nullptr, *q16 = nullptr, *ctx16 = nullptr, *act16 = nullptr, *y16 = nullptr, *xcat16 = nullptr;
  // TMA tensor maps of the fp16 activation buffers for the many-row GEMM, per tile height 64 / 128 / 256
  alignas(64) unsigned char tm_xn[3][128], tm_y16[3][128], tm_ctx[3][128], tm_xperm[3][128], tm_act[3][128];
  float *dn_pre = nullptr, *dn_oraw = nullptr, *dn_ab = nullptr;   // many-token DeltaNet: scan inputs (q | k per key head, v and decay | beta per value head), raw outputs [rows][Hv*D]
  int pass_max_n = 1;                            // longest sequence of the pass being enqueued
  float* ones = nullptr;       // [8] weights 1.0 (the combine of pre-weighted partial rows)
  __half* xperm16 = nullptr;   // [rows * used][H]: activation rows in expert-sorted order
  int4* gprob = nullptr;       // [n_expert] GEMM problem per expert
  int* n_expert_dev = nullptr;
  float* ss_part = nullptr;   // [rows][SS_LD] partial sums of squares of the residual rows
  float *r_logits = nullptr, *topk_w = nullptr, *margin = nullptr;
  int32_t *topk = nullptr, *ids_dev = nullptr, *next_ids = nullptr, *history = nullptr;
  int *r_ticket = nullptr, *err_flag = nullptr, *err_host = nullptr, *n_entries = nullptr, *cols = nullptr, *row_slot = nullptr, *row_pos = nullptr, *logit_rows = nullptr, *hist_len = nullptr;
  int4* entries = nullptr;
  int64_t* distinct_dev = nullptr;     // experts streamed by the work lists built so far (device counter)
  int64_t single_row_layers = 0;       // (row, layer) pairs of fused passes, whose experts are selected inside the expert kernel
  SeqDesc* seqs = nullptr;
  float* rope = nullptr;
  int proj_ld = 0, max_entries = 0, nsplit = 0, split_cells = 0;
  // sequence state
  std::vector<float*> dn_state, dn_ring, dn_mid;   // per DeltaNet layer
  std::vector<__half*> kcache, vcache;             // per attention layer (+ draft)
  int64_t state_slot_stride = 0, ring_slot_stride = 0, kv_slot_stride = 0, mid_seq_stride = 0;
  std::vector<int> past, draft_past;
  int cur = 0;
  // speculation
  bool speculating = false, spec_first = false;
  int spec_pos0 = -1, spec_n = 0;
  int dcur = 0;        // slot whose draft cache the draft calls read and write (MTPHead.UseSlot)
  // running totals over the passes this graph ran (the reference's GraphStats: llm/graph.go:527-589)
  b200_graph_stats stats{};
  // host staging (pinned)
  uint8_t* stage = nullptr; size_t stage_bytes = 0;
  float *logits_host = nullptr, *resid_host = nullptr, *hidden_host = nullptr;
  int32_t* ids_host = nullptr;
  // trace
  float *tr_mid = nullptr, *tr_out = nullptr, *tr_w = nullptr, *tr_margin = nullptr;
  int32_t* tr_topk = nullptr;
  int last_rows = 0;
  // replay
  std::map<int, cudaGraphExec_t> decode_graphs, greedy_graphs;
  std::map<int, float*> decode_h;  // residual buffer a replayed decode graph of M rows finishes in
  long long* timeline = nullptr;  // [launch][8] phase timestamps when B200_TIMELINE is set
  int timeline_cap = 0;
  int launches = 0, last_launches = 0, draft_vocab = 0, draft_vocab_default = 0, resid_off = 0;
  float last_ms = 0.f;
  // expert parallelism (ep.cuh): exchange arena, peers' arenas as mapped here, switch
  EpParams ep{};
  uint8_t* ep_arena = nullptr;
  size_t ep_arena_bytes = 0;
  int* ep_epoch = nullptr;
  std::vector<void*> ep_mapped;
  bool ep_ready = false, ep_on = false;
  // checkpoints: DeltaNet state + rings of a slot at a token boundary
  struct Ckpt { int slot, past; std::vector<float*> state, ring; };
  std::map<int, Ckpt> ckpts;
  int next_ckpt = 1;
  std::vector<void*> allocs;

  ~Graph();
  int init(Model* model, const b200_graph_opts& opts);
  int enqueue_pass(int M, int n_seq, int n_logit_rows, const PassFlags& f);
  static int entry_cols(int M);
  int max_entries_for(int M) const;
  uint32_t fp16_weight_mask(int M, int n_logit_rows) const;
  int run_rows(const int32_t* ids, const int* slots, const int* pos, int M, const std::vector<SeqDesc>& sq, const std::vector<int>& lrows, const PassFlags& f);
  int extend(const int32_t* ids, int n, const PassFlags& f, const float** logits_out, const float** hidden_out);
  int decode_rows(const int32_t* slots, const int32_t* ids, int n, const float** logits_out);
  int generate_greedy(const int32_t* slots, const int32_t* first, int n, int steps, int32_t* out);
  int draft_rows(const float* hs, const int32_t* ids, int n, int vocab_k, const float** resid, const float** logits_out);
  int reset_slot(int slot);
  int keep(int k);
  int checkpoint(int* handle);
  int restore(int handle);
  int64_t trace(int what, void* dst, int64_t nbytes);
  int residual_row(int r, float* dst);
  int pass_experts(int* out);
  int inject_wait_timeout();
  int finish_pass();
  int ep_prepare(int rank, int world);
  int ep_export(int rank, int world, void* handle64);
  int ep_attach(const void* handles64);
  int ep_attach_local(Graph* const* peers, int world);
  int synth_context(int slot, int cells, uint64_t seed);
  template <class T> int dalloc(T** p, size_t n, bool zero = true);
};

}  // namespace b200
