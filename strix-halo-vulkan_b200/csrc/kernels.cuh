// Launch wrappers of the token-loop kernels (definitions in kernels.cu / qgemv.cu).
#pragma once
#include "common.cuh"
#include "qgemv.cuh"
#include "qgemm.cuh"

namespace b200 {

// ---- layout -----------------------------------------------------------------------------
int64_t device_row_stride(uint32_t type, int64_t k);
// GGUF rows -> device rows (re-lays Q6_K / Q8_0 rows as planes; plain copy otherwise) and back.
int repack_rows(uint32_t type, int64_t k, int64_t rows, const uint8_t* gguf_dev, uint8_t* dst_dev, cudaStream_t st);
int unpack_rows(uint32_t type, int64_t k, int64_t rows, const uint8_t* dev, uint8_t* gguf_dev, cudaStream_t st);
// f32 values of rows [row0, row0+rows) of a device tensor (bit-exact with gguf/dequant.go)
int dequant_rows(const DTensor& t, int64_t row0, int64_t rows, float* out, cudaStream_t st);

// ---- pass description ---------------------------------------------------------------------
// A pass advances `n_seq` sequences; sequence i owns activation rows [row0, row0+n) and
// its tokens sit at positions pos0, pos0+1, ... of slot `slot`.
struct SeqDesc {
  int slot, row0, n, pos0;
};

struct EmbedParams {
  DTensor embd;
  const int32_t* ids;  // [M]
  float* h;            // [M][H]
  int M, H;
  const float* gamma;  // optional: the first consumer's norm weights
  __half* xn;          // [M][H] fp16 normalised rows (when gamma is given)
  float eps;
  float* ss_out;       // optional: sum of squares of each row, [M][SS_LD] part 0
};
int launch_embed(const EmbedParams& p, cudaStream_t st);

// K-quant projections; `pdl` marks the launch as a programmatic dependent of the previous kernel.
int launch_qgemv(uint32_t type, int pro, int epi, bool dual, bool grouped, const QGemvParams& p, int max_entries, bool pdl, cudaStream_t st);
// passes of at most QG_FUSED_ROWS rows: per row, every selected expert's down projection with the routing weights applied,
// left as a few partial rows for the next projection to add
int launch_moe_down1(uint32_t type, const MoeDown1Params& p, int rows, bool pdl, cudaStream_t st);
int moe_down1_split(int used, int K);
int qgemv_groups(int K, int N);
int launch_row_tail(const TailParams& tp, bool pdl, cudaStream_t st);
// rows of a fused pass: residual + expert partial rows + next RMSNorm, once per row (hsrc, down, topk_w, used, gamma, h_out, xn_out)
int launch_combine_rows(const QGemvParams& p, bool pdl, cudaStream_t st);
int launch_concat_norm(const float* e, const float* hs, const float* enorm, const float* hnorm, float eps, int H, int M, __half* xcat, bool pdl, cudaStream_t st);

int launch_router(const RouterParams& p, bool pdl, cudaStream_t st);
// selection + work list only, for passes whose logits come from launch_qgemm (the shared gate is computed here)
bool router_mma_fits(const RouterParams& p);
int launch_router_mma(const RouterParams& p, bool pdl, cudaStream_t st);
int launch_route_rows(const RouterParams& p, bool pdl, cudaStream_t st);
// work list only, from routing that is already in p.topk (expert-parallel passes: the gathered routing)
int launch_ep_worklist(const RouterParams& p, bool pdl, cudaStream_t st);
int launch_moe_gather(const __half* xn, const int* cols, int pairs, int slots1, int H, __half* xperm, bool pdl, cudaStream_t st);


struct DnStepParams {
  const float* proj; int64_t ldp;            // [M][ldp]: q | k | v | z
  const __half* xn;                          // [M][H] normalised block input (fp16)
  const float *alpha_w, *beta_w;             // [Hv][H] F32
  const float *conv_w, *ssm_a, *dt_bias;     // [cw][K], [Hv], [Hv]
  float* state;                              // [slots][Hv][D][D], s[j][i] = S[i][j]
  int64_t state_slot_stride;
  float* ring;                               // [slots][Hv*4][DN_RING][DN_RING_W]
  int64_t ring_slot_stride;
  const SeqDesc* seqs; int n_seq;
  const float* norm_w;                       // [D] ssm_norm, shared by all heads
  __half* y16;                               // [M][Hv*D] gated-norm output: fp16(rms(o) * norm_w * sigmoid(z))
  float* mid;                                // speculation: [n_seq][rows][Hv][D][D] state after each token; the slot's own state is then left untouched
  int64_t mid_stride, mid_seq_stride;        // floats between consecutive rows / sequences of mid
  // many-token form (launch_dn_scan): state-independent inputs of the scan for every row, and its raw outputs
  float* pre;                                // [Hk][pre_rows][256] q | k, [Hv][pre_rows][128] v, [Hv][pre_rows][2] decay | beta
  int64_t pre_rows;
  float* o_raw;                              // [M][Hv*D]
  float* ab;                                 // [M][2*Hv] alpha | beta projections of every row
  int H, Hk, Hv, D, conv;
  float eps;
  Timeline tl;
};
constexpr int DN_RING = 8;      // positions kept per ring
constexpr int DN_RING_W = 288;  // conv inputs per CTA: q 128 | k 128 | v 32
int launch_dn_step(const DnStepParams& p, bool pdl, cudaStream_t st);
// four launches: alpha / beta projections of all rows, the rest of the state-independent part, the scan, the gated
// norm (max_n = longest sequence)
int launch_dn_scan(const DnStepParams& p, int M, int max_n, bool pdl, cudaStream_t st);

struct AttnParams {
  const float* proj; int64_t ldp;            // [M][ldp]: per head (q | gate) x Hq, then k, then v
  const float *q_norm, *k_norm;              // [hd]
  const float* rope;                         // [n_kv][half][2] cos, sin
  __half *kcache, *vcache;                   // [slots][n_kv][Hkv][hd]
  int64_t slot_stride;                       // halves per slot
  const int* row_slot; const int* row_pos;   // [M]
  __half* q16;                               // [M][Hq][hd]
  float* partial;                            // [M][Hq][nsplit][hd+2]
  __half* ctx16;                             // [M][Hq*hd]
  int M, Hq, Hkv, hd, rope_dims, n_kv, split_cells, nsplit;
  int rope_off;                              // rotary position = cell + rope_off (1 for the draft layer)
  int one_row_per_seq;                       // every sequence has exactly one row in this pass (plain decode)
  float eps;
  int* err;                                  // device error word: set when a bounded wait gives up
  Timeline tl;
};
int launch_attn_pack(const AttnParams& p, bool pdl, cudaStream_t st);
int launch_attn_decode(const AttnParams& p, bool pdl, cudaStream_t st);
int launch_attn_merge(const AttnParams& p, bool pdl, cudaStream_t st);
// tiled causal attention of a many-row pass of one sequence, straight to the gated context rows (no partials, no merge)
bool attn_prefill_fits(const AttnParams& p);
int launch_attn_prefill(const AttnParams& p, bool pdl, cudaStream_t st);

// a one-thread kernel whose bounded wait must run out: sets *err (failure detection without a fault)
int launch_wait_timeout_probe(int* err, cudaStream_t st);

int launch_argmax(const float* logits, int M, int V, int32_t* out, bool pdl, cudaStream_t st);

// rows of the same pass: ids[i] = next[i], pos[i] += 1 (device-resident greedy loop)
int launch_advance(int32_t* ids, const int32_t* next, int* row_pos, SeqDesc* seqs, int M, int32_t* history, int* hist_len, cudaStream_t st);

}  // namespace b200
