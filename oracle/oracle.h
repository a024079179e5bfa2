/* TEST INFRASTRUCTURE — C ABI of the CPU oracle. Not product code: only tests, the smoke
 * check and the benchmark's cpu-baseline leg may load this library.
 *
 * The oracle restates, on the CPU, the reference's per-block CPU code for the language
 * model's token loop (llm/deltanet.go, llm/attn.go with compress ratio 0, llm/moe.go,
 * llm/hc.go helpers, llm/sample.go Argmax) joined by a plain pre-norm residual stream
 * (attn_norm / ffn_norm / output_norm), which the reference does not have.
 *
 * PARITY PINNING: block formats, dequantisers, the Q4_K/Q5_K quantiser and the f32->f16
 * rounding are pinned against the reference's committed fixtures. Everything above the
 * block-format level (per-block tensors, logits, token ids) is "parity unpinned": the
 * reference pins those only with llama.cpp trace dumps of a 111 GB checkpoint that are
 * not available, and its Go code cannot be compiled here. */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
  const char* name;
  uint32_t type;     /* ggml type id */
  uint32_t n_dims;
  int64_t dims[4];   /* ggml order: dims[0] = row length */
  const void* data;  /* host pointer, must outlive the model */
} orc_tensor;

typedef struct {
  int32_t n_layer, n_embd, vocab;
  int32_t n_head, n_head_kv, head_dim, rope_dims;
  float rope_base, eps;
  int32_t n_expert, n_expert_used, ffn_expert, ffn_shared;
  int32_t dn_head_dim, dn_heads_k, dn_heads_v, dn_conv;
  int32_t has_draft; /* 1: blk.<n_layer>.* holds an MTP draft layer */
} orc_config;

/* Optional per-token outputs of orc_extend; any pointer may be NULL. n = tokens in the call. */
typedef struct {
  float* mix_out;  /* [n][n_layer][n_embd] token-mixer (DeltaNet / attention) output */
  float* ffn_out;  /* [n][n_layer][n_embd] MoE block output */
  float* hidden;   /* [n][n_layer][n_embd] residual stream after the layer */
  float* normed;   /* [n][n_embd] output_norm(h) before the head */
  int32_t* topk;   /* [n][n_layer][n_expert_used] routed experts in slot order */
  float* topk_w;   /* [n][n_layer][n_expert_used] normalised routing weights */
  float* margin;   /* [n][n_layer] (p_k - p_{k+1}) / p_k at the top-k boundary */
  float* logits;   /* [n][vocab] every row's logits */
  /* INPUT, optional: [n][n_layer][n_expert_used] experts to route to, in slot order, instead of the oracle's own
   * top-k (entries < 0: own choice). The oracle still reports its own selection and margin in topk / margin; the
   * routing weights are its own probabilities of the forced experts. A checker uses this to follow the routing
   * of the implementation under test across a documented near-tie, so that everything after it stays comparable. */
  const int32_t* force_topk;
} orc_trace;

typedef struct orc_model orc_model;
typedef struct orc_seq orc_seq;

/* numerics: 0 = exact f32 everywhere (the reference's `Exact`), 1 = device-like: every
 * matmul input, the SwiGLU output, K, V and the attention probabilities are rounded to
 * fp16 where the reference's device path stores them as fp16. */
enum { ORC_EXACT = 0, ORC_DEVICE_LIKE = 1 };
/* OR-ed into `numerics`: the named weight matrices are rounded to fp16 after dequantisation, as the
 * reference's many-row tensor-core GEMMs do when they unpack weights into LDS (shaders/llm_gemm.comp
 * MODE 2, shaders/llm_moe_gemm.comp:260-261, 428-430), while its decode GEMVs keep the f32 value
 * (shaders/llm_gemv.comp:133-186). Which matrices a pass rounds depends on its row count. */
enum {
  ORC_W16_DN_QKV = 1 << 8, ORC_W16_DN_GATE = 1 << 9, ORC_W16_DN_OUT = 1 << 10,
  ORC_W16_ATTN_Q = 1 << 11, ORC_W16_ATTN_K = 1 << 12, ORC_W16_ATTN_V = 1 << 13, ORC_W16_ATTN_OUT = 1 << 14,
  ORC_W16_ROUTER = 1 << 15, ORC_W16_EXPERTS = 1 << 16, ORC_W16_SHARED = 1 << 17, ORC_W16_HEAD = 1 << 18
};

uint16_t orc_f32_to_f16(float f);
float orc_f16_to_f32(uint16_t h);
int64_t orc_row_bytes(uint32_t type, int64_t n);
int orc_dequantize(uint32_t type, const void* data, int64_t n, float* dst);
/* The same elements as the many-row tensor-core kernels multiply them: fp16 values formed with the f32
 * factors carried as fp16 hi + lo pairs (the correctly rounded fp16 of orc_dequantize's value, or a neighbour). */
int orc_dequantize_w16(uint32_t type, const void* data, int64_t n, float* dst);
int orc_quantize(uint32_t type, const float* src, int64_t rows, int64_t k, void* dst);

/* y[rows] = W[rows][k] . x, serial f32 accumulation (llm/hc.go:255-264). */
int orc_matvec(uint32_t type, const void* w, int64_t rows, int64_t k, const float* x, float* y);
/* dst = src * gamma / sqrt(mean(src^2) + eps), f64 sum (llm/hc.go:176-190). */
void orc_rmsnorm(const float* src, const float* gamma, int n, float eps, float* dst);
int32_t orc_argmax(const float* logits, int64_t n);

orc_model* orc_model_create(const orc_config* cfg, const orc_tensor* tensors, int n_tensors, char* err, int err_len);
void orc_model_destroy(orc_model* m);
orc_seq* orc_seq_create(const orc_model* m);
orc_seq* orc_seq_clone(const orc_seq* s);
void orc_seq_destroy(orc_seq* s);
int32_t orc_seq_past(const orc_seq* s);

/* Advances the sequence by n tokens; logits_last (may be NULL) gets the last row's [vocab]. */
int orc_extend(const orc_model* m, orc_seq* s, const int32_t* ids, int n, int numerics,
               float* logits_last, const orc_trace* trace);

/* MTP draft layer (llm/mtp.go:352-384, 542-669 with one residual stream): one draft step.
 * h_prev [n_embd] is the trunk's (or the draft's own) residual of the previous position,
 * id the token at the next position; writes the draft's residual to h_out and its logits
 * (trunk head over the first draft_vocab ids) to logits. The draft keeps its own KV cache
 * in `ds`. */
int orc_draft_step(const orc_model* m, orc_seq* ds, const float* h_prev, int32_t id, int numerics,
                   float* h_out, float* logits, int32_t draft_vocab);
orc_seq* orc_draft_seq_create(const orc_model* m);

#ifdef __cplusplus
}
#endif
