/* C ABI of the B200 token-loop library (libb200llm.so).
 *
 * It replaces, for the language model's token loop only, what the reference's Go host
 * reaches through its Vulkan cgo layer: the method set of `llm.Graph` that
 * `backend/llm.go` and `backend/llm_sched.go` call. Plain pointers and sizes only; every
 * function returns a status (0 = ok) and leaves a message for b200_last_error().
 *
 * Threading: calls on one handle must be serialised by the caller (the reference runs
 * them from a single goroutine inside Device.Do, backend/device.go:23-81). The library
 * binds its device at every entry, so calls may arrive on any OS thread.
 *
 * Ownership: weights are copied to the device when added (the caller may unmap its
 * checkpoint afterwards). Returned logits / hidden pointers are pinned host buffers owned
 * by the graph, valid until the next call on the same graph (llm/graph.go:1382,1546).
 */
#ifndef B200_LLM_H
#define B200_LLM_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200_OK = 0,
  B200_EINVAL = 1,    /* refused before anything was launched: bad shape, id, slot, state */
  B200_ECAPACITY = 2, /* more rows / cells / slots than the graph was created for */
  B200_ECUDA = 3,     /* a CUDA call failed; the message carries cudaGetErrorString */
  B200_ENCCL = 4,
  B200_ETIMEOUT = 5,
  B200_ESTATE = 6,    /* call order violated (e.g. Keep without a speculative pass) */
  B200_ENOMEM = 7,
  B200_EIO = 8
};

/* Hyper-parameters, read by the host from GGUF metadata the way llm/model.go:66-96,
 * 375-407, 441-468 reads them. */
typedef struct {
  int32_t n_layer, n_embd, vocab;
  int32_t n_head, n_head_kv, head_dim, rope_dims;
  float rope_base, eps;
  int32_t n_expert, n_expert_used, ffn_expert, ffn_shared;
  int32_t dn_head_dim, dn_heads_k, dn_heads_v, dn_conv;
  int32_t has_draft; /* 1: blk.<n_layer>.* is an MTP draft layer (llm/mtp.go:36-48) */
} b200_config;

/* Mirrors llm.GraphOpts (llm/graph.go:57-126). */
typedef struct {
  int32_t max_tokens;  /* rows per pass; longer inputs are cut into chunks (MaxTokens) */
  int32_t n_kv;        /* cells per slot (NKV) */
  int32_t slots;       /* independent sequences (Slots) */
  int32_t speculative; /* keep per-row state planes so Keep(k) can pick a prefix (Speculative) */
  int32_t spec_rows;   /* largest verify pass, depth + 1 (SpecRows) */
  int32_t attn_split_cells; /* cells per split of the decode attention; 0 = default */
  int32_t use_cuda_graph;   /* 1: replay single-token passes as a captured CUDA graph (vk.Prerecorded) */
  int32_t trace;            /* 1: keep per-layer hidden states and routing for b200_graph_trace */
} b200_graph_opts;

/* Weight matrices a pass multiplies as fp16-rounded values (b200_graph_fp16_weight_mask). */
enum {
  B200_W16_DN_QKV = 1 << 8, B200_W16_DN_GATE = 1 << 9, B200_W16_DN_OUT = 1 << 10,
  B200_W16_ATTN_Q = 1 << 11, B200_W16_ATTN_K = 1 << 12, B200_W16_ATTN_V = 1 << 13, B200_W16_ATTN_OUT = 1 << 14,
  B200_W16_ROUTER = 1 << 15, B200_W16_EXPERTS = 1 << 16, B200_W16_SHARED = 1 << 17, B200_W16_HEAD = 1 << 18
};

/* Running totals of a graph (llm.GraphStats, llm/graph.go:527-589, reduced to what one CUDA stream can tell). */
typedef struct {
  int64_t passes;        /* passes run (Runs) */
  int64_t rows;          /* activation rows those passes carried */
  int64_t launches;      /* kernel launches or graph nodes issued (Dispatches) */
  double device_ms;      /* device time between the first and the last kernel of every pass (GPU) */
  double host_ms;        /* host wall clock around enqueue + wait of every pass (Submit) */
  int32_t last_rows, last_launches;
  float last_device_ms;
  int64_t expert_streams; /* routed experts whose weights the passes streamed, summed over layers and passes (what
                             a step's byte count needs: a many-slot pass touches far fewer than rows x used) */
} b200_graph_stats;

/* Graph.ExtendInput's argument (llm/graph.go:1716): token ids plus, in the reference, image spans.
 * The vision tower is not part of this library: n_images must be 0. */
typedef struct {
  const int32_t* ids;
  int32_t n;
  int32_t n_images;
} b200_input;

typedef struct b200_model b200_model;
typedef struct b200_graph b200_graph;

const char* b200_last_error(void);
int32_t b200_device_count(void);

/* ---- checkpoint (replaces the weight staging of llm.NewGraph, llm/graph.go:609-876) ---- */
int32_t b200_model_new(const b200_config* cfg, int32_t device, b200_model** out);
/* One GGUF tensor: ggml type id, dims in ggml order (dims[0] = row length), host bytes in the
 * file's own block layout (gguf.Tensor.Data, gguf/gguf.go:175-244). */
int32_t b200_model_add_tensor(b200_model* m, const char* name, uint32_t type, uint32_t n_dims, const int64_t* dims, const void* host_data);
/* A synthetic tensor generated and quantised on the device: rule 0 = normal(p0, p1),
 * rule 1 = -exp(uniform(p0, p1)). Used by the benchmark for checkpoints too large to ship. */
int32_t b200_model_add_synthetic(b200_model* m, const char* name, uint32_t type, uint32_t n_dims, const int64_t* dims, uint64_t seed, int32_t rule, float p0, float p1);
int32_t b200_model_finalize(b200_model* m);
/* Parses a GGUF v2/v3 file (gguf/gguf.go:265-403) and adds every tensor. */
int32_t b200_model_open_gguf(const char* path, int32_t device, b200_model** out);
int32_t b200_model_config(const b200_model* m, b200_config* out);
int64_t b200_model_weight_bytes(const b200_model* m);
/* Tensor bytes back in GGUF block layout (for checking synthetic checkpoints on the host). */
int64_t b200_model_tensor_bytes(const b200_model* m, const char* name);
int32_t b200_model_read_tensor(const b200_model* m, const char* name, void* dst, int64_t nbytes);
void b200_model_free(b200_model* m);

/* ---- graph: llm.Graph's method set ---------------------------------------------------- */
int32_t b200_graph_create(b200_model* m, const b200_graph_opts* opts, b200_graph** out); /* NewGraph  llm/graph.go:609 */
void b200_graph_destroy(b200_graph* g);                                                    /* Destroy   :2534 */
int32_t b200_graph_slots(const b200_graph* g);                                             /* Slots     :902 */
int32_t b200_graph_nkv(const b200_graph* g);                                               /* NKV       :881 */
int32_t b200_graph_use_slot(b200_graph* g, int32_t slot);                                  /* UseSlot   :916 */
int32_t b200_graph_reset(b200_graph* g);                                                   /* Reset     :1079 */
int32_t b200_graph_past(const b200_graph* g);
/* Declares the current slot to hold `past` cells without running them: moving `past` back is the
 * reference's Rewind of the KV cache (cells past the end are masked, llm/graph.go:1071-1078); moving
 * it forward exposes whatever the cache holds (zeros after creation) and exists for throughput
 * measurements on long contexts that are "already prefilled". The DeltaNet state is not touched. */
int32_t b200_graph_set_past(b200_graph* g, int32_t past);
/* Forward = Reset + Extend (:1695). logits: [vocab] of the last row; hidden: [n_embd], the last row of the
 * residual stream BEFORE output_norm. (The reference's Extend returns `norm`, the head mixer's output, i.e. the
 * tensor the head reads, llm/graph.go:1775; here the normalisation happens inside the head kernel's staging and
 * is never materialised, so the un-normed row is what comes back. A host that wants the reference's quantity
 * applies output_norm to it.) */
int32_t b200_graph_forward(b200_graph* g, const int32_t* ids, int32_t n, const float** logits, const float** hidden);
int32_t b200_graph_extend(b200_graph* g, const int32_t* ids, int32_t n, const float** logits, const float** hidden); /* Extend :1709 */
int32_t b200_graph_extend_input(b200_graph* g, const b200_input* in, const float** logits, const float** hidden);    /* ExtendInput :1716 */
/* Every row's logits [n][vocab] and residual [n][n_embd]; n <= spec_rows when speculating (ExtendRows :1383). */
int32_t b200_graph_extend_rows(b200_graph* g, const int32_t* ids, int32_t n, const float** logits, const float** residual);
/* Last row's logits plus every row's residual (ExtendResidual :1468). */
int32_t b200_graph_extend_residual(b200_graph* g, const int32_t* ids, int32_t n, const float** logits, const float** residual);
/* One token for each of n distinct slots in one pass; logits [n][vocab] (DecodeRows :1527, llm/batch.go:45-63). */
int32_t b200_graph_decode_rows(b200_graph* g, const int32_t* slots, const int32_t* ids, int32_t n, const float** logits);
/* Sequence checkpoints (Checkpoint/Restore :1004,:1037): DeltaNet state + conv rings of the
 * current slot; KV cells below the mark stay in place. */
int32_t b200_graph_checkpoint(b200_graph* g, int32_t* handle_out);
int32_t b200_graph_restore(b200_graph* g, int32_t handle);
int32_t b200_graph_checkpoint_free(b200_graph* g, int32_t handle);
/* Speculation (Speculate/Keep/Commit/Rewind :1122-1302). */
int32_t b200_graph_speculate(b200_graph* g, int32_t on);
int32_t b200_graph_speculating(const b200_graph* g);                                      /* Speculating :1157 */
/* SpeculateFirst (:1166): a speculative pass is then ended by Commit (all rows) or KeepFirst (row 0 only), never
 * by Rewind. Here every row of a speculative pass already leaves its own state plane, so the switch costs nothing
 * and only arms that rule. */
int32_t b200_graph_speculate_first(b200_graph* g, int32_t on);
int32_t b200_graph_keep_first(b200_graph* g);
int32_t b200_graph_keep(b200_graph* g, int32_t k);
int32_t b200_graph_commit(b200_graph* g);
int32_t b200_graph_rewind(b200_graph* g);

/* Row r of the residual the last pass left, [n_embd] into dst (ResidualRow :1454): after a one-token Extend
 * row 0 is that token's, after DecodeRows row r is slot r's. */
int32_t b200_graph_residual_row(b200_graph* g, int32_t r, float* dst);
/* Distinct experts the last pass's last layer routed to, over all its rows (PassExperts :1677). */
int32_t b200_graph_pass_experts(b200_graph* g, int32_t* out);
/* Which weight matrices a pass of `rows` rows that returns `logit_rows` rows of logits sends through the
 * tensor-core kernels, i.e. multiplies rounded to fp16 after dequantisation as the reference's many-row
 * GEMMs do (shaders/llm_gemm.comp MODE 2, shaders/llm_moe_gemm.comp:260-261); the others stay exact as in
 * its decode GEMVs. A B200_W16_* bit set. A checker that wants the pass's arithmetic mirrors this set. */
uint32_t b200_graph_fp16_weight_mask(const b200_graph* g, int32_t rows, int32_t logit_rows);
int32_t b200_graph_stats_get(const b200_graph* g, b200_graph_stats* out);                  /* Stats :527-589 */
int32_t b200_graph_stats_reset(b200_graph* g);

/* Device-resident greedy decoding: only token ids cross the bus. Each of n slots advances
 * `steps` tokens starting from first_ids; out_ids is [steps][n]. */
int32_t b200_graph_generate_greedy(b200_graph* g, const int32_t* slots, const int32_t* first_ids, int32_t n, int32_t steps, int32_t* out_ids);
/* Milliseconds of device time of the last generate_greedy call (CUDA events on its stream). */
float b200_graph_last_device_ms(const b200_graph* g);
/* Kernel launches issued by the last pass (or per step of the last generate_greedy). */
int32_t b200_graph_last_launches(const b200_graph* g);

/* Phase timestamps of the last pass, when the process was started with B200_TIMELINE set (the
 * reference keeps a GPU timestamp per dispatch, vk/shim.h:222-229): dst [launch][8] globaltimer ns,
 * phases 0 start, 1 producer done, 2 activations staged, 3 first weights landed, 4 main loop done,
 * 5 tail start, 6 tail end. Returns the number of launches written, 0 when off. */
int32_t b200_graph_timeline(b200_graph* g, int64_t* dst, int32_t max_launches);

/* Trace of the last pass (opts.trace = 1): what = 0 residual after the token mixer
 * [n_layer][rows][n_embd], 1 residual after the MoE block, 2 routed experts
 * [n_layer][rows][used] (int32), 3 routing weights [n_layer][rows][used+1], 4 top-k margin
 * [n_layer][rows]. Returns bytes written or a negative status. */
int64_t b200_graph_trace(b200_graph* g, int32_t what, void* dst, int64_t nbytes);

/* ---- expert parallelism over NVLink peer memory (no counterpart in the reference, which keeps every expert on
 * one device: llm/gpu_moe.go:693-705) -----------------------------------------------------------------------------
 * `world` ranks, one GPU each, every rank holding the checkpoint and its own slots. With the switch on, a
 * batched decode pass (b200_graph_decode_rows / _generate_greedy with the SAME row count on every rank, called at
 * the same time) runs each MoE layer expert-parallel: rank r computes the routed experts
 * [r * n_expert / world, (r + 1) * n_expert / world) for the rows of ALL ranks; rows and routing travel as peer
 * stores into buffers every rank exposes, outputs travel back the same way, and the row's owner adds them in slot
 * order, so the logits are those of the same pass with all experts local. world * rows must fit max_tokens.
 * Waits on a peer are bounded (2 s): a rank that never arrives turns the pass into B200_ETIMEOUT.
 *
 * One process per GPU: every rank calls _ep_export, the hosts exchange the 64-byte handles (any transport), every
 * rank calls _ep_attach with all of them in rank order. Ranks that share a process (one graph per device) call
 * _ep_prepare and then _ep_attach_local with the graphs in rank order instead. */
typedef struct { unsigned char bytes[64]; } b200_ep_handle;
int32_t b200_graph_ep_export(b200_graph* g, int32_t rank, int32_t world, b200_ep_handle* out);
int32_t b200_graph_ep_attach(b200_graph* g, const b200_ep_handle* handles /* [world] */);
int32_t b200_graph_ep_prepare(b200_graph* g, int32_t rank, int32_t world);
int32_t b200_graph_ep_attach_local(b200_graph* g, b200_graph* const* graphs /* [world] */, int32_t world);
int32_t b200_graph_ep_enable(b200_graph* g, int32_t on);

/* Fills `cells` cells of the current slot's KV caches (fp16, per layer: keys normal(0,1), values normal(0,0.5))
 * and its DeltaNet state (normal(0,0.05)) with seeded values and declares them prefilled. For throughput
 * measurements of long contexts that are "already there": the timed decode then reads real, non-zero caches. */
int32_t b200_graph_synth_context(b200_graph* g, int32_t cells, uint64_t seed);

/* ---- MTP draft head (llm.MTPHead, llm/mtp.go:441-760) ---------------------------------- */
/* One draft step per row: seeds from residual rows hs [n][n_embd] and token ids (the tokens
 * one position ahead), runs the draft layer on the current slot's draft cache, returns the
 * draft's residual [n][n_embd] and logits over the first `vocab_k` ids [n][vocab_k]. */
int32_t b200_draft_rows(b200_graph* g, const float* hs, const int32_t* ids, int32_t n, int32_t vocab_k, const float** residual, const float** logits);
/* The draft's lm head projects onto the first k ids only for calls that pass vocab_k = 0 (SetVocab, llm/mtp.go:675);
 * k a multiple of 16, 0 = the whole vocabulary. */
int32_t b200_draft_set_vocab(b200_graph* g, int32_t k);
/* Slot whose draft cache the draft calls use (MTPHead.UseSlot :514); b200_graph_use_slot moves it along too. */
int32_t b200_draft_use_slot(b200_graph* g, int32_t slot);
int32_t b200_draft_slots(const b200_graph* g);                                            /* Slots :512 */
int32_t b200_draft_reset(b200_graph* g);                                                  /* Reset :508 */
int32_t b200_draft_max_rows(const b200_graph* g);                                         /* MaxRows :536 */
int32_t b200_draft_wide(const b200_graph* g);                                             /* Wide / NEmbd :440: one residual stream, so both are n_embd */
int32_t b200_draft_past(const b200_graph* g);
int32_t b200_draft_rewind(b200_graph* g, int32_t past);

/* ---- unit entry points used by the parity tests ------------------------------------------ */
/* n elements of `type` in GGUF block layout -> f32 through the device layout and the device
 * dequantiser (bit-exact with gguf/dequant.go:54-100). */
int32_t b200_dequantize(uint32_t type, const void* host_data, int64_t n, float* host_out);
/* y[m][rows] = W[rows][k] . fp16(x[m][k]) through the fused K-quant projection kernel. */
int32_t b200_qgemv(uint32_t type, const void* host_w, int64_t rows, int64_t k, const float* host_x, int32_t m, float* host_y);
/* y[m][rows] = fp16(W[rows][k]) . fp16(x[m][k]) through the tensor-core (tcgen05 / TMEM) projection of
 * many-row passes; tile_rows = activation rows per tile (64, 128 or 256). The reference's prefill GEMM
 * arithmetic: dequantised weights rounded to fp16 (shaders/llm_gemm.comp MODE 2). */
int32_t b200_qgemm(uint32_t type, const void* host_w, int64_t rows, int64_t k, const float* host_x, int32_t m, int32_t tile_rows, float* host_y);
/* No counterpart in the reference. The same projection for callers that cannot allocate device
 * memory when they need it: a latency-critical thread that must not block on the allocator's lock
 * (cudaMalloc / cudaFree serialise on it and may synchronise the device), or a process whose
 * device memory was budgeted up front. All pointers are DEVICE pointers the caller already owns;
 * the fp16 staging of the activations (256 KiB) and the word a timed-out wait is reported through
 * live in file-scope device arrays that every GPU loading the library holds until exit.
 * Limits: Q4_K / Q5_K weights in checkpoint block layout, 16-byte aligned; m <= 8 rows; k a
 * multiple of 256, at most 16384; and m staged rows of k elements plus one stage of 16 weight rows
 * must fit the kernel's 220 KiB of shared memory (e.g. Q4_K: 8 rows up to k = 7680, 1 row up to
 * k = 16384; Q5_K: 8 rows up to k = 7168, 1 row up to k = 16128). Anything larger is refused with
 * B200_ECAPACITY and a message that names the largest m that fits that k.
 * The work is queued on the legacy default stream and the call returns after it is done; what the
 * caller queued on a non-blocking stream to produce dev_x must have finished before the call. The
 * first call on a device looks the arrays' addresses up: make it before any stream capture. All
 * calls share the arrays, which keep the last call's contents (the error word is cleared by every
 * call, the staging is overwritten where it is read), so calls that overlap on the device race.
 * Calls no cudaMalloc, cudaFree or other allocating routine. B200_ETIMEOUT: a bounded wait inside
 * the kernel gave up and dev_y is not valid. */
int32_t b200_qgemv_static(uint32_t type, const void* dev_w, int64_t rows, int64_t k, const float* dev_x, int32_t m, float* dev_y);
/* Failure-detection check that faults nothing: queues, on the graph's stream, a small kernel whose bounded
 * wait can never be satisfied (its barrier expects more bytes than are copied). It gives up after its limit,
 * sets the graph's error word and returns; the next pass on the graph then reports B200_ETIMEOUT and clears
 * the word, after which the graph is usable again. */
int32_t b200_graph_inject_wait_timeout(b200_graph* g);
/* The repo's quantiser on the device (llm/quantk.go:87-179): rows x k f32 -> GGUF blocks. */
int32_t b200_quantize(uint32_t type, const float* host_src, int64_t rows, int64_t k, void* host_dst);

#ifdef __cplusplus
}
#endif
#endif
