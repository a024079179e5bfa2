// Routing of the MoE block: parameters of the router kernel and the per-token selection,
// shared with the expert projection kernel, which repeats the selection per CTA for single-row passes.
#pragma once
#include "common.cuh"

namespace b200 {

struct RouterParams {
  const __half* xn;                                // [M][H] ffn_norm output, fp16 (when h is null)
  const float* h; const float* gamma; const float* ss_in; int ss_n; float eps;  // or: normalise the residual rows here
  __half* xn_out;                                  // ... and leave the fp16 rows for the expert kernels (CTA 0)
  DTensor router;                                  // [nE][H], F32 / F16 / Q8_0 (planes)
  const float* sh_gate;                            // [H] F32
  int M, H, nE, used;
  float* logits;       // [M][nE]
  float* probs;        // optional [M][nE]: the softmax, for inspection
  int32_t* topk;       // [M][used]
  float* topk_w;       // [M][used+1] (last = sigmoid(shared gate))
  float* margin;       // [M] optional: (p_k - p_{k+1}) / p_k
  int4* entries; int* n_entries; int* cols;   // expert work list for the grouped kernels
  int* ticket;         // [1 + ceil(M / 8)]: all rows, then one per group of eight rows
  int4* gprob;         // optional [nE]: {expert, first sorted row, rows, first sorted row} per expert (GemmProblem)
  int max_entries;
  int defer;           // 1: stop after the logits; the expert kernel that follows selects the experts itself
  int ecols;           // columns per work-list entry (8, or 4 for passes of some tens of rows; 0 means 8)
  // expert parallelism: the work list keeps the experts [e_lo, e_hi) only (e_hi == 0: all) and makes shared-expert
  // entries for the rows [sh_lo, sh_hi) only (sh_hi == 0: all rows)
  int e_lo, e_hi, sh_lo, sh_hi;
  int* n_pairs;        // optional: the number of (row, slot) pairs in cols (routed pairs of the kept experts + shared rows)
  int64_t* distinct;   // optional: += the number of experts this pass's work list touches (for the byte count of a step)
  Timeline tl;
};

#ifdef __CUDACC__
// softmax + top-k + weights of one token by one warp; a lane owns experts lane + 32*i in registers
// (reference: llm/moe.go:219-282, 426-443; shaders/llm_moe_route_decode.comp:84-213)
template <int NPL>
__device__ __forceinline__ int route_token(const RouterParams& p, int n, int lane, bool write = true, int want_slot = -1, int* sm_topk = nullptr) {
  int wanted = -1;
  const int nE = p.nE, used = p.used;
  float pv[NPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NPL; i++) {
    const int e = lane + 32 * i;
    pv[i] = e < nE ? __ldcg(p.logits + (size_t)n * nE + e) : -INFINITY;
    mx = fmaxf(mx, pv[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NPL; i++) { pv[i] = lane + 32 * i < nE ? expf(pv[i] - mx) : 0.f; sum += pv[i]; }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
#pragma unroll
  for (int i = 0; i < NPL; i++) {
    pv[i] = lane + 32 * i < nE ? pv[i] * inv : -1.f;
    if (write && p.probs != nullptr && lane + 32 * i < nE) p.probs[(size_t)n * nE + lane + 32 * i] = pv[i];
  }
  // top-k by descending probability, ties to the lower index (llm/moe.go:249-252). Probabilities
  // are non-negative, so their bit patterns order like unsigned integers: one warp-wide max of the
  // values, then one warp-wide min of the indices that hold it.
  float wsum = 0.f, last_p = 0.f, myw = 0.f;
  for (int k = 0; k <= used; k++) {
    // the lane's maximum by a tree (depth log2 NPL), then the lowest of its slots that holds it
    float t[NPL];
#pragma unroll
    for (int i = 0; i < NPL; i++) t[i] = pv[i];
#pragma unroll
    for (int w = NPL / 2; w >= 1; w >>= 1) {
#pragma unroll
      for (int i = 0; i < w; i++) t[i] = fmaxf(t[i], t[i + w]);
    }
    const float bv = t[0];
    uint32_t eq = 0;
#pragma unroll
    for (int i = 0; i < NPL; i++) eq |= (pv[i] == bv ? 1u : 0u) << i;
    const int bi = __ffs((int)eq) - 1;
    const uint32_t key = bv < 0.f ? 0u : __float_as_uint(bv) + 1u;          // taken / absent entries sort last
    const uint32_t best = __reduce_max_sync(0xffffffffu, key);
    const uint32_t mine = key == best && best != 0u ? (uint32_t)(lane + 32 * bi) : 0x7fffffffu;
    const int widx = (int)__reduce_min_sync(0xffffffffu, mine);
    const float wv = best == 0u ? -1.f : __uint_as_float(best - 1u);
    if (k == used) {
      if (write && lane == 0 && p.margin) p.margin[n] = last_p > 0.f ? (last_p - fmaxf(wv, 0.f)) / last_p : 0.f;
      break;
    }
    if ((widx & 31) == lane) {
#pragma unroll
      for (int i = 0; i < NPL; i++) if (i == (widx >> 5)) pv[i] = -1.f;
    }
    if (k == want_slot) wanted = widx;
    if (lane == k) { myw = wv; if (write) p.topk[(size_t)n * used + k] = widx; if (sm_topk != nullptr) sm_topk[k] = widx; }
    wsum += wv; last_p = wv;
  }
  // normalise the weights (llm/moe.go:256-282)
  if (wsum < 6.103515625e-5f) wsum = 6.103515625e-5f;
  if (write && lane < used) p.topk_w[(size_t)n * (used + 1) + lane] = myw / wsum;
  return wanted;
}

#endif

}  // namespace b200
