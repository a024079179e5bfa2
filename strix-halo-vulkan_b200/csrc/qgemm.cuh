// Many-row K-quant projection as a tensor-core GEMM (tcgen05 / TMEM).
//
//   Y[t][n] = sum_k fp16(W[n][k]) * X16[t][k]      t < T rows of activations, n < N weight rows
//
// Replaces the reference's prefill projection and prefill expert kernels (shaders/llm_gemm.comp MODE 2,
// shaders/llm_moe_gemm.comp:1-110), keeping their arithmetic: K-quant weights dequantised in f32
// (d*sc*q - dmin*m, unfused) and rounded to fp16, fp16 activations, f32 accumulation.
//
// Design (B200): one CTA owns a 128-weight-row x TN-activation-row output tile whose f32 accumulator
// lives in tensor memory. Per 64-element K step
//   - warp 0 fetches the activation tile [TN][64] with one TMA tensor copy (128-byte swizzle),
//   - warps 2..5 (one thread per weight row) read the row's quant bytes with 128-bit loads, dequantise
//     64 values and store them as the swizzled K-major fp16 tile the tensor core reads,
//   - one thread of warp 1 issues four tcgen05.mma (M 128, N TN, K 16) on shared-memory descriptors and
//     commits the stage's "empty" barrier.
// After the last K step warps 2..5 read the accumulator back (tcgen05.ld, one TMEM lane = one weight
// row per thread) and write / add it to the f32 output. Every barrier wait is bounded; a wait that
// gives up sets the error word and the CTA leaves after releasing its tensor memory.
#pragma once
#include "common.cuh"

namespace b200 {

enum { GEMM_STORE = 0, GEMM_RESID = 1, GEMM_SWIGLU = 2 };

// One GEMM problem of a launch (a dense projection has one; the expert kernels one per expert).
struct GemmProblem {
  int expert;          // weights start at w + expert * expert_stride (0 for a dense projection)
  int x_row0;          // first activation row (into the tensor map's row axis)
  int count;           // activation rows
  int y_row0;          // first output row
};

struct QGemmParams {
  const GemmProblem* problems;  // device array; null: the single problem `one`
  const int* n_problems;        // device count (grouped), null: 1
  GemmProblem one;
  int max_problems;             // upper bound of *n_problems
  int max_count;                // upper bound of a problem's activation rows
  const uint8_t* w;             // weight rows [N][K] in device layout
  const uint8_t* w2;            // GEMM_SWIGLU: the `up` tensor (w is `gate`)
  int64_t expert_stride;        // bytes between consecutive experts
  int64_t stride;               // bytes per weight row
  int K, N;
  float* y; int64_t ldy;        // STORE / RESID: f32 [.][ldy]
  __half* y16;                  // SWIGLU: fp16 [.][ldy]
  const int* y_rows;            // optional: output row ids (row y_row0 + i is written to y_rows[y_row0 + i])
  int* err;
};

int launch_qgemm(uint32_t type, int epi, int tn, const QGemmParams& p, const void* tmap_host, bool pdl, cudaStream_t st);
// 128-byte tensor map of an fp16 activation buffer [rows][K] for boxes of [tn][64]; `out` is 128 bytes.
int make_x_tensor_map(const __half* x, int64_t rows, int K, int tn, void* out);

}  // namespace b200
