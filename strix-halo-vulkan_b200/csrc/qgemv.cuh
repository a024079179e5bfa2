// Fused K-quant dequant "GEMV" for 1..8 activation rows per launch column-tile.
//
// y[n][r] = sum_k W[r][k] * x16[n][k], W read as the checkpoint's own K-quant blocks.
//
// Replaces the reference's dense decode projection and decode expert FFN kernels
// (shaders/llm_gemv.comp:116-263, shaders/llm_moe_gemv.comp:586-786), keeping their
// arithmetic: activations staged as fp16, weights never rounded, f32 accumulation.
//
// Design (B200): a CTA of 8 warps owns 16-row weight tiles; its warps split K by
// super-block so that every warp issues all of its 128-bit weight loads before anything
// else. Nibbles are turned into fp16 A-fragments of mma.sync.m16n8k16 directly in
// registers as the exact integers sc*q (<= 63*31, exact in fp16); the <= 8 activation
// rows are the B-fragments, read from shared memory; the super-block scale d, and the
// min term dmin * sum_s m_s * sum_{k in s} x_k (itself one more mma over the eight
// sub-block sums, split into fp16 hi + lo parts), are applied in f32 per super-block.
// Partial sums of the K-slices are added in warp order (deterministic), and a column's
// result depends on that column alone, so a batched pass equals each row stepped alone.
//
// Q6_K has no integer sub-scale small enough: sc*(q-32) can reach 4064 and is rounded to
// fp16 above 2048 (relative error <= 2^-12 on those weights).
#pragma once
#include "common.cuh"
#include "router.cuh"
#ifdef __CUDACC__
#include <cooperative_groups.h>
#endif

namespace b200 {

constexpr int QG_WARPS = 8;
constexpr int QG_THREADS = QG_WARPS * 32;
constexpr int QG_MAXCOLS = 8;
constexpr int QG_FUSED_ROWS = 8;  // passes of at most this many rows fold norms and the MoE combine into the staging of the consumers

enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU = 2 };
enum { PRO_F16 = 0, PRO_NORM = 1, PRO_COMBINE = 2 };
constexpr int QG_COMBINE_MAX_K = 2048;  // PRO_COMBINE keeps a row's values in registers: 8 per thread
constexpr int SS_LD = 512;  // partial sums of squares kept per activation row

struct QGemvParams {
  // weights: up to 4 row segments of one fused projection (same type and K)
  const uint8_t* w[4];
  const uint8_t* w2[4];      // DUAL: the second tensor (up), same shape as w
  int seg_end[4];            // exclusive end row of each segment
  int nseg;
  int64_t stride;            // bytes per row
  int K, N;
  // grouped (per-expert) mode: entries[e] = {expert (<0: shared expert, uses ws/ws2), col_off, col_cnt, 0}
  const int4* entries;
  const int* n_entries;
  const int* cols;           // column -> x / y row ids
  int64_t expert_stride;     // bytes between consecutive experts
  const uint8_t* ws;         // shared expert weights (grouped mode)
  const uint8_t* ws2;
  int x_div;                 // grouped: x row = cols[c] / x_div
  // grouped, passes of at most QG_FUSED_ROWS rows: the router kernel stopped after the logits (route.defer); every
  // CTA selects the experts of its row itself (one warp, a few hundred instructions) instead of waiting for a last
  // router CTA to do it, and the first CTA of a row leaves the row's selection for the kernels after it
  int route_here;
  RouterParams route;
  // plain mode columns: rows [ztile*8, ztile*8+8) of M
  int M;
  int xcols;                 // columns the shared-memory layout is sized for (1..8)
  int nstage;                // weight pipeline stages in shared memory (1..QG_MAX_STAGES)
  int* err;                  // device error word: set when a bounded wait gives up
  Timeline tl;
  const int* row_ids;        // optional: plain mode column c reads row row_ids[c] and writes row c
  // activations. PRO_F16: fp16 rows in natural order. PRO_NORM: the f32 residual rows `hsrc`, normalised
  // while they are staged: x = fp16(h * gamma / sqrt(sum(ss_in[row][0..ss_n)) / K + eps)); the sums of
  // squares arrive as per-CTA partials from the kernel that wrote h, added in a fixed order
  const __half* x;
  int64_t ldx;
  const float* hsrc;
  const float* gamma;
  const float* ss_in;
  int ss_n;
  float eps;
  __half* xn_out;            // PRO_NORM / PRO_COMBINE: optional copy of the normalised rows, [.][K], written by CTA 0
  // PRO_COMBINE: the rows are the residual `hsrc` plus the MoE block's output that the expert down
  // projection left per slot: v = h + (sum_s down[row][s] * topk_w[row][s] in slot order, then the gated
  // shared expert) (reference: llm/moe.go:347-357, 403-406). Every CTA forms the rows it needs and their
  // sums of squares itself; CTA 0 also writes them to `h_out`, which must not alias `hsrc` (other CTAs
  // are still reading it).
  const float* down;         // [.][used+1][K]
  const float* topk_w;       // [.][used+1]
  int used;
  float* h_out;              // [.][K]
  float* ss_out;             // STORE / RESID: optional partial sums of squares of the rows written, [.][SS_LD], part = tile group
  // epilogue
  float* y;                  // STORE / RESID: float [.][ldy]
  int64_t ldy;
  __half* y16;               // SWIGLU: half [.][ldy]
};

__host__ __device__ inline int qg_xstride(int K) {
  int base = 2 * K + 16 * (K / 64);
  int pad = (64 - base % 128 + 128) % 128;
  return base + pad;
}
constexpr int QG_MAX_STAGES = 8;
// bytes of one pipeline stage: the tiles one CTA works on per iteration, copied whole
__host__ __device__ inline size_t qg_stage_bytes(int K, int64_t stride, bool dual) {
  const int nb = K / 256;
  const int wpt = nb >= 8 ? 8 : nb >= 4 ? 4 : nb >= 2 ? 2 : 1;
  return (size_t)(QG_WARPS / wpt) * 16 * (size_t)stride * (dual ? 2 : 1);
}
__host__ __device__ inline size_t qg_fixed_smem(int K, int xcols, bool dual) {
  size_t xs = (size_t)xcols * qg_xstride(K);
  size_t sx = (size_t)xcols * (K / 32) * 2 * sizeof(__half);  // hi and lo planes
  size_t red = (size_t)2 * QG_WARPS * 16 * 8 * sizeof(float) * (dual ? 2 : 1);  // double-buffered
  return ((xs + ((sx + 15) & ~(size_t)15) + red) + 127) & ~(size_t)127;
}

// byte offset of activation element k inside a staged row: 4-groups hold [x0,x2,x1,x3]
// (the order the nibble unpack produces pairs in), 16 bytes of padding per 64 elements.
__device__ __forceinline__ int xs_off(int k) {
  int k4 = k & 3;
  int p = (k4 == 1) ? 2 : (k4 == 2) ? 1 : k4;
  return 2 * ((k & ~3) | p) + 16 * (k >> 6);
}

struct Frag8 {  // A registers of the 8 mmas one 16-byte quad feeds, for one row
  uint32_t lo02[4], lo13[4], hi02[4], hi13[4];
};

constexpr uint32_t H2_1024 = 0x64006400u;

__device__ __forceinline__ uint32_t half2_const(float v) {
  __half2 h = __float2half2_rn(v);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ---- Q4_K ---------------------------------------------------------------------------
// Block: d, dmin (fp16), 12 bytes of packed 6-bit (scale, min), 128 bytes of nibbles
// (reference: gguf/dequant.go:238-276). Thread t of a quad takes 16-byte quads t and t+4:
// groups t>>1 and (t>>1)+2, i.e. sub-blocks {2th, 2th+1} and {4+2th, 5+2th}.
struct Q4KRow {
  uint4 hdr, qa, qb;
};

__device__ __forceinline__ void q4k_issue(Q4KRow& r, const uint8_t* blk, int t) {
  r.hdr = lds128(blk);
  r.qa = lds128(blk + 16 + 16 * t);
  r.qb = lds128(blk + 16 + 16 * (t + 4));
}

// (scale, min) byte pairs of the thread's two groups: *_a for quad a, *_b for quad b.
__device__ __forceinline__ void k4_scales(const uint4& hdr, int th, uint32_t& sc_a, uint32_t& m_a, uint32_t& sc_b, uint32_t& m_b) {
  int sel = th * 16;
  uint32_t s0 = (hdr.y >> sel) & 0xFFFFu, s1 = (hdr.z >> sel) & 0xFFFFu, s2 = (hdr.w >> sel) & 0xFFFFu;
  sc_a = s0 & 0x3F3Fu;
  m_a = s1 & 0x3F3Fu;
  sc_b = (s2 & 0x0F0Fu) | ((s0 >> 2) & 0x3030u);
  m_b = ((s2 >> 4) & 0x0F0Fu) | ((s1 >> 2) & 0x3030u);
}

// two bytes (b0, b1) -> half2(b0, b1), exact
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t two_bytes) {
  uint32_t magic = __byte_perm(two_bytes, 0x64646464u, 0x4140);  // (b0, 0x64, b1, 0x64)
  return hadd2_u(magic, half2_const(-1024.f));
}

struct ScaleConst {  // per (row, group): constants turning magic halves into sc*q
  uint32_t sl, ol, sh, oh;
};
__device__ __forceinline__ ScaleConst make_scale_const(uint32_t sc_pair_bytes) {
  uint32_t sc2 = bytes_to_half2(sc_pair_bytes);     // (sc_even, sc_odd)
  uint32_t se = __byte_perm(sc2, 0, 0x1010);        // (sc_even, sc_even)
  uint32_t so = __byte_perm(sc2, 0, 0x3232);        // (sc_odd, sc_odd)
  ScaleConst c;
  c.sl = se;
  c.ol = hmul2_u(se, half2_const(-1024.f));         // <= 64512, exact
  c.sh = hmul2_u(so, half2_const(0.0625f));
  c.oh = hmul2_u(so, half2_const(-64.f));
  return c;
}

// One 32-bit word of nibbles (bytes b0..b3): low nibbles belong to the even sub-block,
// high nibbles to the odd one. Pairs come out as (b0,b2) and (b1,b3).
__device__ __forceinline__ void q4_unpack_word(uint32_t w, const ScaleConst& c, uint32_t& lo02, uint32_t& lo13, uint32_t& hi02, uint32_t& hi13) {
  uint32_t w8 = w >> 8;
  lo02 = hfma2_u(lop3_or_and(w, 0x000F000Fu, H2_1024), c.sl, c.ol);    // (1024+q)*sc - 1024*sc
  hi02 = hfma2_u(lop3_or_and(w, 0x00F000F0u, H2_1024), c.sh, c.oh);    // (1024+16q)*sc/16 - 64*sc
  lo13 = hfma2_u(lop3_or_and(w8, 0x000F000Fu, H2_1024), c.sl, c.ol);
  hi13 = hfma2_u(lop3_or_and(w8, 0x00F000F0u, H2_1024), c.sh, c.oh);
}

// ---- Q5_K ---------------------------------------------------------------------------
// Q4_K plus a 32-byte plane of fifth bits at offset 16; nibbles start at 48
// (reference: gguf/dequant.go:282-318). Bit s of qh[l] belongs to sub-block s.
struct Q5KRow {
  uint4 hdr, qh, qa, qb;
};
__device__ __forceinline__ void q5k_issue(Q5KRow& r, const uint8_t* blk, int t) {
  r.hdr = lds128(blk);
  r.qh = lds128(blk + 16 + 16 * (t & 1));
  r.qa = lds128(blk + 48 + 16 * t);
  r.qb = lds128(blk + 48 + 16 * (t + 4));
}
// s_even = 2*group. v5 bytes = nibble | bit<<4, then (b0,b2) / (b1,b3) pairs as magic halves.
__device__ __forceinline__ void q5_unpack_word(uint32_t w, uint32_t qh, int s_even, const ScaleConst& c, uint32_t& lo02, uint32_t& lo13,
                                               uint32_t& hi02, uint32_t& hi13) {
  // bit s of every byte -> bit 4 of that byte: rotate right by (s - 4) mod 32
  uint32_t rl = __funnelshift_r(qh, qh, (s_even - 4) & 31);
  uint32_t rh = __funnelshift_r(qh, qh, (s_even - 3) & 31);
  uint32_t lo = lop3_or_andb(w & 0x0F0F0F0Fu, rl, 0x10101010u);
  uint32_t hi = lop3_or_andb((w >> 4) & 0x0F0F0F0Fu, rh, 0x10101010u);
  uint32_t neg = c.ol;  // -1024*sc_even
  lo02 = hfma2_u(__byte_perm(lo, 0x64646464u, 0x4240), c.sl, neg);
  lo13 = hfma2_u(__byte_perm(lo, 0x64646464u, 0x4341), c.sl, neg);
  // odd sub-block: constants (sc_odd, -1024*sc_odd) = (16*sh, 16*oh)
  uint32_t so = hmul2_u(c.sh, half2_const(16.f)), oo = hmul2_u(c.oh, half2_const(16.f));
  hi02 = hfma2_u(__byte_perm(hi, 0x64646464u, 0x4240), so, oo);
  hi13 = hfma2_u(__byte_perm(hi, 0x64646464u, 0x4341), so, oo);
}

// ---- Q6_K (row planes, see DTensor) ---------------------------------------------------
// Per block: ql[128], qh[64], 16 int8 scales, fp16 d (reference: gguf/dequant.go:331-356).
// Unit u = t (+4): half hf = u>>2, lh = (u>>1)&1, l0 = 16*(u&1): low nibbles are quarter lh,
// high nibbles quarter lh+2, of elements l0..l0+15; element k = 128*hf + 32*quarter + l.
struct Q6KRow {
  uint4 qla, qlb, qha, qhb, sc;
  uint32_t d;
};
__device__ __forceinline__ void q6k_issue(Q6KRow& r, const uint8_t* row, int nb, int blk, int t) {
  const uint8_t* ql = row + (size_t)blk * 128;
  const uint8_t* qh = row + (size_t)nb * 128 + (size_t)blk * 64;
  const uint8_t* sc = row + (size_t)nb * 192 + (size_t)blk * 16;
  const uint8_t* d = row + (size_t)nb * 208 + (size_t)blk * 2;
  r.qla = lds128(ql + 16 * t);
  r.qlb = lds128(ql + 64 + 16 * t);
  r.qha = lds128(qh + 16 * (t & 1));
  r.qhb = lds128(qh + 32 + 16 * (t & 1));
  r.sc = lds128(sc);
  r.d = *reinterpret_cast<const unsigned short*>(d);
}
__device__ __forceinline__ int q6_scale(const uint4& sc, int idx) {  // int8 scale idx of the block
  uint32_t w = idx < 4 ? sc.x : idx < 8 ? sc.y : idx < 12 ? sc.z : sc.w;
  return (int)(int8_t)((w >> (8 * (idx & 3))) & 0xFF);
}
__device__ __forceinline__ void q6_unpack_word(uint32_t w, uint32_t qh, int lh, uint32_t sc_lo2, uint32_t sc_hi2, uint32_t& lo02, uint32_t& lo13,
                                               uint32_t& hi02, uint32_t& hi13) {
  // 2-bit field of quarter c sits at bits 2c..2c+1 of the qh byte; move it to bits 4..5
  uint32_t rl = __funnelshift_r(qh, qh, (2 * lh - 4) & 31);
  uint32_t rh = __funnelshift_r(qh, qh, (2 * lh) & 31);  // quarter lh+2: (2*(lh+2) - 4)
  uint32_t lo = lop3_or_andb(w & 0x0F0F0F0Fu, rl, 0x30303030u);
  uint32_t hi = lop3_or_andb((w >> 4) & 0x0F0F0F0Fu, rh, 0x30303030u);
  const uint32_t off = half2_const(-1056.f);  // 1024 magic + 32 centre
  lo02 = hmul2_u(hadd2_u(__byte_perm(lo, 0x64646464u, 0x4240), off), sc_lo2);
  lo13 = hmul2_u(hadd2_u(__byte_perm(lo, 0x64646464u, 0x4341), off), sc_lo2);
  hi02 = hmul2_u(hadd2_u(__byte_perm(hi, 0x64646464u, 0x4240), off), sc_hi2);
  hi13 = hmul2_u(hadd2_u(__byte_perm(hi, 0x64646464u, 0x4341), off), sc_hi2);
}

// 8 mmas of one quad pair (rows g and g+8): words w0/w1, activations at element base kb
// (low nibbles) and kb+hi_off (high nibbles).
template <class Unpack0, class Unpack1>
__device__ __forceinline__ void quad_mmas(float (&C)[4], const uint8_t* xrow, bool live, int kb, int hi_off, const uint4& q0, const uint4& q1,
                                          Unpack0 un0, Unpack1 un1) {
  const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w}, w1[4] = {q1.x, q1.y, q1.z, q1.w};
  uint4 xl0 = make_uint4(0, 0, 0, 0), xl1 = xl0, xh0 = xl0, xh1 = xl0;
  if (live) {
    const uint8_t* pl = xrow + 2 * kb + 16 * (kb >> 6);
    const uint8_t* ph = xrow + 2 * (kb + hi_off) + 16 * ((kb + hi_off) >> 6);
    xl0 = *reinterpret_cast<const uint4*>(pl);
    xl1 = *reinterpret_cast<const uint4*>(pl + 16);
    xh0 = *reinterpret_cast<const uint4*>(ph);
    xh1 = *reinterpret_cast<const uint4*>(ph + 16);
  }
  const uint32_t bl[8] = {xl0.x, xl0.y, xl0.z, xl0.w, xl1.x, xl1.y, xl1.z, xl1.w};
  const uint32_t bh[8] = {xh0.x, xh0.y, xh0.z, xh0.w, xh1.x, xh1.y, xh1.z, xh1.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    uint32_t a_lo[4], a_hi[4];
    un0(i, w0[i], a_lo[0], a_lo[2], a_hi[0], a_hi[2]);
    un1(i, w1[i], a_lo[1], a_lo[3], a_hi[1], a_hi[3]);
    mma16816(C, a_lo, bl[2 * i], bl[2 * i + 1]);
    mma16816(C, a_hi, bh[2 * i], bh[2 * i + 1]);
  }
}

template <int TYPE>
struct RowRegs;
template <> struct RowRegs<T_Q4_K> { using type = Q4KRow; };
template <> struct RowRegs<T_Q5_K> { using type = Q5KRow; };
template <> struct RowRegs<T_Q6_K> { using type = Q6KRow; };

template <int TYPE>
__device__ __forceinline__ void issue_row(typename RowRegs<TYPE>::type& r, const uint8_t* row, int nb, int blk, int t) {
  if constexpr (TYPE == T_Q4_K) q4k_issue(r, row + (size_t)blk * 144, t);
  else if constexpr (TYPE == T_Q5_K) q5k_issue(r, row + (size_t)blk * 176, t);
  else q6k_issue(r, row, nb, blk, t);
}

// Accumulates one super-block of rows (g, g+8) into acc (C layout: [0],[1] row g cols 2t,2t+1;
// [2],[3] row g+8).
template <int TYPE>
__device__ __forceinline__ void block_accumulate(float (&acc)[4], const typename RowRegs<TYPE>::type& r0, const typename RowRegs<TYPE>::type& r1,
                                                 const uint8_t* xrow, const __half* sxrow, bool live, int blk, int t) {
  const int th = t >> 1, hb = t & 1;
  float C[4] = {0.f, 0.f, 0.f, 0.f}, C2[4] = {0.f, 0.f, 0.f, 0.f};
  if constexpr (TYPE == T_Q4_K || TYPE == T_Q5_K) {
    uint32_t sca0, ma0, scb0, mb0, sca1, ma1, scb1, mb1;
    k4_scales(r0.hdr, th, sca0, ma0, scb0, mb0);
    k4_scales(r1.hdr, th, sca1, ma1, scb1, mb1);
    const ScaleConst ca0 = make_scale_const(sca0), cb0 = make_scale_const(scb0);
    const ScaleConst ca1 = make_scale_const(sca1), cb1 = make_scale_const(scb1);
    const int ka = blk * 256 + 64 * th + 16 * hb, kb = ka + 128;
    if constexpr (TYPE == T_Q4_K) {
      quad_mmas(C, xrow, live, ka, 32, r0.qa, r1.qa,
                [&](int, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q4_unpack_word(w, ca0, a, b, c, d); },
                [&](int, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q4_unpack_word(w, ca1, a, b, c, d); });
      quad_mmas(C2, xrow, live, kb, 32, r0.qb, r1.qb,
                [&](int, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q4_unpack_word(w, cb0, a, b, c, d); },
                [&](int, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q4_unpack_word(w, cb1, a, b, c, d); });
    } else {
      const uint32_t h0[4] = {r0.qh.x, r0.qh.y, r0.qh.z, r0.qh.w}, h1[4] = {r1.qh.x, r1.qh.y, r1.qh.z, r1.qh.w};
      const int sa = 2 * th, sb = 4 + 2 * th;
      quad_mmas(C, xrow, live, ka, 32, r0.qa, r1.qa,
                [&](int i, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q5_unpack_word(w, h0[i], sa, ca0, a, b, c, d); },
                [&](int i, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q5_unpack_word(w, h1[i], sa, ca1, a, b, c, d); });
      quad_mmas(C2, xrow, live, kb, 32, r0.qb, r1.qb,
                [&](int i, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q5_unpack_word(w, h0[i], sb, cb0, a, b, c, d); },
                [&](int i, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q5_unpack_word(w, h1[i], sb, cb1, a, b, c, d); });
    }
    // min term: one mma over the 8 sub-block sums; even t carries the hi parts, odd t the lo parts
    float Cm[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t am[4] = {bytes_to_half2(ma0), bytes_to_half2(ma1), bytes_to_half2(mb0), bytes_to_half2(mb1)};
    uint32_t b0 = 0, b1 = 0;
    if (live) {
      const __half* p = sxrow + blk * 8;  // sxrow: this column's hi plane (even t) or lo plane (odd t)
      b0 = *reinterpret_cast<const uint32_t*>(p + 2 * th);
      b1 = *reinterpret_cast<const uint32_t*>(p + 4 + 2 * th);
    }
    mma16816(Cm, am, b0, b1);
#pragma unroll
    for (int i = 0; i < 4; i++) C[i] += C2[i];
    const float d0 = h2f_lo(r0.hdr.x), dm0 = h2f_hi(r0.hdr.x), d1 = h2f_lo(r1.hdr.x), dm1 = h2f_hi(r1.hdr.x);
    acc[0] = fmaf(-dm0, Cm[0], fmaf(d0, C[0], acc[0]));
    acc[1] = fmaf(-dm0, Cm[1], fmaf(d0, C[1], acc[1]));
    acc[2] = fmaf(-dm1, Cm[2], fmaf(d1, C[2], acc[2]));
    acc[3] = fmaf(-dm1, Cm[3], fmaf(d1, C[3], acc[3]));
  } else {  // Q6_K
    // unit a = t: hf 0, lh = th, l0 = 16*hb; unit b = t+4: hf 1
    const int sia = hb + 2 * th, sib = 8 + hb + 2 * th;  // scale index of the low-nibble quarter; high is +4
    auto sc2 = [](int s) { return half2_const((float)s); };
    const uint32_t sla0 = sc2(q6_scale(r0.sc, sia)), sha0 = sc2(q6_scale(r0.sc, sia + 4));
    const uint32_t slb0 = sc2(q6_scale(r0.sc, sib)), shb0 = sc2(q6_scale(r0.sc, sib + 4));
    const uint32_t sla1 = sc2(q6_scale(r1.sc, sia)), sha1 = sc2(q6_scale(r1.sc, sia + 4));
    const uint32_t slb1 = sc2(q6_scale(r1.sc, sib)), shb1 = sc2(q6_scale(r1.sc, sib + 4));
    const uint32_t ha0[4] = {r0.qha.x, r0.qha.y, r0.qha.z, r0.qha.w}, hb0[4] = {r0.qhb.x, r0.qhb.y, r0.qhb.z, r0.qhb.w};
    const uint32_t ha1[4] = {r1.qha.x, r1.qha.y, r1.qha.z, r1.qha.w}, hb1[4] = {r1.qhb.x, r1.qhb.y, r1.qhb.z, r1.qhb.w};
    const int ka = blk * 256 + 32 * th + 16 * hb, kb = ka + 128;
    quad_mmas(C, xrow, live, ka, 64, r0.qla, r1.qla,
              [&](int i, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q6_unpack_word(w, ha0[i], th, sla0, sha0, a, b, c, d); },
              [&](int i, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q6_unpack_word(w, ha1[i], th, sla1, sha1, a, b, c, d); });
    quad_mmas(C2, xrow, live, kb, 64, r0.qlb, r1.qlb,
              [&](int i, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q6_unpack_word(w, hb0[i], th, slb0, shb0, a, b, c, d); },
              [&](int i, uint32_t w, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) { q6_unpack_word(w, hb1[i], th, slb1, shb1, a, b, c, d); });
#pragma unroll
    for (int i = 0; i < 4; i++) C[i] += C2[i];
    const float d0 = __half2float(__ushort_as_half((unsigned short)r0.d)), d1 = __half2float(__ushort_as_half((unsigned short)r1.d));
    acc[0] = fmaf(d0, C[0], acc[0]);
    acc[1] = fmaf(d0, C[1], acc[1]);
    acc[2] = fmaf(d1, C[2], acc[2]);
    acc[3] = fmaf(d1, C[3], acc[3]);
  }
}


// ---- row-level helpers -------------------------------------------------------------------
// Executed by one whole CTA (QG_THREADS threads) for one activation row: the row kernels of passes of
// more than QG_FUSED_ROWS rows, the embedding gather and the draft head's input use them.

// xn[k] = fp16(h[k] * gamma[k] / sqrt(mean(h^2) + eps))   (reference: llm/hc.go:176-190)
__device__ __forceinline__ void row_rmsnorm_f16(const float* h, const float* gamma, float eps, int H, __half* xn, float* scratch) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float s = 0.f;
  for (int k = tid * 4; k < H; k += QG_THREADS * 4) {
    float4 v = *reinterpret_cast<const float4*>(h + k);
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  s = warp_sum(s);
  __syncthreads();
  if (lane == 0) scratch[warp] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < QG_WARPS; w++) tot += scratch[w];
  const float scale = 1.0f / sqrtf(tot / (float)H + eps);
  for (int k = tid * 4; k < H; k += QG_THREADS * 4) {
    float4 v = *reinterpret_cast<const float4*>(h + k);
    float4 g = *reinterpret_cast<const float4*>(gamma + k);
    __half2 a = __floats2half2_rn(v.x * scale * g.x, v.y * scale * g.y), b = __floats2half2_rn(v.z * scale * g.z, v.w * scale * g.w);
    *reinterpret_cast<uint2*>(xn + k) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
  }
}

// h += sum_k w_k * down_k (slot order) + sigmoid(gate) * shared   (reference: llm/moe.go:347-357, 403-406)
__device__ __forceinline__ void row_moe_combine(float* h, const float* down, const float* w, int used, int H) {
  for (int j = threadIdx.x * 4; j < H; j += QG_THREADS * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < used; k++) {
      const float wk = w[k];
      float4 d = __ldcg(reinterpret_cast<const float4*>(down + (size_t)k * H + j));
      acc.x += d.x * wk; acc.y += d.y * wk; acc.z += d.z * wk; acc.w += d.w * wk;
    }
    const float sg = w[used];
    float4 sh = __ldcg(reinterpret_cast<const float4*>(down + (size_t)used * H + j));
    float4 hv = *reinterpret_cast<float4*>(h + j);
    hv.x += acc.x + sh.x * sg; hv.y += acc.y + sh.y * sg; hv.z += acc.z + sh.z * sg; hv.w += acc.w + sh.w * sg;
    *reinterpret_cast<float4*>(h + j) = hv;
  }
}

// Row kernels (row_tail_kernel) for passes of more than QG_FUSED_ROWS rows
struct TailParams {
  int mode;             // 1 rmsnorm, 2 MoE combine + rmsnorm
  float* h;             // [M][H] residual stream
  const float* down;    // [M][used+1][H]
  const float* topk_w;  // [M][used+1]
  int used, H, M;
  const float* gamma;
  __half* xn;
  float eps;
};

// ---- activation staging ------------------------------------------------------------------
// Copies `ncols` fp16 activation rows into shared memory in the permuted, padded layout the
// B fragments are read in, and forms the per-sub-block sums (fp16 hi + lo planes) of the min
// term. sxs layout: [plane(2)][xcols][K/32] halves.
// sub-block sums of the staged fp16 values, as fp16 hi + lo planes
__device__ __forceinline__ void stage_sx(int K, int xcols, const uint8_t* xs, __half* sxs, int ncols, int xstride) {
  const int nsub = K / 32;
  for (int i = threadIdx.x; i < ncols * nsub; i += QG_THREADS) {
    const int c = i / nsub, s = i - c * nsub;
    const uint8_t* src = xs + (size_t)c * xstride + 64 * s + 16 * (s >> 1);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      uint4 v = *reinterpret_cast<const uint4*>(src + 16 * j);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; q++) sum += h2f_lo(w[q]) + h2f_hi(w[q]);
    }
    __half hi = __float2half_rn(sum);
    __half lo = __float2half_rn(sum - __half2float(hi));
    sxs[(size_t)c * nsub + s] = hi;
    sxs[(size_t)(xcols + c) * nsub + s] = lo;
  }
  __syncthreads();
}

// one fp16 row into the permuted layout, by threads t of nt
__device__ __forceinline__ void copy_x_row(const __half* src, int K, uint8_t* dst, int t, int nt) {
  // every CTA reads the same row: each starts at another 128-byte line so the L2 slices are not all asked for
  // the same line at the same moment
  t = (t + 8 * (int)((blockIdx.x + blockIdx.y) % (unsigned)(nt / 8))) % nt;
  for (int k = t * 8; k < K; k += nt * 8) {
    uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + k));
    uint4 o;
    o.x = __byte_perm(v.x, v.y, 0x5410); o.y = __byte_perm(v.x, v.y, 0x7632);
    o.z = __byte_perm(v.z, v.w, 0x5410); o.w = __byte_perm(v.z, v.w, 0x7632);
    *reinterpret_cast<uint4*>(dst + 2 * k + 16 * (k >> 6)) = o;
  }
}
__device__ __forceinline__ void stage_x_f16(const __half* x, int64_t ldx, int K, int xcols, uint8_t* xs, __half* sxs, int ncols, const int* xrows,
                                            int xstride, bool copied = false) {
  if (!copied) {
    for (int c = 0; c < ncols; c++) copy_x_row(x + (int64_t)xrows[c] * ldx, K, xs + (size_t)c * xstride, threadIdx.x, QG_THREADS);
    __syncthreads();
  }
  stage_sx(K, xcols, xs, sxs, ncols, xstride);
}

// 1 / sqrt(mean(h^2) + eps) of row `row` from the partial sums its producer left, by one warp
__device__ __forceinline__ float scale_from_parts(const float* ss_in, int ss_n, int64_t row, int K, float eps) {
  float s = 0.f;
  for (int i = threadIdx.x & 31; i < ss_n; i += 32) s += __ldcg(ss_in + row * SS_LD + i);
  s = warp_sum(s);
  return 1.0f / sqrtf(s / (float)K + eps);
}

// RMSNorm fused into the staging (reference: llm/hc.go:176-190): each CTA normalises the rows it needs
__device__ __forceinline__ void stage_x_norm(const QGemvParams& p, uint8_t* xs, __half* sxs, float* scratch, int ncols, const int* xrows, int xstride,
                                             bool write_xn) {
  const int warp = threadIdx.x >> 5, K = p.K;
  // element index of this thread, rotated by whole 128-byte lines per CTA (every CTA reads the same rows)
  const int tid = (threadIdx.x + 8 * (int)((blockIdx.x + blockIdx.y) & 31)) & (QG_THREADS - 1);
  // the residual values do not depend on the scale: fetch the first batch before reducing the partials
  constexpr int PRE = 2;
  float4 hpre[PRE], gpre[PRE];
  const float* src0 = p.hsrc + (int64_t)xrows[0] * K;
#pragma unroll
  for (int i = 0; i < PRE; i++) {
    const int k = tid * 4 + i * QG_THREADS * 4;
    if (k < K) { hpre[i] = __ldcg(reinterpret_cast<const float4*>(src0 + k)); gpre[i] = *reinterpret_cast<const float4*>(p.gamma + k); }
  }
  if (warp < ncols) {
    const float sc = scale_from_parts(p.ss_in, p.ss_n, xrows[warp], K, p.eps);
    if ((threadIdx.x & 31) == 0) scratch[warp] = sc;
  }
  __syncthreads();
  for (int c = 0; c < ncols; c++) {
    const int64_t row = xrows[c];
    const float* src = p.hsrc + row * (int64_t)K;
    const float scale = scratch[c];
    uint8_t* dst = xs + (size_t)c * xstride;
    int i = 0;
    for (int k = tid * 4; k < K; k += QG_THREADS * 4, i++) {
      float4 h, g;
      if (c == 0 && i < PRE) { h = hpre[i < PRE ? i : 0]; g = gpre[i < PRE ? i : 0]; }
      else { h = __ldcg(reinterpret_cast<const float4*>(src + k)); g = *reinterpret_cast<const float4*>(p.gamma + k); }
      const float v0 = h.x * scale * g.x, v1 = h.y * scale * g.y, v2 = h.z * scale * g.z, v3 = h.w * scale * g.w;
      __half2 a = __floats2half2_rn(v0, v2), b = __floats2half2_rn(v1, v3);  // stored order [x0,x2,x1,x3]
      *reinterpret_cast<uint2*>(dst + 2 * k + 16 * (k >> 6)) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
      if (write_xn) {
        __half2 n0 = __floats2half2_rn(v0, v1), n1 = __floats2half2_rn(v2, v3);
        *reinterpret_cast<uint2*>(p.xn_out + row * K + k) = make_uint2(*reinterpret_cast<uint32_t*>(&n0), *reinterpret_cast<uint32_t*>(&n1));
      }
    }
  }
  __syncthreads();
  stage_sx(K, p.xcols, xs, sxs, ncols, xstride);
}

// The MoE combine and the RMSNorm that follows it, fused into the staging: columns go four at a time,
// a thread keeping its 8 values of each in registers between the sum of squares and the scaling.
__device__ __forceinline__ void stage_x_combine(const QGemvParams& p, uint8_t* xs, __half* sxs, float* scratch, int ncols, const int* xrows,
                                                int xstride, bool writer, const float4* pre_gam = nullptr, const float4* pre_h = nullptr) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, K = p.K, slots1 = p.used + 1;
  // Element index of this thread, rotated per CTA (every CTA reads the same rows: they should not all ask for the
  // same line at the same moment). The rotation moves whole warps, and the warps' sums of squares are added in the
  // order of the elements, not of the warps: every CTA, whatever its index and whatever the launch's grid, forms the
  // same sums in the same order, so a row's normalised values do not depend on which CTA computes them.
  const int rot = (int)((blockIdx.x + blockIdx.y) & 7);
  const int et = (tid + 32 * rot) & (QG_THREADS - 1);
  const int ewarp = (warp + rot) & (QG_WARPS - 1);   // the warp-sized group of elements this warp holds
  // the norm weights are fetched with the first loads, not after the reduction
  float4 gam[2];
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int k = et * 4 + i * QG_THREADS * 4;
    gam[i] = pre_gam != nullptr ? pre_gam[i] : k < K ? *reinterpret_cast<const float4*>(p.gamma + k) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int c0 = 0; c0 < ncols; c0 += 4) {
    float4 v[4][2];
    float sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
      const int c = c0 + cc < ncols ? c0 + cc : ncols - 1;
      const int64_t row = xrows[c];
      const float* hrow = p.hsrc + row * K;
      const float* dn = p.down + row * slots1 * K;
      const float* w = p.topk_w + row * slots1;   // read by every thread alongside its rows (one trip to L2, not two)
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int k = et * 4 + i * QG_THREADS * 4;
        v[cc][i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < K && c0 + cc < ncols) {
          const float4 hv = pre_h != nullptr ? pre_h[i] : __ldcg(reinterpret_cast<const float4*>(hrow + k));
          const float4 sh = __ldcg(reinterpret_cast<const float4*>(dn + (size_t)p.used * K + k));
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 5
          for (int s = 0; s < p.used; s++) {
            const float4 d = __ldcg(reinterpret_cast<const float4*>(dn + (size_t)s * K + k));
            const float wk = __ldcg(w + s);
            acc.x += d.x * wk; acc.y += d.y * wk; acc.z += d.z * wk; acc.w += d.w * wk;
          }
          const float sg = __ldcg(w + p.used);
          float4 r;
          r.x = hv.x + (acc.x + sh.x * sg); r.y = hv.y + (acc.y + sh.y * sg); r.z = hv.z + (acc.z + sh.z * sg); r.w = hv.w + (acc.w + sh.w * sg);
          v[cc][i] = r;
          sq[cc] += (r.x * r.x + r.y * r.y) + (r.z * r.z + r.w * r.w);
          if (writer) *reinterpret_cast<float4*>(p.h_out + row * K + k) = r;
        }
      }
    }
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
      sq[cc] = warp_sum(sq[cc]);
      if (lane == 0) scratch[ewarp * 4 + cc] = sq[cc];
    }
    __syncthreads();
#pragma unroll
    for (int cc = 0; cc < 4; cc++) {
      if (c0 + cc >= ncols) break;
      float t2 = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < QG_WARPS; w2++) t2 += scratch[w2 * 4 + cc];
      const float scale = 1.0f / sqrtf(t2 / (float)K + p.eps);
      uint8_t* dst = xs + (size_t)(c0 + cc) * xstride;
      const int64_t row = xrows[c0 + cc];
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int k = et * 4 + i * QG_THREADS * 4;
        if (k < K) {
          const float4 g = gam[i];
          const float v0 = v[cc][i].x * scale * g.x, v1 = v[cc][i].y * scale * g.y, v2 = v[cc][i].z * scale * g.z, v3 = v[cc][i].w * scale * g.w;
          __half2 a = __floats2half2_rn(v0, v2), b = __floats2half2_rn(v1, v3);  // stored order [x0,x2,x1,x3]
          *reinterpret_cast<uint2*>(dst + 2 * k + 16 * (k >> 6)) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
          if (writer && p.xn_out != nullptr) {
            __half2 n0 = __floats2half2_rn(v0, v1), n1 = __floats2half2_rn(v2, v3);
            *reinterpret_cast<uint2*>(p.xn_out + row * K + k) = make_uint2(*reinterpret_cast<uint32_t*>(&n0), *reinterpret_cast<uint32_t*>(&n1));
          }
        }
      }
    }
    __syncthreads();
  }
  stage_sx(K, p.xcols, xs, sxs, ncols, xstride);
}

// ---- the kernel ----------------------------------------------------------------------------
// grid.x: persistent CTAs walking the row-tile groups; grid.y: (row, slot) of a grouped launch that
// routes for itself, else 0; grid.z: column tile of 8 activation rows (plain mode). A grouped launch over
// a work list is one row of CTAs that share the list's (entry, group) units evenly.
//
// Weights reach the SM as whole tiles (16 consecutive rows are one contiguous run of the
// checkpoint's own blocks) through cp.async.bulk into a ring of shared-memory stages, each
// completing on its mbarrier, so many tiles are in flight per SM without holding registers.
template <int TYPE, int PRO, int EPI, bool DUAL, bool GROUPED>
__global__ void __launch_bounds__(QG_THREADS, (GROUPED || TYPE == T_Q6_K) ? 3 : 2) qgemv_kernel(const QGemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int K = p.K, nb = K / 256;
  const int wpt = nb >= 8 ? 8 : nb >= 4 ? 4 : nb >= 2 ? 2 : 1;  // warps per tile (K-slices)
  const int tpc = QG_WARPS / wpt;                               // tiles per CTA and iteration
  const int xstride = qg_xstride(K);
  constexpr int RED = QG_WARPS * 128 * (DUAL ? 2 : 1);          // floats per reduction buffer
  uint8_t* xs = smem;
  __half* sxs = reinterpret_cast<__half*>(smem + (size_t)p.xcols * xstride);
  float* red = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(sxs) + (((size_t)p.xcols * (K / 32) * 2 * sizeof(__half) + 15) & ~(size_t)15));
  uint8_t* stages = smem + qg_fixed_smem(K, p.xcols, DUAL);
  const size_t tile_bytes = (size_t)16 * p.stride;
  const size_t stage_bytes = (size_t)tpc * tile_bytes * (DUAL ? 2 : 1);
  const int NS = p.nstage;
  __shared__ float scratch[4 * QG_WARPS];
  __shared__ float ssq[2][QG_WARPS][8];
  __shared__ int col_rows[QG_MAXCOLS], xrows[QG_MAXCOLS];
  __shared__ int route_expert, route_topk[32];
  __shared__ __align__(8) uint64_t full_bar[QG_MAX_STAGES];

  const int tiles = (p.N + 15) / 16;
  const int ngroups = (tiles + tpc - 1) / tpc;
  const int lt = warp / wpt, kslice = warp % wpt;

  tl_mark(p.tl, 0);
  if (tid == 0) {
    for (int s = 0; s < NS; s++) mbar_init(&full_bar[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  // What this CTA walks is a sequence of units, each one row-tile group of one weight matrix. Plain launches and
  // launches that route for themselves take the groups blockIdx.x, blockIdx.x + gridDim.x, ... of the one matrix they
  // are given. Launches over a work list cut the whole list, entries * groups units, into one contiguous run per CTA:
  // every CTA gets the same share whatever the list's length (known only on the device), a run stages the activation
  // rows of an entry once, and the weight ring runs ahead across the entries' boundaries.
  const uint8_t *wa = nullptr, *wb = nullptr;
  int ncols = 0, col_off = 0, n_units = 0;
  long long u0 = 0;
  bool active = true, x_copied = false;
  bool flat = false;
  auto own_units = [&]() { return (int)blockIdx.x < ngroups ? (ngroups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0; };
  if constexpr (GROUPED) {
    pdl_wait();  // the entries (or the logits) are written by the router kernel
    if (p.route_here) {
      // blockIdx.y = row * (used + 1) + slot: every row of the pass is routed and computed on its own, exactly as a
      // single-row pass would do it, so a pass of several rows gives each row the single-row result bit for bit
      const int used = p.route.used, slots1 = used + 1, y = blockIdx.y, row = y / slots1, slot = y - row * slots1;
      const bool writer = blockIdx.x == 0 && slot == 0;
      active = row < p.route.M;
      if (warp == 0) {
        if (active) {
          const int ex = p.route.nE <= 512 ? route_token<16>(p.route, row, lane, writer, slot, route_topk) : route_token<32>(p.route, row, lane, writer, slot, route_topk);
          if (lane == 0) route_expert = slot < used ? ex : -1;
        }
      } else if constexpr (PRO == PRO_F16) {
        // meanwhile the other warps stage the row's activations (they do not depend on the routing)
        if (active) copy_x_row(p.x + (int64_t)row * p.ldx, K, xs, tid - 32, QG_THREADS - 32);
      }
      x_copied = PRO == PRO_F16;  // for every thread alike: the barrier below covers the copy
      __syncthreads();
      if (writer && p.route.entries != nullptr) {  // the row's part of the work list: one entry per slot, the shared expert last
        if (tid < used) { p.route.entries[row * slots1 + tid] = make_int4(route_topk[tid], row * slots1 + tid, 1, 0); p.route.cols[row * slots1 + tid] = row * slots1 + tid; }
        if (tid == used) {
          p.route.entries[row * slots1 + used] = make_int4(-1, row * slots1 + used, 1, 0); p.route.cols[row * slots1 + used] = row * slots1 + used;
          if (row == 0) *p.route.n_entries = p.route.M * slots1;
        }
      }
      if (active) {
        const int ex = route_expert;
        col_off = y; ncols = 1;
        wa = ex >= 0 ? p.w[0] + (size_t)ex * p.expert_stride : p.ws;
        if constexpr (DUAL) wb = ex >= 0 ? p.w2[0] + (size_t)ex * p.expert_stride : p.ws2;
        n_units = own_units();
      }
    } else {
      flat = true;
      const long long U = (long long)*p.n_entries * ngroups, C = (long long)gridDim.x * gridDim.y, c = (long long)blockIdx.y * gridDim.x + blockIdx.x;
      u0 = c * U / C;
      n_units = (int)((c + 1) * U / C - u0);
    }
  } else {
    ncols = p.M - (int)blockIdx.z * QG_MAXCOLS;
    if (ncols > QG_MAXCOLS) ncols = QG_MAXCOLS;
    col_off = (int)blockIdx.z * QG_MAXCOLS;
    n_units = own_units();
  }
  // thread 0 is the producer: one bulk copy per tile (and per tensor when DUAL)
  auto issue_group = [&](int grp, int s, const uint8_t* ga, const uint8_t* gb) {
    uint32_t total = 0;
    for (int l = 0; l < tpc; l++) {
      const int tile = grp * tpc + l;
      if (tile < tiles) total += (uint32_t)(min(16, p.N - tile * 16) * p.stride) * (DUAL ? 2 : 1);
    }
    mbar_expect_tx(&full_bar[s], total);
    for (int l = 0; l < tpc; l++) {
      const int tile = grp * tpc + l;
      if (tile >= tiles) continue;
      const uint32_t bytes = (uint32_t)(min(16, p.N - tile * 16) * p.stride);
      const uint8_t *base = ga, *base2 = gb;
      int seg_r0 = 0;
      if constexpr (!GROUPED) {
        int sg = 0;
        while (sg + 1 < p.nseg && tile * 16 >= p.seg_end[sg]) sg++;
        seg_r0 = sg > 0 ? p.seg_end[sg - 1] : 0;
        base = p.w[sg];
        if constexpr (DUAL) base2 = p.w2[sg];
      }
      uint8_t* dst = stages + (size_t)s * stage_bytes + (size_t)l * tile_bytes * (DUAL ? 2 : 1);
      bulk_copy_g2s(dst, base + (size_t)(tile * 16 - seg_r0) * p.stride, bytes, &full_bar[s]);
      if constexpr (DUAL) bulk_copy_g2s(dst + tile_bytes, base2 + (size_t)(tile * 16 - seg_r0) * p.stride, bytes, &full_bar[s]);
    }
  };
  // unit j of this CTA goes to ring stage j % NS
  auto issue_unit = [&](int j) {
    if (flat) {
      const long long u = u0 + j;
      const int en = (int)(u / ngroups), grp = (int)(u - (long long)en * ngroups);
      const int ex = p.entries[en].x;
      const uint8_t* ga = ex >= 0 ? p.w[0] + (size_t)ex * p.expert_stride : p.ws;
      const uint8_t* gb = nullptr;
      if constexpr (DUAL) gb = ex >= 0 ? p.w2[0] + (size_t)ex * p.expert_stride : p.ws2;
      issue_group(grp, j % NS, ga, gb);
    } else {
      issue_group((int)blockIdx.x + j * (int)gridDim.x, j % NS, wa, wb);
    }
  };
  if (tid == 0)
    for (int k = 0; k < NS && k < n_units; k++) issue_unit(k);
  // Single-row combine: the norm weights and the residual row (final four kernels back) are fetched before the
  // wait, so that only the partial rows of the down projection are asked of L2 once it is over.
  float4 pre_g[2], pre_h[2];
  bool pre = false;
  if constexpr (PRO == PRO_COMBINE) {
    if (p.M == 1) {
      pre = true;
      const int et = (tid + 32 * (int)((blockIdx.x + blockIdx.y) & 7)) & (QG_THREADS - 1);   // as in stage_x_combine
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int k = et * 4 + i * QG_THREADS * 4;
        pre_g[i] = k < K ? *reinterpret_cast<const float4*>(p.gamma + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        pre_h[i] = k < K ? __ldcg(reinterpret_cast<const float4*>(p.hsrc + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  }
  if constexpr (!GROUPED) pdl_wait();
  pdl_launch();
  tl_mark(p.tl, 1);

  bool live = false;
  const uint8_t* xrow = xs;
  const __half* sxrow = sxs;
  // the activation rows of the current entry (or of this launch's column tile) into shared memory
  auto stage_rows = [&]() {
    if (tid < QG_MAXCOLS) {
      const int c = tid < ncols ? tid : 0;
      int id;
      if constexpr (GROUPED) id = p.route_here ? col_off + c : p.cols[col_off + c];
      else id = p.row_ids ? p.row_ids[col_off + c] : col_off + c;
      col_rows[tid] = id;
      xrows[tid] = GROUPED ? id / p.x_div : id;
    }
    __syncthreads();
    if constexpr (PRO == PRO_COMBINE) stage_x_combine(p, xs, sxs, scratch, ncols, xrows, xstride, blockIdx.x == 0 && blockIdx.y == 0, pre ? pre_g : nullptr, pre ? pre_h : nullptr);
    else if constexpr (PRO == PRO_NORM) stage_x_norm(p, xs, sxs, scratch, ncols, xrows, xstride, p.xn_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0);
    else stage_x_f16(p.x, p.ldx, K, p.xcols, xs, sxs, ncols, xrows, xstride, x_copied);
    live = g < ncols;
    xrow = xs + (size_t)(live ? g : 0) * xstride;
    sxrow = sxs + (size_t)((t & 1) * p.xcols + (live ? g : 0)) * (K / 32);
  };
  if (active && !flat) { stage_rows(); tl_mark(p.tl, 2); }

  int cur = -1, buf = 0;
  for (int it = 0; it < n_units; it++) {
    int grp;
    if (flat) {
      const long long u = u0 + it;
      const int en = (int)(u / ngroups);
      grp = (int)(u - (long long)en * ngroups);
      if (en != cur) {
        if (cur >= 0) __syncthreads();   // every warp is done with the rows and the row ids of the entry before
        const int4 e = p.entries[en];
        col_off = e.y; ncols = e.z; cur = en;
        stage_rows();
      }
    } else {
      grp = (int)blockIdx.x + it * (int)gridDim.x;
    }
    const int s = it % NS;
    if (!mbar_wait(&full_bar[s], (uint32_t)((it / NS) & 1))) {
      if (p.err != nullptr && tid == 0) atomicExch(p.err, 1);  // a copy never landed: report and leave
      return;
    }
    if (it == 0) tl_mark(p.tl, 3);
    float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
    const int tile = grp * tpc + lt;
    if (tile < tiles) {
      int r0 = g, r1 = g + 8;
      const int nrows = min(16, p.N - tile * 16);
      if (r0 >= nrows) r0 = nrows - 1;
      if (r1 >= nrows) r1 = nrows - 1;
      const uint8_t* tb = stages + (size_t)s * stage_bytes + (size_t)lt * tile_bytes * (DUAL ? 2 : 1);
      for (int blk = kslice; blk < nb; blk += wpt) {
        typename RowRegs<TYPE>::type a0, a1;
        issue_row<TYPE>(a0, tb + (size_t)r0 * p.stride, nb, blk, t);
        issue_row<TYPE>(a1, tb + (size_t)r1 * p.stride, nb, blk, t);
        block_accumulate<TYPE>(acc, a0, a1, xrow, sxrow, live, blk, t);
        if constexpr (DUAL) {
          issue_row<TYPE>(a0, tb + tile_bytes + (size_t)r0 * p.stride, nb, blk, t);
          issue_row<TYPE>(a1, tb + tile_bytes + (size_t)r1 * p.stride, nb, blk, t);
          block_accumulate<TYPE>(acc2, a0, a1, xrow, sxrow, live, blk, t);
        }
      }
    }
    // cross-warp reduction in warp order, double-buffered so one barrier per group suffices
    float* myred = red + (size_t)buf * RED + (size_t)warp * 128;
    myred[g * 8 + 2 * t] = acc[0]; myred[g * 8 + 2 * t + 1] = acc[1];
    myred[(g + 8) * 8 + 2 * t] = acc[2]; myred[(g + 8) * 8 + 2 * t + 1] = acc[3];
    if constexpr (DUAL) {
      float* r2 = myred + QG_WARPS * 128;
      r2[g * 8 + 2 * t] = acc2[0]; r2[g * 8 + 2 * t + 1] = acc2[1];
      r2[(g + 8) * 8 + 2 * t] = acc2[2]; r2[(g + 8) * 8 + 2 * t + 1] = acc2[3];
    }
    __syncthreads();
    // every warp is done with stage s: refill it with the unit NS iterations ahead
    if (tid == 0 && it + NS < n_units) { fence_proxy_async(); issue_unit(it + NS); }
    const float* rb = red + (size_t)buf * RED;
    float sq = 0.f;  // this thread's column is tid & 7 in every iteration
    for (int i = tid; i < tpc * 128; i += QG_THREADS) {
      const int l2 = i >> 7, rc = i & 127, r = rc >> 3, c = rc & 7;
      const int grow = (grp * tpc + l2) * 16 + r;
      if (grow >= p.N || c >= ncols) continue;
      float v = 0.f, v2 = 0.f;
      for (int w = 0; w < wpt; w++) {
        v += rb[(size_t)(l2 * wpt + w) * 128 + rc];
        if constexpr (DUAL) v2 += rb[(size_t)(QG_WARPS + l2 * wpt + w) * 128 + rc];
      }
      const int64_t orow = (!GROUPED && p.row_ids != nullptr) ? col_off + c : col_rows[c];
      if constexpr (EPI == EPI_STORE) { p.y[orow * p.ldy + grow] = v; sq += v * v; }
      else if constexpr (EPI == EPI_RESID) { const float nv = p.y[orow * p.ldy + grow] + v; p.y[orow * p.ldy + grow] = nv; sq += nv * nv; }
      else {  // SwiGLU of (gate, up) rounded to fp16 (reference: shaders/llm_moe_gemv.comp:777-781)
        float sw = v * sigmoid_acc(v) * v2;
        p.y16[orow * p.ldy + grow] = __float2half_rn(sw);
      }
    }
    if constexpr (EPI != EPI_SWIGLU && !GROUPED) {
      if (p.ss_out != nullptr) {  // sum of squares of this group's rows per column, in a fixed order
        sq += __shfl_xor_sync(0xffffffffu, sq, 8);
        sq += __shfl_xor_sync(0xffffffffu, sq, 16);
        if (lane < 8) ssq[buf][warp][lane] = sq;
        __syncthreads();
        if (tid < ncols) {
          float t2 = 0.f;
#pragma unroll
          for (int w = 0; w < QG_WARPS; w++) t2 += ssq[buf][w][tid];
          const int64_t orow = p.row_ids != nullptr ? col_off + tid : col_rows[tid];
          p.ss_out[orow * SS_LD + grp] = t2;
        }
      }
    }
    buf ^= 1;
  }
  tl_mark(p.tl, 4);
}

// -----------------------------------------------------------------------------------------
// Expert down projections of a single-row pass with the routing weights applied: part[r][row] =
// sum over the slots s of CTA r of w_s * (W_down[e_s][row] . act[s]) (reference: llm/moe.go:347-357,
// 403-406; shaders/llm_moe_combine.comp:48-63). The consumer then adds `split` partial rows instead of
// used + 1 expert rows. `split` CTAs share a tile (one (slot, super-block) unit per warp); the weighted
// sums are added in warp order. grid N / 16 * split, block QG_THREADS.
// -----------------------------------------------------------------------------------------
struct MoeDown1Params {
  const uint8_t* w;         // routed down weights [nE][N][K]
  const uint8_t* ws;        // shared expert
  int64_t expert_stride, stride;
  int K, N, used;
  const int32_t* topk;      // [rows][used]
  const float* topk_w;      // [rows][used + 1]
  const __half* act;        // [rows][used + 1][K]
  float* part;              // [rows][split][N] weighted partial sums, one row per CTA of a tile; blockIdx.y is the row
  int split;                // CTAs per tile (1..4)
  int* err;
  Timeline tl;
};
constexpr int MD_MAXSLOTS = 16;

// shared memory of a CTA that holds `maxloc` slots
__host__ __device__ inline size_t md_smem(int K, int maxloc, int64_t stride) {
  size_t xs = (size_t)maxloc * qg_xstride(K);
  size_t sx = (((size_t)maxloc * (K / 32) * 2 * sizeof(__half)) + 15) & ~(size_t)15;
  return ((xs + sx + 127) & ~(size_t)127) + (size_t)maxloc * 16 * (size_t)stride;
}

template <int TYPE>
__global__ void __launch_bounds__(QG_THREADS) moe_down1_kernel(const MoeDown1Params p) {
  // `split` CTAs share one 16-row tile: CTA r of them takes the slots s = r, r + split, ... and leaves its
  // weighted sum as partial row r; the next projection adds the partial rows to the residual while staging
  const int CL = p.split, rank = blockIdx.x % CL;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int K = p.K, nb = K / 256, slots1 = p.used + 1, xstride = qg_xstride(K);
  const int nloc = (slots1 - rank + CL - 1) / CL;   // slots of this CTA
  const int maxloc = (slots1 + CL - 1) / CL;
  uint8_t* xs = smem;
  __half* sxs = reinterpret_cast<__half*>(smem + (size_t)maxloc * xstride);
  uint8_t* tiles = smem + (((size_t)maxloc * xstride + ((((size_t)maxloc * (K / 32) * 2 * sizeof(__half)) + 15) & ~(size_t)15) + 127) & ~(size_t)127);
  const size_t tile_bytes = (size_t)16 * p.stride;
  __shared__ float red[QG_WARPS][16], wgt[MD_MAXSLOTS];
  __shared__ int expert[MD_MAXSLOTS];
  __shared__ __align__(8) uint64_t bar;
  tl_mark(p.tl, 0);
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  pdl_wait();   // the selection and the activations come from the kernel before
  pdl_launch();
  tl_mark(p.tl, 1);
  const int prow = blockIdx.y;   // row of the pass: each row is finished exactly as a single-row pass finishes its own
  const int32_t* topk = p.topk + (size_t)prow * p.used;
  const float* topk_w = p.topk_w + (size_t)prow * slots1;
  const __half* act = p.act + (size_t)prow * slots1 * K;
  if (tid < nloc) {
    const int s = rank + tid * CL;
    expert[tid] = s < p.used ? __ldcg(topk + s) : -1;
    wgt[tid] = __ldcg(topk_w + s);
  }
  __syncthreads();
  const int tile = blockIdx.x / CL, nrows = min(16, p.N - tile * 16);
  if (tid == 0 && nloc > 0) {
    mbar_expect_tx(&bar, (uint32_t)(nloc * nrows * p.stride));
    for (int i = 0; i < nloc; i++) {
      const uint8_t* base = expert[i] >= 0 ? p.w + (size_t)expert[i] * p.expert_stride : p.ws;
      bulk_copy_g2s(tiles + (size_t)i * tile_bytes, base + (size_t)tile * 16 * p.stride, (uint32_t)(nrows * p.stride), &bar);
    }
  }
  for (int i = 0; i < nloc; i++) copy_x_row(act + (size_t)(rank + i * CL) * K, K, xs + (size_t)i * xstride, tid, QG_THREADS);
  __syncthreads();
  stage_sx(K, maxloc, xs, sxs, nloc, xstride);
  tl_mark(p.tl, 2);
  bool ok = true;
  if (nloc > 0 && !mbar_wait(&bar, 0)) {
    if (p.err != nullptr && tid == 0) atomicExch(p.err, 1);  // a copy never landed: report, contribute nothing
    ok = false;
  }
  tl_mark(p.tl, 3);
  int r0 = g, r1 = g + 8;
  if (r0 >= nrows) r0 = nrows - 1;
  if (r1 >= nrows) r1 = nrows - 1;
  const bool live = g == 0;  // the single activation row sits in column 0 of the mma's N axis
  float tot0 = 0.f, tot1 = 0.f;
  for (int u = warp; ok && u < nloc * nb; u += QG_WARPS) {
    const int i = u / nb, blk = u - i * nb;
    const uint8_t* tb = tiles + (size_t)i * tile_bytes;
    typename RowRegs<TYPE>::type a0, a1;
    issue_row<TYPE>(a0, tb + (size_t)r0 * p.stride, nb, blk, t);
    issue_row<TYPE>(a1, tb + (size_t)r1 * p.stride, nb, blk, t);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    block_accumulate<TYPE>(acc, a0, a1, xs + (size_t)i * xstride, sxs + (size_t)((t & 1) * maxloc + i) * (K / 32), live, blk, t);
    tot0 = fmaf(wgt[i], acc[0], tot0);   // column 0: rows g and g + 8 on the lanes with t == 0
    tot1 = fmaf(wgt[i], acc[2], tot1);
  }
  if (t == 0) { red[warp][g] = tot0; red[warp][g + 8] = tot1; }
  __syncthreads();
  if (tid < nrows) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < QG_WARPS; w++) v += red[w][tid];
    p.part[((size_t)prow * CL + rank) * p.N + (size_t)tile * 16 + tid] = v;
  }
  tl_mark(p.tl, 4);
}

}  // namespace b200
