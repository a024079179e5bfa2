// TEST INFRASTRUCTURE — CPU oracle, not product code.
//
// Block formats, dequantisers and quantisers of the GGUF K-quant family, restated on
// the CPU from the reference's own Go code. Only tests, the smoke check and the
// benchmark's cpu-baseline leg may link this.
//
// Pinned against the reference's committed known-answer fixtures:
//   gguf/testdata/dequant_{in,ref}.bin  (bit-exact, all 11 formats)
//   llm/testdata/quant_{in,ref}.bin     (Q4_K / Q5_K round trip, equal after fp16 rounding)
//   safetensors/testdata/f32_to_f16.txt (f32 -> f16 round-to-nearest-even)
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace orc {

// ggml type ids (gguf/gguf.go:53-88).
enum GgmlType : uint32_t {
  T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8,
  T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ4_NL = 20, T_BF16 = 30,
};

// Block geometry (gguf/gguf.go:101-134): elements per block, bytes per block.
inline bool block_geometry(uint32_t t, int* elems, int* nbytes) {
  switch (t) {
    case T_F32: *elems = 1; *nbytes = 4; return true;
    case T_F16: *elems = 1; *nbytes = 2; return true;
    case T_BF16: *elems = 1; *nbytes = 2; return true;
    case T_Q4_1: *elems = 32; *nbytes = 20; return true;
    case T_Q5_0: *elems = 32; *nbytes = 22; return true;
    case T_Q5_1: *elems = 32; *nbytes = 24; return true;
    case T_Q8_0: *elems = 32; *nbytes = 34; return true;
    case T_IQ4_NL: *elems = 32; *nbytes = 18; return true;
    case T_Q4_K: *elems = 256; *nbytes = 144; return true;
    case T_Q5_K: *elems = 256; *nbytes = 176; return true;
    case T_Q6_K: *elems = 256; *nbytes = 210; return true;
  }
  return false;
}

inline int64_t row_bytes(uint32_t t, int64_t n) {
  int e, b;
  if (!block_geometry(t, &e, &b) || n % e) return -1;
  return n / e * b;
}

// ---- fp16 (safetensors/safetensors.go:425,472; llm/hc.go:316-360) -------------------

inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal half: renormalise
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400));
      bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3ff) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | man << 13;
  } else {
    bits = sign | (exp + 112) << 23 | man << 13;
  }
  float f; memcpy(&f, &bits, 4); return f;
}

// Round-to-nearest-even, subnormals kept, overflow to infinity.
inline uint16_t f32_to_f16(float f) {
  uint32_t b; memcpy(&b, &f, 4);
  uint16_t sign = (uint16_t)((b >> 16) & 0x8000);
  int32_t exp = (int32_t)((b >> 23) & 0xff) - 127;
  uint32_t man = b & 0x7fffff;
  if (exp == 128) return sign | 0x7c00 | (man ? (0x200 | (uint16_t)(man >> 13)) : 0);
  if (exp > 15) return sign | 0x7c00;
  if (exp < -25) return sign;
  if (exp < -14) {
    uint32_t shift = (uint32_t)(-exp - 14) + 13;
    uint32_t full = man | 0x800000;
    uint32_t q = full >> shift, rem = full & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    return sign | (uint16_t)q;
  }
  uint32_t q = man >> 13, rem = man & 0x1fff;
  uint32_t e = (uint32_t)(exp + 15) << 10;
  uint32_t v = e + q;  // a mantissa carry bumps the exponent (and may reach inf)
  if (rem > 0x1000 || (rem == 0x1000 && (q & 1))) v++;
  return sign | (uint16_t)v;
}

inline float f16_round(float x) { return f16_to_f32(f32_to_f16(x)); }

inline float bf16_to_f32(uint16_t h) {
  uint32_t b = (uint32_t)h << 16; float f; memcpy(&f, &b, 4); return f;
}

inline float rd_f16(const uint8_t* p) { uint16_t h; memcpy(&h, p, 2); return f16_to_f32(h); }

// ---- dequantisers (gguf/dequant.go:128-356) -----------------------------------------

static const int8_t kIQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// ggml's get_scale_min_k4 (gguf/dequant.go:238-243).
inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
  if (j < 4) { *sc = q[j] & 63; *m = q[j + 4] & 63; }
  else { *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

inline void dequant_q4_k(const uint8_t* blk, float* out) {
  float d = rd_f16(blk), dmin = rd_f16(blk + 2);
  const uint8_t* scales = blk + 4; const uint8_t* q = blk + 16;
  int is = 0;
  for (int j = 0; j < 256; j += 64) {
    uint8_t sc, m;
    scale_min_k4(is, scales, &sc, &m); float d1 = d * (float)sc, m1 = dmin * (float)m;
    scale_min_k4(is + 1, scales, &sc, &m); float d2 = d * (float)sc, m2 = dmin * (float)m;
    for (int l = 0; l < 32; l++) *out++ = d1 * (float)(q[l] & 0xF) - m1;
    for (int l = 0; l < 32; l++) *out++ = d2 * (float)(q[l] >> 4) - m2;
    q += 32; is += 2;
  }
}

inline void dequant_q5_k(const uint8_t* blk, float* out) {
  float d = rd_f16(blk), dmin = rd_f16(blk + 2);
  const uint8_t* scales = blk + 4; const uint8_t* qh = blk + 16; const uint8_t* ql = blk + 48;
  int is = 0; uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < 256; j += 64) {
    uint8_t sc, m;
    scale_min_k4(is, scales, &sc, &m); float d1 = d * (float)sc, m1 = dmin * (float)m;
    scale_min_k4(is + 1, scales, &sc, &m); float d2 = d * (float)sc, m2 = dmin * (float)m;
    for (int l = 0; l < 32; l++) *out++ = d1 * (float)((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
    for (int l = 0; l < 32; l++) *out++ = d2 * (float)((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
    ql += 32; is += 2; u1 <<= 2; u2 <<= 2;
  }
}

inline void dequant_q6_k(const uint8_t* blk, float* out) {
  const uint8_t* ql = blk; const uint8_t* qh = blk + 128; const int8_t* sc = (const int8_t*)(blk + 192);
  float d = rd_f16(blk + 208);
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; l++) {
      int is = l / 16;
      uint8_t h = qh[n / 4 + l];
      int q1 = (int)((ql[n / 2 + l] & 0xF) | (((h >> 0) & 3) << 4)) - 32;
      int q2 = (int)((ql[n / 2 + l + 32] & 0xF) | (((h >> 2) & 3) << 4)) - 32;
      int q3 = (int)((ql[n / 2 + l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
      int q4 = (int)((ql[n / 2 + l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32;
      const int8_t* g = sc + n / 16 + is;
      out[n + l] = d * (float)g[0] * (float)q1;
      out[n + l + 32] = d * (float)g[2] * (float)q2;
      out[n + l + 64] = d * (float)g[4] * (float)q3;
      out[n + l + 96] = d * (float)g[6] * (float)q4;
    }
  }
}

inline void dequant_q8_0(const uint8_t* blk, float* out) {
  float d = rd_f16(blk);
  for (int j = 0; j < 32; j++) out[j] = (float)(int8_t)blk[2 + j] * d;
}

inline void dequant_q4_1(const uint8_t* blk, float* out) {
  float d = rd_f16(blk), m = rd_f16(blk + 2);
  for (int j = 0; j < 16; j++) {
    out[j] = (float)(blk[4 + j] & 0x0F) * d + m;
    out[j + 16] = (float)(blk[4 + j] >> 4) * d + m;
  }
}

inline void dequant_q5_0(const uint8_t* blk, float* out) {
  float d = rd_f16(blk); uint32_t qh; memcpy(&qh, blk + 2, 4);
  for (int j = 0; j < 16; j++) {
    uint8_t xh0 = (uint8_t)(((qh >> j) << 4) & 0x10), xh1 = (uint8_t)((qh >> (j + 12)) & 0x10);
    out[j] = (float)((int)((blk[6 + j] & 0x0F) | xh0) - 16) * d;
    out[j + 16] = (float)((int)((blk[6 + j] >> 4) | xh1) - 16) * d;
  }
}

inline void dequant_q5_1(const uint8_t* blk, float* out) {
  float d = rd_f16(blk), m = rd_f16(blk + 2); uint32_t qh; memcpy(&qh, blk + 4, 4);
  for (int j = 0; j < 16; j++) {
    uint8_t xh0 = (uint8_t)(((qh >> j) << 4) & 0x10), xh1 = (uint8_t)((qh >> (j + 12)) & 0x10);
    out[j] = (float)((blk[8 + j] & 0x0F) | xh0) * d + m;
    out[j + 16] = (float)((blk[8 + j] >> 4) | xh1) * d + m;
  }
}

inline void dequant_iq4_nl(const uint8_t* blk, float* out) {
  float d = rd_f16(blk);
  for (int j = 0; j < 16; j++) {
    out[j] = d * (float)kIQ4NL[blk[2 + j] & 0xF];
    out[j + 16] = d * (float)kIQ4NL[blk[2 + j] >> 4];
  }
}

// n elements of `type` at `data` -> dst. Returns 0, or -1 for an unknown type or a
// count that is not a whole number of blocks (gguf/dequant.go:54-100).
// ---- weights as the many-row tensor-core kernels see them -------------------------------
// The reference's many-row GEMMs unpack a weight slab into LDS as `float16_t(ds * nib - dm)`: the f32 value
// rounded to fp16 once (shaders/llm_moe_gemm.comp:260-261, 428-430). The CUDA kernels form the same value in
// fp16 arithmetic, with the two f32 factors d*sc and dmin*m carried as fp16 hi + lo pairs:
//   w = fp16( fp16(q*hi(ds) + hi(-dm)) + fp16(q*lo(ds) + lo(-dm)) )
// (each fp16(...) one fused multiply-add rounded once). That lands on the correctly rounded value or on a
// neighbour of it (checked against the plain rounding over the reference's golden blocks by the oracle's
// own tests), and it is what this function restates, so that a many-row pass is compared with an oracle that
// multiplies bit-identical weights.
inline float f16_round_d(double x) {
  if (x == 0.0 || !std::isfinite(x)) return (float)x;
  int e;
  std::frexp(x, &e);                      // |x| = f * 2^e, f in [0.5, 1)
  int q = e - 11;                         // quantum 2^q keeps 11 significant bits
  if (q < -24) q = -24;                   // subnormal range of fp16
  const double r = std::nearbyint(std::ldexp(x, -q));   // ties to even
  return (float)std::ldexp(r, q);
}
inline void h16_split(float v, float* hi, float* lo) { *hi = f16_round(v); *lo = f16_round(v - *hi); }
inline float w16_k(int q, float dh, float dl, float nh, float nl) {
  const float t1 = f16_round_d((double)q * dh + nh), t2 = f16_round_d((double)q * dl + nl);
  return f16_round_d((double)t1 + (double)t2);
}
inline float w16_s(int a, float dh, float dl) { return f16_round_d((double)a * dh + (double)f16_round_d((double)a * dl)); }

inline void dequant_w16_q45_k(const uint8_t* blk, float* out, bool q5) {
  float d = rd_f16(blk), dmin = rd_f16(blk + 2);
  const uint8_t* scales = blk + 4; const uint8_t* qh = blk + 16; const uint8_t* ql = blk + (q5 ? 48 : 16);
  for (int j = 0; j < 4; j++) {
    for (int half = 0; half < 2; half++) {
      uint8_t sc, m;
      scale_min_k4(2 * j + half, scales, &sc, &m);
      float dh, dl, nh, nl;
      h16_split(d * (float)sc, &dh, &dl);
      h16_split(-(dmin * (float)m), &nh, &nl);
      for (int l = 0; l < 32; l++) {
        int q = half ? (ql[32 * j + l] >> 4) : (ql[32 * j + l] & 0xF);
        if (q5 && ((qh[l] >> (2 * j + half)) & 1)) q += 16;
        out[64 * j + 32 * half + l] = w16_k(q, dh, dl, nh, nl);
      }
    }
  }
}
inline void dequant_w16_q6_k(const uint8_t* blk, float* out) {
  const uint8_t* ql = blk; const uint8_t* qh = blk + 128; const int8_t* sc = (const int8_t*)(blk + 192);
  float d = rd_f16(blk + 208);
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; l++) {
      int is = l / 16;
      uint8_t h = qh[n / 4 + l];
      const int q[4] = {(int)((ql[n / 2 + l] & 0xF) | (((h >> 0) & 3) << 4)) - 32, (int)((ql[n / 2 + l + 32] & 0xF) | (((h >> 2) & 3) << 4)) - 32,
                        (int)((ql[n / 2 + l] >> 4) | (((h >> 4) & 3) << 4)) - 32, (int)((ql[n / 2 + l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32};
      const int8_t* g = sc + n / 16 + is;
      for (int k = 0; k < 4; k++) {
        float dh, dl;
        h16_split(d * (float)g[2 * k], &dh, &dl);
        out[n + l + 32 * k] = w16_s(q[k], dh, dl);
      }
    }
  }
}
// n elements of `type` as fp16-representable weights; types the tensor-core kernels do not take are rounded once.
inline int dequantize_w16(uint32_t type, const void* data, int64_t n, float* dst);

inline int dequantize(uint32_t type, const void* data, int64_t n, float* dst) {
  int e, nb;
  if (!block_geometry(type, &e, &nb) || n % e) return -1;
  const uint8_t* p = (const uint8_t*)data;
  int64_t blocks = n / e;
  switch (type) {
    case T_F32: memcpy(dst, p, (size_t)n * 4); return 0;
    case T_F16: for (int64_t i = 0; i < n; i++) dst[i] = rd_f16(p + 2 * i); return 0;
    case T_BF16: for (int64_t i = 0; i < n; i++) { uint16_t h; memcpy(&h, p + 2 * i, 2); dst[i] = bf16_to_f32(h); } return 0;
    case T_Q8_0: for (int64_t b = 0; b < blocks; b++) dequant_q8_0(p + b * 34, dst + b * 32); return 0;
    case T_Q4_1: for (int64_t b = 0; b < blocks; b++) dequant_q4_1(p + b * 20, dst + b * 32); return 0;
    case T_Q5_0: for (int64_t b = 0; b < blocks; b++) dequant_q5_0(p + b * 22, dst + b * 32); return 0;
    case T_Q5_1: for (int64_t b = 0; b < blocks; b++) dequant_q5_1(p + b * 24, dst + b * 32); return 0;
    case T_IQ4_NL: for (int64_t b = 0; b < blocks; b++) dequant_iq4_nl(p + b * 18, dst + b * 32); return 0;
    case T_Q4_K: for (int64_t b = 0; b < blocks; b++) dequant_q4_k(p + b * 144, dst + b * 256); return 0;
    case T_Q5_K: for (int64_t b = 0; b < blocks; b++) dequant_q5_k(p + b * 176, dst + b * 256); return 0;
    case T_Q6_K: for (int64_t b = 0; b < blocks; b++) dequant_q6_k(p + b * 210, dst + b * 256); return 0;
  }
  return -1;
}

// ---- quantisers ----------------------------------------------------------------------
// The uncalibrated ("rtn", no importance matrix) arm of the reference's quantiser:
// llm/quantk.go:87-179 (asymEnc.Encode), llm/sim.go:982-1060 (makeQkxQuants),
// llm/sim.go:757-830 (makeQxQuants), llm/sim.go:1172-1180 (nearestInt), and
// llm/quantk.go:211-226 (packScaleMinK4). float32 accumulators on purpose
// (llm/sim.go:803-808). Compile with -ffp-contract=off: the reference's host language
// does not fuse multiply-adds on x86-64.

inline int dequantize_w16(uint32_t type, const void* data, int64_t n, float* dst) {
  const uint8_t* p = (const uint8_t*)data;
  if (type == T_Q4_K || type == T_Q5_K) {
    if (n % 256) return -1;
    const int bb = type == T_Q4_K ? 144 : 176;
    for (int64_t b = 0; b < n / 256; b++) dequant_w16_q45_k(p + b * bb, dst + b * 256, type == T_Q5_K);
    return 0;
  }
  if (type == T_Q6_K) {
    if (n % 256) return -1;
    for (int64_t b = 0; b < n / 256; b++) dequant_w16_q6_k(p + b * 210, dst + b * 256);
    return 0;
  }
  int rc = dequantize(type, data, n, dst);   // Q8_0: fp16(d * q) is the single rounding; F16/F32: rounded once
  if (rc == 0) for (int64_t i = 0; i < n; i++) dst[i] = f16_round(dst[i]);
  return rc;
}

inline float nearest_int(float v) { return (float)nearbyint((double)v); }  // round-half-even

inline float make_qkx_quants(const float* x, int n, int nmax, const float* w, uint8_t* lv, uint8_t* laux,
                             float rmin, float rdelta, int nstep, float* the_min) {
  float mn = x[0], mx = x[0];
  float sum_w = w[0], sum_x = w[0] * x[0];
  for (int i = 1; i < n; i++) {
    if (x[i] < mn) mn = x[i];
    if (x[i] > mx) mx = x[i];
    sum_w += w[i];
    sum_x += w[i] * x[i];
  }
  if (mn > 0) mn = 0;
  if (mx <= mn) {
    for (int i = 0; i < n; i++) lv[i] = 0;
    *the_min = -mn;
    return 0.f;
  }
  float iscale = (float)nmax / (mx - mn);
  float scale = 1 / iscale;
  float best_err = 0;
  for (int i = 0; i < n; i++) {
    float l = nearest_int(iscale * (x[i] - mn));
    if (l < 0) l = 0;
    if (l > (float)nmax) l = (float)nmax;
    lv[i] = (uint8_t)l;
    float diff = scale * (float)lv[i] + mn - x[i];
    best_err += w[i] * diff * diff;
  }
  if (nstep < 1) { *the_min = -mn; return scale; }
  for (int is = 0; is <= nstep; is++) {
    iscale = (rmin + rdelta * (float)is + (float)nmax) / (mx - mn);
    float sum_l = 0, sum_l2 = 0, sum_xl = 0;
    for (int i = 0; i < n; i++) {
      float l = nearest_int(iscale * (x[i] - mn));
      if (l < 0) l = 0;
      if (l > (float)nmax) l = (float)nmax;
      laux[i] = (uint8_t)l;
      float fl = (float)laux[i];
      sum_l += w[i] * fl;
      sum_l2 += w[i] * fl * fl;
      sum_xl += w[i] * fl * x[i];
    }
    float det = sum_w * sum_l2 - sum_l * sum_l;
    if (det <= 0) continue;
    float this_scale = (sum_w * sum_xl - sum_x * sum_l) / det;
    float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / det;
    if (this_min > 0) { this_min = 0; this_scale = sum_xl / sum_l2; }
    float err = 0;
    for (int i = 0; i < n; i++) {
      float diff = this_scale * (float)laux[i] + this_min - x[i];
      err += w[i] * diff * diff;
    }
    if (err < best_err) {
      memcpy(lv, laux, (size_t)n);
      best_err = err; scale = this_scale; mn = this_min;
    }
  }
  *the_min = -mn;
  return scale;
}

inline void pack_scale_min_k4(uint8_t* dst, const int* ls, const int* lm) {
  memset(dst, 0, 12);
  for (int j = 0; j < 8; j++) {
    uint8_t s = (uint8_t)ls[j], m = (uint8_t)lm[j];
    if (j < 4) { dst[j] = s; dst[j + 4] = m; }
    else {
      dst[j + 4] = (uint8_t)((s & 0xF) | ((m & 0xF) << 4));
      dst[j - 4] |= (uint8_t)((s >> 4) << 6);
      dst[j] |= (uint8_t)((m >> 4) << 6);
    }
  }
}

// One 256-element super-block -> levels L[256] (0..nmax), fp16 d/dmin, packed scales.
inline void encode_k_super(const float* x, int bits, uint16_t* d16, uint16_t* dmin16, uint8_t* scales12, uint8_t* L) {
  const int nmax = bits == 5 ? 31 : 15;
  const float rmin = bits == 5 ? -0.5f : -1.f;
  const int nstep = bits == 5 ? 15 : 20;
  float scales[8], mins[8], w[32];
  uint8_t laux[32];
  float max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; j++) {
    const float* g = x + 32 * j;
    float sum2 = 0;
    for (int i = 0; i < 32; i++) sum2 += g[i] * g[i];
    float avx = sqrtf(sum2 / 32.f);
    for (int i = 0; i < 32; i++) w[i] = avx + fabsf(g[i]);
    scales[j] = make_qkx_quants(g, 32, nmax, w, L + 32 * j, laux, rmin, 0.1f, nstep, &mins[j]);
    if (scales[j] > max_scale) max_scale = scales[j];
    if (mins[j] > max_min) max_min = mins[j];
  }
  float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
  float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
  int ls[8], lm[8];
  for (int j = 0; j < 8; j++) {
    float a = nearest_int(inv_scale * scales[j]), b = nearest_int(inv_min * mins[j]);
    ls[j] = a < 0 ? 0 : a > 63 ? 63 : (int)a;
    lm[j] = b < 0 ? 0 : b > 63 ? 63 : (int)b;
  }
  pack_scale_min_k4(scales12, ls, lm);
  *d16 = f32_to_f16(max_scale / 63.f);
  *dmin16 = f32_to_f16(max_min / 63.f);
  float df = f16_to_f32(*d16), dminf = f16_to_f32(*dmin16);
  for (int j = 0; j < 8; j++) {
    float ds = df * (float)ls[j], dm = dminf * (float)lm[j];
    if (ds == 0) continue;  // levels of the search stay; they dequantise through a zero scale
    for (int i = 0; i < 32; i++) {
      float l = nearest_int((x[32 * j + i] + dm) / ds);
      if (l < 0) l = 0;
      if (l > (float)nmax) l = (float)nmax;
      L[32 * j + i] = (uint8_t)l;
    }
  }
}

inline void quantize_q4_k_block(const float* x, uint8_t* blk) {
  uint8_t L[256]; uint16_t d, dmin;
  encode_k_super(x, 4, &d, &dmin, blk + 4, L);
  memcpy(blk, &d, 2); memcpy(blk + 2, &dmin, 2);
  uint8_t* q = blk + 16;
  for (int j = 0; j < 256; j += 64) {
    for (int l = 0; l < 32; l++) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
    q += 32;
  }
}

inline void quantize_q5_k_block(const float* x, uint8_t* blk) {
  uint8_t L[256]; uint16_t d, dmin;
  encode_k_super(x, 5, &d, &dmin, blk + 4, L);
  memcpy(blk, &d, 2); memcpy(blk + 2, &dmin, 2);
  uint8_t* qh = blk + 16; uint8_t* ql = blk + 48;
  memset(qh, 0, 32);
  uint8_t m1 = 1, m2 = 2;
  for (int n = 0; n < 256; n += 64) {
    for (int j = 0; j < 32; j++) {
      int l1 = L[n + j], l2 = L[n + j + 32];
      if (l1 > 15) { l1 -= 16; qh[j] |= m1; }
      if (l2 > 15) { l2 -= 16; qh[j] |= m2; }
      ql[j] = (uint8_t)(l1 | (l2 << 4));
    }
    m1 <<= 2; m2 <<= 2; ql += 32;
  }
}

// ggml's make_qx_quants with rmse_type 1 and no importance (llm/sim.go:757-830),
// levels returned biased by nmax.
inline float make_qx_quants(const float* x, int n, int nmax, int8_t* L) {
  float amax = 0, maxval = 0;
  for (int i = 0; i < n; i++) { float a = fabsf(x[i]); if (a > amax) { amax = a; maxval = x[i]; } }
  if (amax < 1e-15f) { for (int i = 0; i < n; i++) L[i] = 0; return 0.f; }
  float lon = (float)-nmax, hin = (float)(nmax - 1);
  float iscale = -(float)nmax / maxval;
  float sumlx = 0, suml2 = 0;
  for (int i = 0; i < n; i++) {
    float l = nearest_int(iscale * x[i]);
    if (l < lon) l = lon;
    if (l > hin) l = hin;
    L[i] = (int8_t)((int)l + nmax);
    float w = x[i] * x[i];
    sumlx += w * x[i] * l;
    suml2 += w * l * l;
  }
  float scale = suml2 != 0 ? sumlx / suml2 : 0.f;
  float best = scale * sumlx;
  for (int is = -9; is <= 9; is++) {
    if (is == 0) continue;
    float tr = -((float)nmax + 0.1f * (float)is) / maxval;
    float sx = 0, s2 = 0;
    for (int i = 0; i < n; i++) {
      float l = nearest_int(tr * x[i]);
      if (l < lon) l = lon;
      if (l > hin) l = hin;
      float w = x[i] * x[i];
      sx += w * x[i] * l;
      s2 += w * l * l;
    }
    if (s2 > 0 && sx * sx > best * s2) {
      for (int i = 0; i < n; i++) {
        float l = nearest_int(tr * x[i]);
        if (l < lon) l = lon;
        if (l > hin) l = hin;
        L[i] = (int8_t)((int)l + nmax);
      }
      scale = sx / s2;
      best = scale * sx;
    }
  }
  return scale;
}

// Q6_K: the published ggml algorithm (quantize_row_q6_K_ref). The reference repo has no
// Q6_K quantiser of its own and no fixture for one; only the Q6_K *dequantiser* is pinned.
inline void quantize_q6_k_block(const float* x, uint8_t* blk) {
  int8_t L[256]; float scales[16];
  float max_scale = 0, max_abs = 0;
  for (int ib = 0; ib < 16; ib++) {
    float s = make_qx_quants(x + 16 * ib, 16, 32, L + 16 * ib);
    scales[ib] = s;
    float a = fabsf(s);
    if (a > max_abs) { max_abs = a; max_scale = s; }
  }
  if (max_abs < 1e-15f) { memset(blk, 0, 210); return; }
  float iscale = -128.f / max_scale;
  uint16_t d16 = f32_to_f16(1 / iscale);
  memcpy(blk + 208, &d16, 2);
  int8_t* sc = (int8_t*)(blk + 192);
  for (int ib = 0; ib < 16; ib++) {
    float v = nearest_int(iscale * scales[ib]);
    sc[ib] = (int8_t)(v > 127 ? 127 : (int)v);
  }
  float df = f16_to_f32(d16);
  for (int j = 0; j < 16; j++) {
    float d = df * (float)sc[j];
    if (d == 0) continue;
    for (int i = 0; i < 16; i++) {
      float l = nearest_int(x[16 * j + i] / d);
      if (l < -32) l = -32;
      if (l > 31) l = 31;
      L[16 * j + i] = (int8_t)((int)l + 32);
    }
  }
  uint8_t* ql = blk; uint8_t* qh = blk + 128;
  for (int j = 0; j < 256; j += 128) {
    for (int l = 0; l < 32; l++) {
      uint8_t q1 = L[j + l] & 0xF, q2 = L[j + l + 32] & 0xF, q3 = L[j + l + 64] & 0xF, q4 = L[j + l + 96] & 0xF;
      ql[l] = (uint8_t)(q1 | (q3 << 4));
      ql[l + 32] = (uint8_t)(q2 | (q4 << 4));
      qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) | ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
    }
    ql += 64; qh += 32;
  }
}

// Q8_0: d = amax/127 stored as fp16, levels round(x/d) half away from zero
// (llm/bank.go:143-198 states the same rule for the int8 bank).
inline void quantize_q8_0_block(const float* x, uint8_t* blk) {
  float amax = 0;
  for (int i = 0; i < 32; i++) { float a = fabsf(x[i]); if (a > amax) amax = a; }
  float d = amax / 127.f;
  float id = d != 0 ? 1.f / d : 0.f;
  uint16_t d16 = f32_to_f16(d);
  memcpy(blk, &d16, 2);
  for (int i = 0; i < 32; i++) blk[2 + i] = (uint8_t)(int8_t)roundf(x[i] * id);
}

// rows x k f32 -> packed blocks. Returns 0 or -1.
inline int quantize(uint32_t type, const float* src, int64_t rows, int64_t k, void* dst) {
  int e, nb;
  if (!block_geometry(type, &e, &nb) || k % e) return -1;
  int64_t blocks = rows * k / e;
  uint8_t* out = (uint8_t*)dst;
  switch (type) {
    case T_F32: memcpy(out, src, (size_t)(rows * k) * 4); return 0;
    case T_F16:
      for (int64_t i = 0; i < rows * k; i++) { uint16_t h = f32_to_f16(src[i]); memcpy(out + 2 * i, &h, 2); }
      return 0;
    case T_Q8_0:
#pragma omp parallel for schedule(static)
      for (int64_t b = 0; b < blocks; b++) quantize_q8_0_block(src + b * 32, out + b * 34);
      return 0;
    case T_Q4_K:
#pragma omp parallel for schedule(static)
      for (int64_t b = 0; b < blocks; b++) quantize_q4_k_block(src + b * 256, out + b * 144);
      return 0;
    case T_Q5_K:
#pragma omp parallel for schedule(static)
      for (int64_t b = 0; b < blocks; b++) quantize_q5_k_block(src + b * 256, out + b * 176);
      return 0;
    case T_Q6_K:
#pragma omp parallel for schedule(static)
      for (int64_t b = 0; b < blocks; b++) quantize_q6_k_block(src + b * 256, out + b * 210);
      return 0;
  }
  return -1;
}

}  // namespace orc
