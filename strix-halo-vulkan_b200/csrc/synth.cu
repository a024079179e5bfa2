// Synthetic checkpoints on the device: seeded values and the repo's K-quant quantiser.
//
// The quantiser restates the reference's uncalibrated arm (llm/quantk.go:87-179 Encode,
// llm/sim.go:982-1060 makeQkxQuants, :757-830 makeQxQuants, :1172-1180 nearestInt,
// llm/quantk.go:211-226 packScaleMinK4) one super-block per thread. This file is compiled
// with -fmad=false: the search compares near-equal f32 sums, and fused multiply-adds would
// choose different rungs than the host implementation does.
#include "model.h"

namespace b200 {

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__global__ void synth_fill_kernel(float* dst, int64_t n, uint64_t seed, int rule, float p0, float p1) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint64_t r = splitmix64(seed ^ splitmix64((uint64_t)i));
  float u1 = ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
  float u2 = ((float)(uint32_t)((r >> 8) & 0xFFFFFF) + 0.5f) * (1.0f / 16777216.0f);
  float v;
  if (rule == 0) v = p0 + p1 * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
  else v = -expf(p0 + (p1 - p0) * u1);
  dst[i] = v;
}

int synth_fill(float* dst, int64_t n, uint64_t seed, int rule, float p0, float p1, cudaStream_t st) {
  synth_fill_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(dst, n, seed, rule, p0, p1);
  B200_CUDA(cudaGetLastError());
  return OK;
}

__device__ __forceinline__ float nearest_int_f(float v) { return rintf(v); }  // round-half-even

__device__ float make_qkx_quants_d(const float* x, int nmax, const float* w, uint8_t* lv, float rmin, float rdelta, int nstep, float* the_min) {
  float mn = x[0], mx = x[0];
  float sum_w = w[0], sum_x = w[0] * x[0];
  for (int i = 1; i < 32; i++) {
    if (x[i] < mn) mn = x[i];
    if (x[i] > mx) mx = x[i];
    sum_w += w[i];
    sum_x += w[i] * x[i];
  }
  if (mn > 0) mn = 0;
  if (mx <= mn) {
    for (int i = 0; i < 32; i++) lv[i] = 0;
    *the_min = -mn;
    return 0.f;
  }
  float iscale = (float)nmax / (mx - mn);
  float scale = 1 / iscale;
  float best_err = 0;
  for (int i = 0; i < 32; i++) {
    float l = nearest_int_f(iscale * (x[i] - mn));
    l = fminf(fmaxf(l, 0.f), (float)nmax);
    lv[i] = (uint8_t)l;
    float diff = scale * (float)lv[i] + mn - x[i];
    best_err += w[i] * diff * diff;
  }
  uint8_t laux[32];
  for (int is = 0; is <= nstep; is++) {
    iscale = (rmin + rdelta * (float)is + (float)nmax) / (mx - mn);
    float sum_l = 0, sum_l2 = 0, sum_xl = 0;
    for (int i = 0; i < 32; i++) {
      float l = nearest_int_f(iscale * (x[i] - mn));
      l = fminf(fmaxf(l, 0.f), (float)nmax);
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
    for (int i = 0; i < 32; i++) {
      float diff = this_scale * (float)laux[i] + this_min - x[i];
      err += w[i] * diff * diff;
    }
    if (err < best_err) {
      for (int i = 0; i < 32; i++) lv[i] = laux[i];
      best_err = err; scale = this_scale; mn = this_min;
    }
  }
  *the_min = -mn;
  return scale;
}

__device__ void pack_scale_min_k4_d(uint8_t* dst, const int* ls, const int* lm) {
  for (int i = 0; i < 12; i++) dst[i] = 0;
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

__global__ void quantize_k45_kernel(const float* src, int64_t nblocks, int bits, uint8_t* dst) {
  int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const float* x = src + b * 256;
  uint8_t* blk = dst + b * (bits == 5 ? 176 : 144);
  const int nmax = bits == 5 ? 31 : 15;
  const float rmin = bits == 5 ? -0.5f : -1.f;
  const int nstep = bits == 5 ? 15 : 20;
  uint8_t L[256];
  float scales[8], mins[8];
  float max_scale = 0, max_min = 0;
  for (int j = 0; j < 8; j++) {
    float g[32], w[32];
    float sum2 = 0;
    for (int i = 0; i < 32; i++) { g[i] = x[32 * j + i]; sum2 += g[i] * g[i]; }
    float avx = sqrtf(sum2 / 32.f);
    for (int i = 0; i < 32; i++) w[i] = avx + fabsf(g[i]);
    scales[j] = make_qkx_quants_d(g, nmax, w, L + 32 * j, rmin, 0.1f, nstep, &mins[j]);
    if (scales[j] > max_scale) max_scale = scales[j];
    if (mins[j] > max_min) max_min = mins[j];
  }
  float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
  float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
  int ls[8], lm[8];
  for (int j = 0; j < 8; j++) {
    float a = nearest_int_f(inv_scale * scales[j]), m = nearest_int_f(inv_min * mins[j]);
    ls[j] = a < 0 ? 0 : a > 63 ? 63 : (int)a;
    lm[j] = m < 0 ? 0 : m > 63 ? 63 : (int)m;
  }
  pack_scale_min_k4_d(blk + 4, ls, lm);
  __half d16 = __float2half_rn(max_scale / 63.f), dm16 = __float2half_rn(max_min / 63.f);
  *reinterpret_cast<__half*>(blk) = d16;
  *reinterpret_cast<__half*>(blk + 2) = dm16;
  float df = __half2float(d16), dminf = __half2float(dm16);
  for (int j = 0; j < 8; j++) {
    float ds = df * (float)ls[j], dm = dminf * (float)lm[j];
    if (ds == 0) continue;
    for (int i = 0; i < 32; i++) {
      float l = nearest_int_f((x[32 * j + i] + dm) / ds);
      l = fminf(fmaxf(l, 0.f), (float)nmax);
      L[32 * j + i] = (uint8_t)l;
    }
  }
  if (bits == 4) {
    uint8_t* q = blk + 16;
    for (int j = 0; j < 256; j += 64) {
      for (int l = 0; l < 32; l++) q[l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
      q += 32;
    }
  } else {
    uint8_t* qh = blk + 16; uint8_t* ql = blk + 48;
    for (int l = 0; l < 32; l++) qh[l] = 0;
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
}

__device__ float make_qx_quants_d(const float* x, int nmax, int8_t* L) {
  float amax = 0, maxval = 0;
  for (int i = 0; i < 16; i++) { float a = fabsf(x[i]); if (a > amax) { amax = a; maxval = x[i]; } }
  if (amax < 1e-15f) { for (int i = 0; i < 16; i++) L[i] = 0; return 0.f; }
  const float lon = (float)-nmax, hin = (float)(nmax - 1);
  float iscale = -(float)nmax / maxval;
  float sumlx = 0, suml2 = 0;
  for (int i = 0; i < 16; i++) {
    float l = fminf(fmaxf(nearest_int_f(iscale * x[i]), lon), hin);
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
    for (int i = 0; i < 16; i++) {
      float l = fminf(fmaxf(nearest_int_f(tr * x[i]), lon), hin);
      float w = x[i] * x[i];
      sx += w * x[i] * l;
      s2 += w * l * l;
    }
    if (s2 > 0 && sx * sx > best * s2) {
      for (int i = 0; i < 16; i++) {
        float l = fminf(fmaxf(nearest_int_f(tr * x[i]), lon), hin);
        L[i] = (int8_t)((int)l + nmax);
      }
      scale = sx / s2;
      best = scale * sx;
    }
  }
  return scale;
}

__global__ void quantize_q6k_kernel(const float* src, int64_t nblocks, uint8_t* dst) {
  int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const float* x = src + b * 256;
  uint8_t* blk = dst + b * 210;
  int8_t L[256]; float scales[16];
  float max_scale = 0, max_abs = 0;
  for (int ib = 0; ib < 16; ib++) {
    float g[16];
    for (int i = 0; i < 16; i++) g[i] = x[16 * ib + i];
    float s = make_qx_quants_d(g, 32, L + 16 * ib);
    scales[ib] = s;
    float a = fabsf(s);
    if (a > max_abs) { max_abs = a; max_scale = s; }
  }
  if (max_abs < 1e-15f) { for (int i = 0; i < 210; i++) blk[i] = 0; return; }
  float iscale = -128.f / max_scale;
  __half d16 = __float2half_rn(1 / iscale);
  *reinterpret_cast<__half*>(blk + 208) = d16;  // 210 * b + 208 is even
  int8_t* sc = (int8_t*)(blk + 192);
  for (int ib = 0; ib < 16; ib++) {
    float v = nearest_int_f(iscale * scales[ib]);
    sc[ib] = (int8_t)(v > 127 ? 127 : (int)v);
  }
  float df = __half2float(d16);
  for (int j = 0; j < 16; j++) {
    float d = df * (float)sc[j];
    if (d == 0) continue;
    for (int i = 0; i < 16; i++) {
      float l = fminf(fmaxf(nearest_int_f(x[16 * j + i] / d), -32.f), 31.f);
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

__global__ void quantize_q80_kernel(const float* src, int64_t nblocks, uint8_t* dst) {
  int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const float* x = src + b * 32;
  uint8_t* blk = dst + b * 34;
  float amax = 0;
  for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
  float d = amax / 127.f;
  float id = d != 0 ? 1.f / d : 0.f;
  *reinterpret_cast<__half*>(blk) = __float2half_rn(d);  // 34 * b is even
  for (int i = 0; i < 32; i++) blk[2 + i] = (uint8_t)(int8_t)roundf(x[i] * id);
}

__global__ void to_f16_kernel(const float* src, int64_t n, __half* dst) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2half_rn(src[i]);
}

int quantize_rows_device(uint32_t type, const float* src, int64_t rows, int64_t k, uint8_t* dst, cudaStream_t st) {
  int e, nb;
  if (!block_geometry(type, &e, &nb) || k % e) { set_error("quantize: bad type or row length"); return EINVAL_; }
  const int64_t blocks = rows * k / e;
  const unsigned grid = (unsigned)((blocks + 127) / 128);
  switch (type) {
    case T_F32: B200_CUDA(cudaMemcpyAsync(dst, src, (size_t)(rows * k) * 4, cudaMemcpyDeviceToDevice, st)); return OK;
    case T_F16: to_f16_kernel<<<(unsigned)((rows * k + 255) / 256), 256, 0, st>>>(src, rows * k, (__half*)dst); break;
    case T_Q8_0: quantize_q80_kernel<<<grid, 128, 0, st>>>(src, blocks, dst); break;
    case T_Q4_K: quantize_k45_kernel<<<grid, 128, 0, st>>>(src, blocks, 4, dst); break;
    case T_Q5_K: quantize_k45_kernel<<<grid, 128, 0, st>>>(src, blocks, 5, dst); break;
    case T_Q6_K: quantize_q6k_kernel<<<grid, 128, 0, st>>>(src, blocks, dst); break;
    default: set_error("quantize: type has no device quantiser"); return EINVAL_;
  }
  B200_CUDA(cudaGetLastError());
  return OK;
}

}  // namespace b200
