// The token loop's non-projection kernels: embedding gather, router + routing, gated
// DeltaNet step, attention pre-pass and split-KV decode attention, MoE combine, argmax,
// and the Q6_K / Q8_0 row re-layout.
#include "kernels.cuh"

#include <cooperative_groups.h>

#include <cmath>

namespace cg = cooperative_groups;

namespace b200 {

// =========================================================================================
// Row layout
// =========================================================================================
bool block_geometry(uint32_t t, int* e, int* b) {
  switch (t) {
    case T_F32: *e = 1; *b = 4; return true;
    case T_F16: case T_BF16: *e = 1; *b = 2; return true;
    case T_Q4_1: *e = 32; *b = 20; return true;
    case T_Q5_0: *e = 32; *b = 22; return true;
    case T_Q5_1: *e = 32; *b = 24; return true;
    case T_Q8_0: *e = 32; *b = 34; return true;
    case T_IQ4_NL: *e = 32; *b = 18; return true;
    case T_Q4_K: *e = 256; *b = 144; return true;
    case T_Q5_K: *e = 256; *b = 176; return true;
    case T_Q6_K: *e = 256; *b = 210; return true;
  }
  return false;
}
int64_t gguf_row_bytes(uint32_t t, int64_t n) {
  int e, b;
  if (!block_geometry(t, &e, &b) || n % e) return -1;
  return n / e * b;
}
int64_t device_row_stride(uint32_t t, int64_t k) {
  int64_t rb = gguf_row_bytes(t, k);
  if (rb < 0) return -1;
  if (t == T_Q6_K || t == T_Q8_0) return (rb + 15) / 16 * 16;
  return rb;
}

// One thread per block. Q6_K: ql | qh | scales | d planes; Q8_0: qs | d planes.
__global__ void repack_kernel(uint32_t type, int64_t nb, int64_t rows, int64_t stride, const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int inverse) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nb * rows) return;
  int64_t r = i / nb, b = i - r * nb;
  uint8_t* drow = dst + (inverse ? 0 : r * stride);
  const uint8_t* srow = src + (inverse ? r * stride : 0);
  if (type == T_Q6_K) {
    const int64_t g = (r * nb + b) * 210;
    uint8_t* gq = inverse ? dst + g : nullptr;
    const uint8_t* gs = inverse ? nullptr : src + g;
    uint8_t* pql = (inverse ? const_cast<uint8_t*>(srow) : drow) + b * 128;
    uint8_t* pqh = (inverse ? const_cast<uint8_t*>(srow) : drow) + nb * 128 + b * 64;
    uint8_t* psc = (inverse ? const_cast<uint8_t*>(srow) : drow) + nb * 192 + b * 16;
    uint8_t* pd = (inverse ? const_cast<uint8_t*>(srow) : drow) + nb * 208 + b * 2;
    if (!inverse) {
      for (int j = 0; j < 128; j++) pql[j] = gs[j];
      for (int j = 0; j < 64; j++) pqh[j] = gs[128 + j];
      for (int j = 0; j < 16; j++) psc[j] = gs[192 + j];
      pd[0] = gs[208]; pd[1] = gs[209];
    } else {
      for (int j = 0; j < 128; j++) gq[j] = pql[j];
      for (int j = 0; j < 64; j++) gq[128 + j] = pqh[j];
      for (int j = 0; j < 16; j++) gq[192 + j] = psc[j];
      gq[208] = pd[0]; gq[209] = pd[1];
    }
  } else {  // Q8_0
    const int64_t g = (r * nb + b) * 34;
    uint8_t* base = inverse ? const_cast<uint8_t*>(srow) : drow;
    uint8_t* pq = base + b * 32;
    uint8_t* pd = base + nb * 32 + b * 2;
    if (!inverse) {
      pd[0] = src[g]; pd[1] = src[g + 1];
      for (int j = 0; j < 32; j++) pq[j] = src[g + 2 + j];
    } else {
      dst[g] = pd[0]; dst[g + 1] = pd[1];
      for (int j = 0; j < 32; j++) dst[g + 2 + j] = pq[j];
    }
  }
}

int repack_rows(uint32_t type, int64_t k, int64_t rows, const uint8_t* gguf_dev, uint8_t* dst_dev, cudaStream_t st) {
  int64_t rb = gguf_row_bytes(type, k);
  if (rb < 0) { set_error("repack: bad type or row length"); return EINVAL_; }
  if (type != T_Q6_K && type != T_Q8_0) {
    B200_CUDA(cudaMemcpyAsync(dst_dev, gguf_dev, (size_t)(rb * rows), cudaMemcpyDeviceToDevice, st));
    return OK;
  }
  int64_t nb = k / (type == T_Q6_K ? 256 : 32), n = nb * rows;
  repack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(type, nb, rows, device_row_stride(type, k), gguf_dev, dst_dev, 0);
  B200_CUDA(cudaGetLastError());
  return OK;
}
int unpack_rows(uint32_t type, int64_t k, int64_t rows, const uint8_t* dev, uint8_t* gguf_dev, cudaStream_t st) {
  int64_t rb = gguf_row_bytes(type, k);
  if (rb < 0) { set_error("unpack: bad type or row length"); return EINVAL_; }
  if (type != T_Q6_K && type != T_Q8_0) {
    B200_CUDA(cudaMemcpyAsync(gguf_dev, dev, (size_t)(rb * rows), cudaMemcpyDeviceToDevice, st));
    return OK;
  }
  int64_t nb = k / (type == T_Q6_K ? 256 : 32), n = nb * rows;
  repack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(type, nb, rows, device_row_stride(type, k), dev, gguf_dev, 1);
  B200_CUDA(cudaGetLastError());
  return OK;
}

// =========================================================================================
// Exact element dequantisation (reference: gguf/dequant.go:128-356), device layout
// =========================================================================================
__device__ __forceinline__ float ld_f16(const uint8_t* p) { return __half2float(*reinterpret_cast<const __half*>(p)); }

__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* q, int* sc, int* m) {
  if (j < 4) { *sc = q[j] & 63; *m = q[j + 4] & 63; }
  else { *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// value of element k of a device row. __fmul_rn / __fsub_rn keep the reference's
// unfused `d*sc*q - dmin*m` so the result is bit-identical to the CPU dequantiser.
__device__ float dequant_elem(uint32_t type, const uint8_t* row, int64_t K, int64_t k) {
  switch (type) {
    case T_F32: return reinterpret_cast<const float*>(row)[k];
    case T_F16: return ld_f16(row + 2 * k);
    case T_BF16: return __uint_as_float((uint32_t)reinterpret_cast<const unsigned short*>(row)[k] << 16);
    case T_Q8_0: {
      int64_t nb = K / 32, b = k / 32;
      float d = ld_f16(row + nb * 32 + b * 2);
      return __fmul_rn((float)(int8_t)row[k], d);
    }
    case T_Q4_K: {
      const uint8_t* blk = row + (k / 256) * 144;
      int e = (int)(k % 256), grp = e / 64, in = e % 64, hi = in / 32, l = in % 32;
      float d = ld_f16(blk), dmin = ld_f16(blk + 2);
      int sc, m; k4_scale_min(2 * grp + hi, blk + 4, &sc, &m);
      int q = hi ? (blk[16 + 32 * grp + l] >> 4) : (blk[16 + 32 * grp + l] & 0xF);
      return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
    }
    case T_Q5_K: {
      const uint8_t* blk = row + (k / 256) * 176;
      int e = (int)(k % 256), grp = e / 64, in = e % 64, hi = in / 32, l = in % 32;
      float d = ld_f16(blk), dmin = ld_f16(blk + 2);
      int sc, m; k4_scale_min(2 * grp + hi, blk + 4, &sc, &m);
      int q = hi ? (blk[48 + 32 * grp + l] >> 4) : (blk[48 + 32 * grp + l] & 0xF);
      if (blk[16 + l] & (1 << (2 * grp + hi))) q += 16;
      return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
    }
    case T_Q6_K: {
      int64_t nb = K / 256, b = k / 256;
      int e = (int)(k % 256), hf = e / 128, in = e % 128, quarter = in / 32, l = in % 32;
      const uint8_t* ql = row + b * 128 + 64 * hf + 32 * (quarter & 1) + l;
      const uint8_t* qh = row + nb * 128 + b * 64 + 32 * hf + l;
      int8_t sc = (int8_t)row[nb * 192 + b * 16 + 8 * hf + l / 16 + 2 * quarter];
      float d = ld_f16(row + nb * 208 + b * 2);
      int nib = quarter >= 2 ? (*ql >> 4) : (*ql & 0xF);
      int q = (nib | (((*qh >> (2 * quarter)) & 3) << 4)) - 32;
      return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    }
  }
  return 0.f;
}

__global__ void dequant_rows_kernel(DTensor t, int64_t row0, int64_t rows, float* out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * t.k) return;
  int64_t r = i / t.k, k = i - r * t.k;
  out[i] = dequant_elem(t.type, t.data + (row0 + r) * t.stride, t.k, k);
}
int dequant_rows(const DTensor& t, int64_t row0, int64_t rows, float* out, cudaStream_t st) {
  int64_t n = rows * t.k;
  dequant_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(t, row0, rows, out);
  B200_CUDA(cudaGetLastError());
  return OK;
}

// Embedding gather on the device (the reference dequantises the row on the host and
// uploads it: llm/model.go:125-144), fused with the first layer's input norm.
__global__ void __launch_bounds__(QG_THREADS) embed_norm_kernel(EmbedParams p) {
  __shared__ float scratch[2 * QG_WARPS];
  const int n = blockIdx.x;
  const int64_t id = p.ids[n];
  const uint8_t* row = p.embd.data + id * p.embd.stride;
  float* h = p.h + (size_t)n * p.H;
  float sq = 0.f;
  for (int k = threadIdx.x; k < p.H; k += blockDim.x) { const float v = dequant_elem(p.embd.type, row, p.H, k); h[k] = v; sq += v * v; }
  if (p.ss_out != nullptr) {  // the first projection normalises from this
    sq = warp_sum(sq);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < QG_WARPS; w++) t += scratch[w];
      p.ss_out[(size_t)n * SS_LD] = t;
    }
  }
  if (p.gamma != nullptr) {
    __syncthreads();
    row_rmsnorm_f16(h, p.gamma, p.eps, p.H, p.xn + (size_t)n * p.H, scratch);
  }
}
int launch_embed(const EmbedParams& p, cudaStream_t st) {
  embed_norm_kernel<<<p.M, QG_THREADS, 0, st>>>(p);
  B200_CUDA(cudaGetLastError());
  return OK;
}

// =========================================================================================
// PDL launch helper
// =========================================================================================
template <class... KArgs, class... Args>
static int launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, bool pdl, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  B200_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
  return OK;
}

// =========================================================================================
// Router: ffn_norm + router GEMV (exact f32 dequant) + softmax + top-k + work list
// (reference: llm/moe.go:219-282; shaders/llm_moe_router.comp, llm_moe_route_decode.comp)
// =========================================================================================
constexpr int RT_ROWS = 8;  // router rows per CTA: one per warp

// Expert work list of a pass from its routing, by one CTA of 256 threads: pair id = n*(used+1) + slot,
// slot == used is the shared expert; entries of at most 8 columns per expert for the column-tiled kernels,
// one GEMM problem per expert for the tensor-core kernels, cols = pairs in expert-sorted order.
__device__ void build_work_list(const RouterParams& p, int* counts, int* offs, int* eoff) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, M = p.M, nE = p.nE, used = p.used;
  const int EC = p.ecols > 0 ? p.ecols : 8;  // columns per entry
  // work list: pair id = n*(used+1) + slot; slot == used is the shared expert
  if (M == 1) {
    if (tid < used) { p.entries[tid] = make_int4(p.topk[tid], tid, 1, 0); p.cols[tid] = tid; }
    if (tid == used) { p.entries[used] = make_int4(-1, used, 1, 0); p.cols[used] = used; *p.n_entries = used + 1; }
    tl_mark(p.tl, 6, true);
    return;
  }
  const int e_lo = p.e_hi > 0 ? p.e_lo : 0, e_hi = p.e_hi > 0 ? p.e_hi : nE;
  const int sh_lo = p.sh_hi > 0 ? p.sh_lo : 0, sh_hi = p.sh_hi > 0 ? p.sh_hi : M;
  for (int i = tid; i <= nE; i += 256) counts[i] = 0;
  __syncthreads();
  for (int i = tid; i < M * used; i += 256) {
    const int e = __ldcg(p.topk + i);
    if (e >= e_lo && e < e_hi) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (p.distinct != nullptr) {   // experts this pass streams (what a step's byte count needs)
    int mine = 0;
    for (int e = tid; e < nE; e += 256) mine += counts[e] > 0;
    mine = __reduce_add_sync(0xffffffffu, mine);
    if (lane == 0 && mine > 0) atomicAdd(reinterpret_cast<unsigned long long*>(p.distinct), (unsigned long long)mine);
  }
  if (warp == 0) {  // exclusive scans of the pair counts and of the entry counts (EC columns per entry)
    const int per = (nE + 31) / 32;
    int c = 0, en = 0;
    for (int i = 0; i < per; i++) { const int e = lane * per + i; if (e < nE) { c += counts[e]; en += (counts[e] + EC - 1) / EC; } }
    int cs = c, es = en;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int a = __shfl_up_sync(0xffffffffu, cs, o), b = __shfl_up_sync(0xffffffffu, es, o);
      if (lane >= o) { cs += a; es += b; }
    }
    int co = cs - c, eo = es - en;
    for (int i = 0; i < per; i++) {
      const int e = lane * per + i;
      if (e < nE) { offs[e] = co; eoff[e] = eo; co += counts[e]; eo += (counts[e] + EC - 1) / EC; }
    }
    const int tot_c = __shfl_sync(0xffffffffu, cs, 31), tot_e = __shfl_sync(0xffffffffu, es, 31);
    if (lane == 0) { offs[nE] = tot_c; eoff[nE] = tot_e; }
  }
  __syncthreads();
  for (int e = tid; e < nE; e += 256) {
    for (int c = 0, i = 0; c < counts[e]; c += EC, i++)
      if (eoff[e] + i < p.max_entries) p.entries[eoff[e] + i] = make_int4(e, offs[e] + c, min(EC, counts[e] - c), 0);
  }
  // one GEMM problem per expert for the tensor-core expert kernels: rows [offs, offs + count) of the expert-sorted order
  if (p.gprob != nullptr) for (int e = tid; e < nE; e += 256) p.gprob[e] = make_int4(e, offs[e], counts[e], offs[e]);
  const int nshr = sh_hi - sh_lo, nsh = (nshr + EC - 1) / EC;
  for (int i = tid; i < nsh; i += 256)
    if (eoff[nE] + i < p.max_entries) p.entries[eoff[nE] + i] = make_int4(-1, offs[nE] + EC * i, min(EC, nshr - EC * i), 0);
  if (tid == 0) { *p.n_entries = min(eoff[nE] + nsh, p.max_entries); if (p.n_pairs != nullptr) *p.n_pairs = offs[nE] + nshr; }
  __syncthreads();
  for (int i = tid; i <= nE; i += 256) counts[i] = 0;
  __syncthreads();
  for (int i = tid; i < M * used; i += 256) {
    const int e = __ldcg(p.topk + i), n = i / used, k = i - n * used;
    if (e < e_lo || e >= e_hi) continue;
    const int pos = atomicAdd(&counts[e], 1);
    p.cols[offs[e] + pos] = n * (used + 1) + k;
  }
  for (int n = tid; n < nshr; n += 256) p.cols[offs[nE] + n] = (sh_lo + n) * (used + 1) + used;
}

// Work list of an expert-parallel pass: the gathered routing of every rank's rows, restricted to the experts
// this rank owns. One CTA.
__global__ void __launch_bounds__(256) ep_worklist_kernel(RouterParams p) {
  __shared__ int counts[1025], offs[1025], eoff[1025];
  pdl_wait();
  pdl_launch();
  build_work_list(p, counts, offs, eoff);
}
int launch_ep_worklist(const RouterParams& p, bool pdl, cudaStream_t st) {
  if (p.nE > 1024 || p.used > 32 || p.M < 2) { set_error("ep_worklist: shape outside kernel limits"); return ECAPACITY; }
  return launch_k(ep_worklist_kernel, dim3(1), dim3(256), 0, pdl, st, p);
}

__global__ void __launch_bounds__(256) router_kernel(RouterParams p) {
  __shared__ int is_last;
  __shared__ int counts[1025], offs[1025], eoff[1025];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, H = p.H, M = p.M;
  const int row = blockIdx.x * RT_ROWS + warp;  // of the nE + 1 outputs; the last is the shared-expert gate
  tl_mark(p.tl, 0);
  const bool q8 = p.router.type == T_Q8_0 && H % 512 == 0 && H <= 4096;
  // the row's weights do not depend on the producer kernel: fetch them first
  uint4 wq[8]; float wd[8];
  if (row < p.nE && q8) {
    const uint8_t* wr = p.router.data + (size_t)row * p.router.stride;
    const int nb = H / 32;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int k0 = lane * 16 + i * 512;
      if (k0 < H) { wq[i] = ldg_stream(wr + k0); wd[i] = ld_f16(wr + nb * 32 + (k0 / 32) * 2); }
    }
  }
  const bool staged = p.h != nullptr;
  float4 hpre[2], gpre[2];
  if (staged) {  // the norm weights do not depend on the producer kernel either
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int k = tid * 4 + i * 1024;
      if (k < H) gpre[i] = *reinterpret_cast<const float4*>(p.gamma + k);
    }
  }
  pdl_wait();
  pdl_launch();
  tl_mark(p.tl, 1);
  extern __shared__ __align__(16) __half rxs[];  // [M][H] when the rows are normalised here
  __shared__ float rscale[8];
  if (staged) {  // ffn_norm fused into the router (M <= 8): every CTA normalises the rows, CTA 0 keeps a copy
    // the first row's values do not depend on the scale: fetch them before reducing the partials
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int k = tid * 4 + i * 1024;
      if (k < H) hpre[i] = __ldcg(reinterpret_cast<const float4*>(p.h + k));
    }
    if (warp < M) {
      const float sc = scale_from_parts(p.ss_in, p.ss_n, warp, H, p.eps);
      if (lane == 0) rscale[warp] = sc;
    }
    __syncthreads();
    auto put = [&](int n, int k, const float4& hv, const float4& g, float scale) {
      __half2 a = __floats2half2_rn(hv.x * scale * g.x, hv.y * scale * g.y), b = __floats2half2_rn(hv.z * scale * g.z, hv.w * scale * g.w);
      const uint2 o = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
      *reinterpret_cast<uint2*>(rxs + (size_t)n * H + k) = o;
      if (blockIdx.x == 0 && p.xn_out != nullptr) *reinterpret_cast<uint2*>(p.xn_out + (size_t)n * H + k) = o;
    };
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int k = tid * 4 + i * 1024;
      if (k < H) put(0, k, hpre[i], gpre[i], rscale[0]);
    }
    for (int n = 0; n < M; n++) {
      const float scale = rscale[n];
      for (int k = tid * 4 + (n == 0 ? 2048 : 0); k < H; k += 1024)
        put(n, k, __ldcg(reinterpret_cast<const float4*>(p.h + (size_t)n * H + k)), *reinterpret_cast<const float4*>(p.gamma + k), scale);
    }
    __syncthreads();
  }
  if (row <= p.nE) {
    // rows of the pass are spread over blockIdx.y in groups of 8 so a many-slot pass fills the machine
    const int n_lo = blockIdx.y * 8, n_hi = min(M, n_lo + 8);
    for (int n = n_lo; n < n_hi; n++) {
      const __half* x = staged ? rxs + (size_t)n * H : p.xn + (size_t)n * H;
      float acc = 0.f;
      if (row == p.nE) {
        for (int k = lane * 8; k < H; k += 256) {
          uint4 xv = *reinterpret_cast<const uint4*>(x + k);
          const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
          float4 g0 = *reinterpret_cast<const float4*>(p.sh_gate + k), g1 = *reinterpret_cast<const float4*>(p.sh_gate + k + 4);
          acc = fmaf(g0.x, h2f_lo(xw[0]), acc); acc = fmaf(g0.y, h2f_hi(xw[0]), acc); acc = fmaf(g0.z, h2f_lo(xw[1]), acc); acc = fmaf(g0.w, h2f_hi(xw[1]), acc);
          acc = fmaf(g1.x, h2f_lo(xw[2]), acc); acc = fmaf(g1.y, h2f_hi(xw[2]), acc); acc = fmaf(g1.z, h2f_lo(xw[3]), acc); acc = fmaf(g1.w, h2f_hi(xw[3]), acc);
        }
      } else if (q8) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int k0 = lane * 16 + i * 512;
          if (k0 < H) {
            uint4 xa = *reinterpret_cast<const uint4*>(x + k0), xb = *reinterpret_cast<const uint4*>(x + k0 + 8);
            const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            const uint32_t w[4] = {wq[i].x, wq[i].y, wq[i].z, wq[i].w};
#pragma unroll
            for (int j = 0; j < 16; j++) {
              const float wv = __fmul_rn((float)(int8_t)((w[j >> 2] >> (8 * (j & 3))) & 0xFF), wd[i]);  // gguf/dequant.go:128-137
              const float xv = (j & 1) ? h2f_hi(xw[j >> 1]) : h2f_lo(xw[j >> 1]);
              acc = fmaf(wv, xv, acc);
            }
          }
        }
      } else {
        const uint8_t* wr = p.router.data + (size_t)row * p.router.stride;
        for (int k = lane; k < H; k += 32) acc = fmaf(dequant_elem(p.router.type, wr, H, k), __half2float(x[k]), acc);
      }
      acc = warp_sum(acc);
      if (lane == 0) {
        if (row == p.nE) p.topk_w[(size_t)n * (p.used + 1) + p.used] = sigmoid_acc(acc);
        else p.logits[(size_t)n * p.nE + row] = acc;
      }
    }
  }
  tl_mark(p.tl, 4);
  if (p.defer) return;  // the expert kernel selects the experts itself
  // Two levels of tickets: the last CTA of a row group (blockIdx.y) routes that group's eight rows, one
  // per warp; the last group to finish builds the work list of the whole pass.
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = (atomicAdd(p.ticket + 1 + blockIdx.y, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (tid == 0) p.ticket[1 + blockIdx.y] = 0;
  tl_mark(p.tl, 5, true);
  const int nE = p.nE, used = p.used;
  {
    const int n = blockIdx.y * 8 + warp;
    if (n < M) {
      if (nE <= 512) route_token<16>(p, n, lane);
      else route_token<32>(p, n, lane);
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = (atomicAdd(p.ticket, 1) == (int)gridDim.y - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (tid == 0) *p.ticket = 0;
  if (p.entries == nullptr) return;   // routing only (expert-parallel passes build their list from the gathered routing)
  build_work_list(p, counts, offs, eoff);
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Router logits of a pass of some tens to hundreds of rows (batched decode): too few rows for the 128-row
// tensor-memory tiles to fill the device (512 experts are four tiles), too many for the per-row dot products
// above. A CTA takes 16 experts x 64 rows; each warp an eighth of the hidden dimension, with the experts on the
// M axis of mma.m16n8k16 and eight column tiles reusing every dequantised fragment. Q8_0 weights become
// fp16(d * q), as in the tensor-core GEMM the longer passes use. A lane reads 16 contiguous weight bytes and the
// matching 32 bytes of an activation row; the k-slots of the four mma steps are assigned to those bytes in A
// and B alike. Warp partials are summed in warp order. grid (nE / 16, ceil(M / 64)), block 256.
__global__ void __launch_bounds__(256) router_mma_kernel(RouterParams p) {
  __shared__ float part[8][16][65];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int H = p.H, M = p.M, e0 = blockIdx.x * 16, n0 = blockIdx.y * 64;
  const int ks = H / 8, nc = ks / 64, k_lo = warp * ks + 16 * t;
  const uint8_t* wa = p.router.data + (size_t)(e0 + g) * p.router.stride;
  const uint8_t* wb = p.router.data + (size_t)(e0 + g + 8) * p.router.stride;
  // the weights do not depend on the producer kernel: fetch them first
  uint4 qa[8], qb[8]; float da[8], db[8];
#pragma unroll
  for (int c = 0; c < 8; c++) {
    if (c < nc) {
      const int k0 = k_lo + 64 * c;
      qa[c] = ldg_stream(wa + k0); qb[c] = ldg_stream(wb + k0);
      da[c] = ld_f16(wa + H + (k0 / 32) * 2); db[c] = ld_f16(wb + H + (k0 / 32) * 2);
    }
  }
  pdl_wait();
  pdl_launch();
  float acc[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; nt++) { acc[nt][0] = 0.f; acc[nt][1] = 0.f; acc[nt][2] = 0.f; acc[nt][3] = 0.f; }
  auto deq2 = [](uint32_t w, int sh, float d) {  // bytes sh, sh + 1 of w as fp16(d * q) pairs
    const float lo = __fmul_rn((float)(int8_t)((w >> (8 * sh)) & 0xFF), d), hi = __fmul_rn((float)(int8_t)((w >> (8 * sh + 8)) & 0xFF), d);
    return pack_half2(lo, hi);
  };
#pragma unroll
  for (int c = 0; c < 8; c++) {
    if (c < nc) {
      const int k0 = k_lo + 64 * c;
      const uint32_t wav[4] = {qa[c].x, qa[c].y, qa[c].z, qa[c].w}, wbv[4] = {qb[c].x, qb[c].y, qb[c].z, qb[c].w};
      uint32_t a[4][4];
#pragma unroll
      for (int s = 0; s < 4; s++) {
        a[s][0] = deq2(wav[s], 0, da[c]); a[s][1] = deq2(wbv[s], 0, db[c]);
        a[s][2] = deq2(wav[s], 2, da[c]); a[s][3] = deq2(wbv[s], 2, db[c]);
      }
#pragma unroll
      for (int nt = 0; nt < 8; nt++) {
        const int row = min(n0 + nt * 8 + g, M - 1);  // rows past the end are not written
        const __half* x = p.xn + (size_t)row * H + k0;
        const uint4 x0 = *reinterpret_cast<const uint4*>(x), x1 = *reinterpret_cast<const uint4*>(x + 8);
        mma16816(acc[nt], a[0], x0.x, x0.y);
        mma16816(acc[nt], a[1], x0.z, x0.w);
        mma16816(acc[nt], a[2], x1.x, x1.y);
        mma16816(acc[nt], a[3], x1.z, x1.w);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < 8; nt++) {
    part[warp][g][nt * 8 + 2 * t] = acc[nt][0]; part[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
    part[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2]; part[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
  }
  __syncthreads();
  for (int i = tid; i < 16 * 64; i += 256) {
    const int e = i & 15, n = i >> 4;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) v += part[w][e][n];
    if (n0 + n < M) p.logits[(size_t)(n0 + n) * p.nE + e0 + e] = v;
  }
}
bool router_mma_fits(const RouterParams& p) {
  return p.router.type == T_Q8_0 && p.H % 512 == 0 && p.H <= 4096 && p.nE % 16 == 0 && p.xn != nullptr;
}
int launch_router_mma(const RouterParams& p, bool pdl, cudaStream_t st) {
  if (!router_mma_fits(p)) { set_error("router_mma: shape outside kernel limits"); return EINVAL_; }
  return launch_k(router_mma_kernel, dim3(p.nE / 16, (p.M + 63) / 64), dim3(256), 0, pdl, st, p);
}

// Routing of a many-row pass whose router logits came from the tensor-core GEMM: one warp per row
// computes the shared-expert gate (f32 weights against the fp16 row) and selects the experts; the last
// CTA builds the work list. grid ceil(M / 8), block 256.
__global__ void __launch_bounds__(256) route_rows_kernel(RouterParams p) {
  __shared__ int is_last;
  __shared__ int counts[1025], offs[1025], eoff[1025];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, H = p.H;
  pdl_wait();
  pdl_launch();
  const int n = blockIdx.x * 8 + warp;
  if (n < p.M) {
    const __half* x = p.xn + (size_t)n * H;
    float acc = 0.f;
    for (int k = lane * 8; k < H; k += 256) {
      uint4 xv = *reinterpret_cast<const uint4*>(x + k);
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
      float4 g0 = *reinterpret_cast<const float4*>(p.sh_gate + k), g1 = *reinterpret_cast<const float4*>(p.sh_gate + k + 4);
      acc = fmaf(g0.x, h2f_lo(xw[0]), acc); acc = fmaf(g0.y, h2f_hi(xw[0]), acc); acc = fmaf(g0.z, h2f_lo(xw[1]), acc); acc = fmaf(g0.w, h2f_hi(xw[1]), acc);
      acc = fmaf(g1.x, h2f_lo(xw[2]), acc); acc = fmaf(g1.y, h2f_hi(xw[2]), acc); acc = fmaf(g1.z, h2f_lo(xw[3]), acc); acc = fmaf(g1.w, h2f_hi(xw[3]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) p.topk_w[(size_t)n * (p.used + 1) + p.used] = sigmoid_acc(acc);
    if (p.nE <= 512) route_token<16>(p, n, lane);
    else route_token<32>(p, n, lane);
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = (atomicAdd(p.ticket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (tid == 0) *p.ticket = 0;
  if (p.entries == nullptr) return;   // routing only
  build_work_list(p, counts, offs, eoff);
}
int launch_route_rows(const RouterParams& p, bool pdl, cudaStream_t st) {
  if (p.nE > 1024 || p.used > 32 || p.H % 8 || p.xn == nullptr) { set_error("route_rows: shape outside kernel limits"); return ECAPACITY; }
  return launch_k(route_rows_kernel, dim3((p.M + 7) / 8), dim3(256), 0, pdl, st, p);
}

int launch_router(const RouterParams& p, bool pdl, cudaStream_t st) {
  if (p.nE > 1024 || p.used > 32 || p.H % 8) { set_error("router: shape outside kernel limits"); return ECAPACITY; }
  int grid = (p.nE + 1 + RT_ROWS - 1) / RT_ROWS;
  size_t smem = 0;
  if (p.h != nullptr) {
    if (p.M > 8) { set_error("router: the fused norm handles at most 8 rows"); return EINVAL_; }
    smem = (size_t)p.M * p.H * sizeof(__half);
    B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    if (smem > 200 * 1024) { set_error("router: rows too long for shared memory"); return ECAPACITY; }
  }
  return launch_k(router_kernel, dim3(grid, p.h != nullptr ? 1 : (p.M + 7) / 8), dim3(256), smem, pdl, st, p);
}

// Expert-sorted copy of the activation rows for the tensor-core expert kernels (the reference's
// shaders/llm_moe_perm.comp): sorted row i holds the row of token cols[i] / (used + 1).
__global__ void __launch_bounds__(256) moe_gather_kernel(const __half* xn, const int* cols, int slots1, int H, __half* xperm) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(xn + (size_t)(cols[i] / slots1) * H);
  uint4* dst = reinterpret_cast<uint4*>(xperm + (size_t)i * H);
  for (int k = threadIdx.x; k < H / 8; k += 256) dst[k] = __ldcg(src + k);
}
int launch_moe_gather(const __half* xn, const int* cols, int pairs, int slots1, int H, __half* xperm, bool pdl, cudaStream_t st) {
  return launch_k(moe_gather_kernel, dim3(pairs), dim3(256), 0, pdl, st, xn, cols, slots1, H, xperm);
}

// Row kernels, one CTA per row, for passes of more than QG_FUSED_ROWS rows: RMSNorm, or MoE combine + RMSNorm.
__global__ void __launch_bounds__(QG_THREADS) row_tail_kernel(TailParams tp) {
  __shared__ float scratch[2 * QG_WARPS];
  pdl_wait();
  pdl_launch();
  const int n = blockIdx.x, slots1 = tp.used + 1;
  float* hrow = tp.h + (size_t)n * tp.H;
  if (tp.mode == 2) {
    row_moe_combine(hrow, tp.down + (size_t)n * slots1 * tp.H, tp.topk_w + (size_t)n * slots1, tp.used, tp.H);
    __syncthreads();
  }
  row_rmsnorm_f16(hrow, tp.gamma, tp.eps, tp.H, tp.xn + (size_t)n * tp.H, scratch);
}
int launch_row_tail(const TailParams& tp, bool pdl, cudaStream_t st) {
  return launch_k(row_tail_kernel, dim3(tp.M), dim3(QG_THREADS), 0, pdl, st, tp);
}

// The MoE block's rows of a fused pass finished once instead of in every consumer CTA's staging: row n = residual +
// the expert partial rows, then the next RMSNorm, by the very function the projection kernels stage with (so the
// values are the ones a single-row pass forms in its next projection, bit for bit). grid M, block QG_THREADS.
__global__ void __launch_bounds__(QG_THREADS) combine_rows_kernel(QGemvParams p) {
  __shared__ __align__(16) uint8_t xs[2 * QG_COMBINE_MAX_K + 16 * (QG_COMBINE_MAX_K / 64) + 128];
  __shared__ __align__(16) __half sxs[2 * (QG_COMBINE_MAX_K / 32)];
  __shared__ float scratch[4 * QG_WARPS];
  __shared__ int xrows[1];
  pdl_wait();
  pdl_launch();
  if (threadIdx.x == 0) xrows[0] = blockIdx.x;
  __syncthreads();
  stage_x_combine(p, xs, sxs, scratch, 1, xrows, qg_xstride(p.K), true);
}
int launch_combine_rows(const QGemvParams& p, bool pdl, cudaStream_t st) {
  if (p.K > QG_COMBINE_MAX_K || p.K % 256 || p.used < 0 || p.used > 32 || p.h_out == nullptr || p.h_out == p.hsrc || p.xn_out == nullptr) { set_error("combine_rows: outside its limits"); return EINVAL_; }
  return launch_k(combine_rows_kernel, dim3(p.M), dim3(QG_THREADS), 0, pdl, st, p);
}

// Draft seed input: xcat[n] = fp16(rms(embd[n], enorm)) | fp16(rms(h_prev[n], hnorm))  (llm/mtp.go:352-384)
__global__ void __launch_bounds__(QG_THREADS) concat_norm_kernel(const float* e, const float* hs, const float* enorm, const float* hnorm, float eps, int H, __half* xcat) {
  __shared__ float scratch[2 * QG_WARPS];
  pdl_wait();
  pdl_launch();
  const int n = blockIdx.x;
  row_rmsnorm_f16(e + (size_t)n * H, enorm, eps, H, xcat + (size_t)n * 2 * H, scratch);
  __syncthreads();
  row_rmsnorm_f16(hs + (size_t)n * H, hnorm, eps, H, xcat + (size_t)n * 2 * H + H, scratch);
}
int launch_concat_norm(const float* e, const float* hs, const float* enorm, const float* hnorm, float eps, int H, int M, __half* xcat, bool pdl, cudaStream_t st) {
  return launch_k(concat_norm_kernel, dim3(M), dim3(QG_THREADS), 0, pdl, st, e, hs, enorm, hnorm, eps, H, xcat);
}

// =========================================================================================
// Gated DeltaNet step: alpha/beta projections, causal conv + SiLU, L2 norm, gates, the
// delta-rule state update and read-out (reference: llm/deltanet.go:263-321, 365-455;
// shaders/llm_dn_conv.comp, llm_dn_scan.comp, llm_seq_hist.comp).
// grid (Hv * 4, n_seq): a CTA owns 32 of the 128 state rows of one value head of one
// sequence, keeps them in registers and walks the sequence's tokens in order. The four CTAs
// of a head form a thread-block cluster: the gated RMSNorm over the head's 128 outputs
// (reference: llm/deltanet.go:326-341, shaders/llm_dn_norm.comp) needs their four partial
// sums of squares, exchanged through distributed shared memory.
// =========================================================================================
__device__ __forceinline__ float softplus_ref(float x) {  // llm/deltanet.go:450-455
  if (x > 20.f) return x;
  return logf(1.0f + expf(x));
}
__device__ __forceinline__ float silu_acc(float x) { return x * sigmoid_acc(x); }

// (Passes of 16 sequences and more use dn_head_kernel below instead.)
__global__ void __cluster_dims__(4, 1, 1) __launch_bounds__(128, 1) dn_step_kernel(DnStepParams p) {
  cg::cluster_group cluster = cg::this_cluster();
  const int D = 128, RB = 4;
  const int h = blockIdx.x / RB, rb = blockIdx.x % RB, hk = h % p.Hk;
  const SeqDesc sq = p.seqs[blockIdx.y];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qk = p.Hk * D, H = p.H;
  __shared__ float qs[128], ks[128], vs[32], red[16], wss[4], cta_ss[2][4];  // cta_ss[token parity][row block]
  const int ch_q = hk * D + tid, ch_k = qk + hk * D + tid, ch_v = 2 * qk + h * D + rb * 32 + (tid & 31);
  const float4 cwq = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch_q * 4);
  const float4 cwk = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch_k * 4);
  const float4 cwv = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch_v * 4);
  const float a_h = p.ssm_a[h], dtb = p.dt_bias[h];
  // everything that does not depend on the producer kernel is fetched before waiting for it:
  // the first token's alpha / beta weight slices, the conv history and the state rows
  float4 pwa[4], pwb[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int k = tid * 4 + 512 * i;
    pwa[i] = k < p.H ? *reinterpret_cast<const float4*>(p.alpha_w + (size_t)h * p.H + k) : make_float4(0.f, 0.f, 0.f, 0.f);
    pwb[i] = k < p.H ? *reinterpret_cast<const float4*>(p.beta_w + (size_t)h * p.H + k) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // conv history: the three inputs before pos0, zeros before the sequence start
  // Every CTA keeps a private ring of its own 288 conv inputs (q 128 | k 128 | v 32), indexed
  // by position, so no CTA ever reads what another one writes.
  float* ring = p.ring + (size_t)sq.slot * p.ring_slot_stride + (size_t)blockIdx.x * (DN_RING * DN_RING_W);
  float hq[3], hkk[3], hv[3];
#pragma unroll
  for (int j = 0; j < 3; j++) {
    const int pos = sq.pos0 - 3 + j;
    const float* r = ring + (size_t)(pos & (DN_RING - 1)) * DN_RING_W;
    hq[j] = pos >= 0 ? r[tid] : 0.f;
    hkk[j] = pos >= 0 ? r[128 + tid] : 0.f;
    hv[j] = pos >= 0 ? r[256 + (tid & 31)] : 0.f;
  }
  // state rows of this warp: j = rb*32 + warp*8 + r, four floats per lane
  float* S = p.state + (size_t)sq.slot * p.state_slot_stride + (size_t)h * D * D;
  const int j0 = rb * 32 + warp * 8;
  float4 s[8];
#pragma unroll
  for (int r = 0; r < 8; r++) s[r] = *reinterpret_cast<const float4*>(S + (size_t)(j0 + r) * D + lane * 4);
  const float oscale = 1.0f / sqrtf((float)D);
  const float nw = lane < 8 ? p.norm_w[j0 + lane] : 0.f;  // gated-norm weight of the row this lane writes
  tl_mark(p.tl, 0);
  pdl_wait();
  pdl_launch();
  tl_mark(p.tl, 1);

  for (int i = 0; i < sq.n; i++) {
    const int row = sq.row0 + i, pos = sq.pos0 + i;
    const float* pr = p.proj + (size_t)row * p.ldp;
    // alpha / beta: F32 weights against the fp16-rounded block input
    const __half* xn = p.xn + (size_t)row * H;
    float pa = 0.f, pb = 0.f;
    auto ab_dot = [&](int k, const float4& wa, const float4& wb) {
      const __half2 x01 = *reinterpret_cast<const __half2*>(xn + k), x23 = *reinterpret_cast<const __half2*>(xn + k + 2);
      const float2 f01 = __half22float2(x01), f23 = __half22float2(x23);
      pa += wa.x * f01.x + wa.y * f01.y + wa.z * f23.x + wa.w * f23.y;
      pb += wb.x * f01.x + wb.y * f01.y + wb.z * f23.x + wb.w * f23.y;
    };
#pragma unroll
    for (int ki = 0; ki < 4; ki++) {
      const int k = tid * 4 + 512 * ki;
      if (k < H) {
        if (i == 0) ab_dot(k, pwa[ki], pwb[ki]);
        else ab_dot(k, *reinterpret_cast<const float4*>(p.alpha_w + (size_t)h * H + k), *reinterpret_cast<const float4*>(p.beta_w + (size_t)h * H + k));
      }
    }
    for (int k = tid * 4 + 2048; k < H; k += 512)
      ab_dot(k, *reinterpret_cast<const float4*>(p.alpha_w + (size_t)h * H + k), *reinterpret_cast<const float4*>(p.beta_w + (size_t)h * H + k));
    // conv + SiLU for q, k (whole head) and this CTA's 32 v channels
    const float cq = pr[ch_q], ck = pr[ch_k], cv = pr[ch_v];
    const float zz = lane < 8 ? pr[2 * qk + p.Hv * D + h * D + j0 + lane] : 0.f;  // the gate, asked for with the other inputs
    const float q = silu_acc(hq[0] * cwq.x + hq[1] * cwq.y + hq[2] * cwq.z + cq * cwq.w);
    const float k = silu_acc(hkk[0] * cwk.x + hkk[1] * cwk.y + hkk[2] * cwk.z + ck * cwk.w);
    const float v = silu_acc(hv[0] * cwv.x + hv[1] * cwv.y + hv[2] * cwv.z + cv * cwv.w);
    hq[0] = hq[1]; hq[1] = hq[2]; hq[2] = cq;
    hkk[0] = hkk[1]; hkk[1] = hkk[2]; hkk[2] = ck;
    hv[0] = hv[1]; hv[1] = hv[2]; hv[2] = cv;
    // the ring keeps every token's conv input by position (rollback = moving `past` back)
    {
      float* rw = ring + (size_t)(pos & (DN_RING - 1)) * DN_RING_W;
      rw[tid] = cq; rw[128 + tid] = ck;
      if (tid < 32) rw[256 + tid] = cv;
    }
    float sq2 = warp_sum(q * q), sk2 = warp_sum(k * k);
    pa = warp_sum(pa); pb = warp_sum(pb);
    __syncthreads();
    if (lane == 0) { red[warp] = sq2; red[4 + warp] = sk2; red[8 + warp] = pa; red[12 + warp] = pb; }
    if (tid < 32) vs[tid] = v;
    __syncthreads();
    const float qn = 1.0f / sqrtf(red[0] + red[1] + red[2] + red[3] + p.eps);
    const float kn = 1.0f / sqrtf(red[4] + red[5] + red[6] + red[7] + p.eps);
    const float alpha = red[8] + red[9] + red[10] + red[11], betar = red[12] + red[13] + red[14] + red[15];
    qs[tid] = q * qn;
    ks[tid] = k * kn;
    __syncthreads();
    const float g = expf(softplus_ref(alpha + dtb) * a_h);
    const float beta = sigmoid_acc(betar);
    const float4 k4 = *reinterpret_cast<const float4*>(ks + lane * 4);
    const float4 q4 = *reinterpret_cast<const float4*>(qs + lane * 4);
    float kv[8], oo[8];
#pragma unroll
    for (int r = 0; r < 8; r++) {
      s[r].x *= g; s[r].y *= g; s[r].z *= g; s[r].w *= g;
      kv[r] = s[r].x * k4.x + s[r].y * k4.y + s[r].z * k4.z + s[r].w * k4.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int r = 0; r < 8; r++) kv[r] += __shfl_xor_sync(0xffffffffu, kv[r], o);
    }
#pragma unroll
    for (int r = 0; r < 8; r++) {
      const float dj = (vs[warp * 8 + r] - kv[r]) * beta;
      s[r].x += dj * k4.x; s[r].y += dj * k4.y; s[r].z += dj * k4.z; s[r].w += dj * k4.w;
      oo[r] = s[r].x * q4.x + s[r].y * q4.y + s[r].z * q4.z + s[r].w * q4.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int r = 0; r < 8; r++) oo[r] += __shfl_xor_sync(0xffffffffu, oo[r], o);
    }
    // gated norm: sum of squares over the head's 128 outputs = four CTA partials, added in rank order
    float ov = oo[0] * oscale, ss = 0.f;
#pragma unroll
    for (int r = 0; r < 8; r++) {
      const float orr = oo[r] * oscale;
      ss += orr * orr;
      ov = lane == r ? orr : ov;
    }
    if (lane == 0) wss[warp] = ss;
    __syncthreads();
    // each CTA pushes its partial into the four CTAs' shared memory (thread r writes to rank r), one cluster
    // barrier, then everyone adds the four local copies in rank order: no CTA reads a peer's memory, so none
    // has to outlive a peer's reads
    if (tid < 4) *cluster.map_shared_rank(&cta_ss[i & 1][rb], tid) = wss[0] + wss[1] + wss[2] + wss[3];
    cluster.sync();
    float tot = 0.f;
#pragma unroll
    for (int r = 0; r < 4; r++) tot += cta_ss[i & 1][r];
    if (lane < 8) {
      const int j = j0 + lane;
      const float nsc = 1.0f / sqrtf(tot / (float)D + p.eps);
      p.y16[(size_t)row * (p.Hv * D) + h * D + j] = __float2half_rn(ov * nsc * nw * sigmoid_acc(zz));
    }
    if (p.mid != nullptr) {  // state after token i, for keep-prefix speculation
      float* Sm = p.mid + (size_t)blockIdx.y * p.mid_seq_stride + (size_t)i * p.mid_stride + (size_t)h * D * D;
#pragma unroll
      for (int r = 0; r < 8; r++) *reinterpret_cast<float4*>(Sm + (size_t)(j0 + r) * D + lane * 4) = s[r];
    }
    __syncthreads();
  }
  if (p.mid == nullptr) {
#pragma unroll
    for (int r = 0; r < 8; r++) *reinterpret_cast<float4*>(S + (size_t)(j0 + r) * D + lane * 4) = s[r];
  }
  tl_mark(p.tl, 4);
}

// -----------------------------------------------------------------------------------------
// Many sequences of one or a few tokens (batched decode): one CTA of sixteen warps per (value head,
// sequence) instead of a cluster of four. The alpha / beta projections and the q / k convolutions are
// computed once per head rather than once per row block, the gated norm's sum of squares is a
// shared-memory reduction rather than a cluster barrier, and the state rows, the conv rings and the
// grouping of every partial sum are those of dn_step_kernel (warp W here is warp W % 4 of row block W / 4).
// -----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512, 2) dn_head_kernel(DnStepParams p) {
  const int D = 128, RB = 4;
  const int h = blockIdx.x, hk = h % p.Hk;
  const SeqDesc sq = p.seqs[blockIdx.y];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qk = p.Hk * D, H = p.H;
  __shared__ float qs[128], ks[128], vs[128], red[40], wss[16];
  // conv roles: threads 0..127 the q channels, 128..255 k, 256..383 the head's v channels; the rest idle there
  const int role = tid >> 7, c = tid & 127;
  const int ch = role == 0 ? hk * D + c : role == 1 ? qk + hk * D + c : 2 * qk + h * D + c;
  // ring of row block rb: [pos][q 128 | k 128 | v 32]; q and k are kept in all four, read from the first
  float* ring0 = p.ring + (size_t)sq.slot * p.ring_slot_stride + (size_t)(h * RB) * (DN_RING * DN_RING_W);
  const int ring_off = role == 0 ? c : role == 1 ? 128 + c : (c >> 5) * (DN_RING * DN_RING_W) + 256 + (c & 31);
  float4 cw = make_float4(0.f, 0.f, 0.f, 0.f);
  float hist[3] = {0.f, 0.f, 0.f};
  if (role < 3) {
    cw = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch * 4);
#pragma unroll
    for (int j = 0; j < 3; j++) {
      const int pos = sq.pos0 - 3 + j;
      hist[j] = pos >= 0 ? ring0[(size_t)(pos & (DN_RING - 1)) * DN_RING_W + ring_off] : 0.f;
    }
  }
  const float a_h = p.ssm_a[h], dtb = p.dt_bias[h];
  // state rows of this warp: j = warp*8 + r, four floats per lane
  float* S = p.state + (size_t)sq.slot * p.state_slot_stride + (size_t)h * D * D;
  const int j0 = warp * 8;
  float4 s[8];
#pragma unroll
  for (int r = 0; r < 8; r++) s[r] = *reinterpret_cast<const float4*>(S + (size_t)(j0 + r) * D + lane * 4);
  const float oscale = 1.0f / sqrtf((float)D);
  tl_mark(p.tl, 0);
  pdl_wait();
  pdl_launch();
  tl_mark(p.tl, 1);

  for (int i = 0; i < sq.n; i++) {
    const int row = sq.row0 + i, pos = sq.pos0 + i;
    const float* pr = p.proj + (size_t)row * p.ldp;
    const __half* xn = p.xn + (size_t)row * H;
    float pa = 0.f, pb = 0.f;
    for (int k = tid * 4; k < H; k += 2048) {
      const float4 wa = *reinterpret_cast<const float4*>(p.alpha_w + (size_t)h * H + k), wb = *reinterpret_cast<const float4*>(p.beta_w + (size_t)h * H + k);
      const __half2 x01 = *reinterpret_cast<const __half2*>(xn + k), x23 = *reinterpret_cast<const __half2*>(xn + k + 2);
      const float2 f01 = __half22float2(x01), f23 = __half22float2(x23);
      pa += wa.x * f01.x + wa.y * f01.y + wa.z * f23.x + wa.w * f23.y;
      pb += wb.x * f01.x + wb.y * f01.y + wb.z * f23.x + wb.w * f23.y;
    }
    float cv = 0.f, act = 0.f;
    if (role < 3) {
      cv = pr[ch];
      act = silu_acc(hist[0] * cw.x + hist[1] * cw.y + hist[2] * cw.z + cv * cw.w);
      hist[0] = hist[1]; hist[1] = hist[2]; hist[2] = cv;
      // the rings keep every token's conv input by position (rollback = moving `past` back)
      float* rw = ring0 + (size_t)(pos & (DN_RING - 1)) * DN_RING_W + ring_off;
      if (role == 2) rw[0] = cv;
      else {
#pragma unroll
        for (int rb = 0; rb < RB; rb++) rw[(size_t)rb * (DN_RING * DN_RING_W)] = cv;
      }
    }
    const float a2 = warp_sum(act * act);  // warps 0..3: q, 4..7: k
    pa = warp_sum(pa); pb = warp_sum(pb);
    __syncthreads();
    if (lane == 0) { red[warp] = pa; red[16 + warp] = pb; if (warp < 8) red[32 + warp] = a2; }
    if (role == 2) vs[c] = act;
    __syncthreads();
    const float qn = 1.0f / sqrtf(red[32] + red[33] + red[34] + red[35] + p.eps);
    const float kn = 1.0f / sqrtf(red[36] + red[37] + red[38] + red[39] + p.eps);
    float alpha = 0.f, betar = 0.f;
#pragma unroll
    for (int w = 0; w < 16; w++) { alpha += red[w]; betar += red[16 + w]; }
    if (role == 0) qs[c] = act * qn;
    if (role == 1) ks[c] = act * kn;
    __syncthreads();
    const float g = expf(softplus_ref(alpha + dtb) * a_h);
    const float beta = sigmoid_acc(betar);
    const float4 k4 = *reinterpret_cast<const float4*>(ks + lane * 4);
    const float4 q4 = *reinterpret_cast<const float4*>(qs + lane * 4);
    float kv[8], oo[8];
#pragma unroll
    for (int r = 0; r < 8; r++) {
      s[r].x *= g; s[r].y *= g; s[r].z *= g; s[r].w *= g;
      kv[r] = s[r].x * k4.x + s[r].y * k4.y + s[r].z * k4.z + s[r].w * k4.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int r = 0; r < 8; r++) kv[r] += __shfl_xor_sync(0xffffffffu, kv[r], o);
    }
#pragma unroll
    for (int r = 0; r < 8; r++) {
      const float dj = (vs[j0 + r] - kv[r]) * beta;
      s[r].x += dj * k4.x; s[r].y += dj * k4.y; s[r].z += dj * k4.z; s[r].w += dj * k4.w;
      oo[r] = s[r].x * q4.x + s[r].y * q4.y + s[r].z * q4.z + s[r].w * q4.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int r = 0; r < 8; r++) oo[r] += __shfl_xor_sync(0xffffffffu, oo[r], o);
    }
    // gated norm: sum of squares over the head's 128 outputs, warp partials grouped by four as the row blocks were
    float ov = oo[0] * oscale, ss = 0.f;
#pragma unroll
    for (int r = 0; r < 8; r++) {
      const float orr = oo[r] * oscale;
      ss += orr * orr;
      ov = lane == r ? orr : ov;
    }
    if (lane == 0) wss[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int rb = 0; rb < RB; rb++) tot += wss[4 * rb] + wss[4 * rb + 1] + wss[4 * rb + 2] + wss[4 * rb + 3];
    if (lane < 8) {
      const int j = j0 + lane;
      const float nsc = 1.0f / sqrtf(tot / (float)D + p.eps);
      const float zz = pr[2 * qk + p.Hv * D + h * D + j];
      p.y16[(size_t)row * (p.Hv * D) + h * D + j] = __float2half_rn(ov * nsc * p.norm_w[j] * sigmoid_acc(zz));
    }
    if (p.mid != nullptr) {  // state after token i, for keep-prefix speculation
      float* Sm = p.mid + (size_t)blockIdx.y * p.mid_seq_stride + (size_t)i * p.mid_stride + (size_t)h * D * D;
#pragma unroll
      for (int r = 0; r < 8; r++) *reinterpret_cast<float4*>(Sm + (size_t)(j0 + r) * D + lane * 4) = s[r];
    }
    __syncthreads();
  }
  if (p.mid == nullptr) {
#pragma unroll
    for (int r = 0; r < 8; r++) *reinterpret_cast<float4*>(S + (size_t)(j0 + r) * D + lane * 4) = s[r];
  }
  tl_mark(p.tl, 4);
}

// -----------------------------------------------------------------------------------------
// The same layer for sequences of many tokens (prefill), as three kernels: everything that does not
// depend on the recurrent state (alpha / beta, conv + SiLU, L2 norms, gates) is computed for all tokens
// in parallel and packed per (head, row block) and token; the scan then walks the tokens with no
// block-wide synchronisation at all; the gated norm runs per token afterwards.
// -----------------------------------------------------------------------------------------
// State-independent inputs of the many-token recurrence, written once per pass by dn_pre_kernel and read by every
// CTA that needs them (the four row blocks of a head share its v, decay and beta; the value heads of a key head
// share its q and k): [Hk][rows][256] normalised q | k, then [Hv][rows][128] v, then [Hv][rows][2] decay | beta.
__device__ __forceinline__ float* dn_pre_qk(const DnStepParams& p, int hk, int64_t row) { return p.pre + ((size_t)hk * p.pre_rows + row) * 256; }
__device__ __forceinline__ float* dn_pre_v(const DnStepParams& p, int h, int64_t row) { return p.pre + (size_t)p.Hk * p.pre_rows * 256 + ((size_t)h * p.pre_rows + row) * 128; }
__device__ __forceinline__ float* dn_pre_gb(const DnStepParams& p, int h, int64_t row) {
  return p.pre + (size_t)p.pre_rows * ((size_t)p.Hk * 256 + (size_t)p.Hv * 128) + ((size_t)h * p.pre_rows + row) * 2;
}
constexpr int DN_PRE_TOKENS = 16;
constexpr int DN_CHUNK_FROM = 64;   // sequences of this many tokens and more run the chunked recurrence, shorter ones the token-by-token scan

// alpha / beta projections of all rows of a pass (llm/deltanet.go:305-318): out[row][o], o = head for alpha, Hv + head
// for beta. A CTA keeps 16 rows of the normalised input in shared memory and walks the 2*Hv weight rows once for all
// of them (a warp per weight row, lanes along K), so the weights are read once per 16 tokens instead of once per
// token and row block. grid ceil(M / 16), block 256, dynamic shared memory 16 * H halves.
constexpr int DN_AB_ROWS = 16;
__global__ void __launch_bounds__(256) dn_ab_kernel(DnStepParams p, int M) {
  extern __shared__ __align__(16) uint8_t dn_ab_smem[];
  __half* xs = reinterpret_cast<__half*>(dn_ab_smem);
  const int H = p.H, r0 = blockIdx.x * DN_AB_ROWS, nr = min(DN_AB_ROWS, M - r0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();
  pdl_launch();
  for (int i = tid; i < DN_AB_ROWS * H / 8; i += 256) {
    const int r = i / (H / 8), c = i - r * (H / 8);
    reinterpret_cast<uint4*>(xs)[i] = r < nr ? __ldcg(reinterpret_cast<const uint4*>(p.xn + (size_t)(r0 + r) * H) + c) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  for (int o = warp; o < 2 * p.Hv; o += 8) {
    const float* w = o < p.Hv ? p.alpha_w + (size_t)o * H : p.beta_w + (size_t)(o - p.Hv) * H;
    float acc[DN_AB_ROWS];
#pragma unroll
    for (int r = 0; r < DN_AB_ROWS; r++) acc[r] = 0.f;
    for (int k = lane * 4; k < H; k += 128) {
      const float4 wv = *reinterpret_cast<const float4*>(w + k);
#pragma unroll
      for (int r = 0; r < DN_AB_ROWS; r++) {
        const uint2 xv = *reinterpret_cast<const uint2*>(xs + (size_t)r * H + k);
        const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&xv.x)), f23 = __half22float2(*reinterpret_cast<const __half2*>(&xv.y));
        acc[r] = fmaf(wv.w, f23.y, fmaf(wv.z, f23.x, fmaf(wv.y, f01.y, fmaf(wv.x, f01.x, acc[r]))));
      }
    }
#pragma unroll
    for (int r = 0; r < DN_AB_ROWS; r++) {
      const float v = warp_sum(acc[r]);
      if (lane == 0 && r < nr) p.ab[(size_t)(r0 + r) * 2 * p.Hv + o] = v;
    }
  }
}

// grid (Hk + Hv, n_seq, 16-token groups), block 128. CTAs [0, Hk): q and k of one key head (conv + SiLU + L2 norm);
// CTAs [Hk, Hk + Hv): v of one value head (conv + SiLU) and the head's decay and beta from the projected alpha / beta.
// Conv inputs of the positions before this pass come from the rings the decode kernels keep per (head, row block).
__global__ void __launch_bounds__(128) dn_pre_kernel(DnStepParams p) {
  const int D = 128, RB = 4;
  const bool is_qk = (int)blockIdx.x < p.Hk;
  const int hd = is_qk ? blockIdx.x : blockIdx.x - p.Hk;     // key head or value head
  const SeqDesc sq = p.seqs[blockIdx.y];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qk = p.Hk * D;
  __shared__ float red[8];
  const int i0 = blockIdx.z * DN_PRE_TOKENS, i1 = min(sq.n, i0 + DN_PRE_TOKENS);
  if (i0 >= sq.n) return;
  // channels of the projection row: two (q, k) for a key head, one (v) for a value head
  const int ch_a = is_qk ? hd * D + tid : 2 * qk + hd * D + tid, ch_b = qk + hd * D + tid;
  const float4 cwa = *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch_a * 4);
  const float4 cwb = is_qk ? *reinterpret_cast<const float4*>(p.conv_w + (size_t)ch_b * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
  const float a_h = is_qk ? 0.f : p.ssm_a[hd], dtb = is_qk ? 0.f : p.dt_bias[hd];
  // ring of the decode kernels' CTA (head, row block): q at 0..127 and k at 128..255 of any CTA of a head whose key head
  // this is (head hd, block 0 is one), v at 256..287 of the block that owns the channel
  const float* ring_a = p.ring + (size_t)sq.slot * p.ring_slot_stride + (size_t)(is_qk ? hd * RB : hd * RB + (tid >> 5)) * (DN_RING * DN_RING_W) + (is_qk ? tid : 256 + (tid & 31));
  const float* ring_b = p.ring + (size_t)sq.slot * p.ring_slot_stride + (size_t)(hd * RB) * (DN_RING * DN_RING_W) + 128 + tid;
  pdl_wait();
  pdl_launch();
  // conv input of token index ii (may be negative: before this pass): the projection row, else the ring
  auto input = [&](int ii, int ch, const float* ring) {
    if (ii >= 0) return p.proj[(size_t)(sq.row0 + ii) * p.ldp + ch];
    const int pos = sq.pos0 + ii;
    return pos >= 0 ? ring[(size_t)(pos & (DN_RING - 1)) * DN_RING_W] : 0.f;
  };
  float ha[3], hb[3] = {0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 3; j++) {
    ha[j] = input(i0 - 3 + j, ch_a, ring_a);
    if (is_qk) hb[j] = input(i0 - 3 + j, ch_b, ring_b);
  }
  for (int i = i0; i < i1; i++) {
    const int row = sq.row0 + i;
    const float* pr = p.proj + (size_t)row * p.ldp;
    const float ca = pr[ch_a];
    const float va = silu_acc(ha[0] * cwa.x + ha[1] * cwa.y + ha[2] * cwa.z + ca * cwa.w);
    ha[0] = ha[1]; ha[1] = ha[2]; ha[2] = ca;
    if (is_qk) {
      const float cb = pr[ch_b];
      const float vb = silu_acc(hb[0] * cwb.x + hb[1] * cwb.y + hb[2] * cwb.z + cb * cwb.w);
      hb[0] = hb[1]; hb[1] = hb[2]; hb[2] = cb;
      const float sq2 = warp_sum(va * va), sk2 = warp_sum(vb * vb);
      __syncthreads();
      if (lane == 0) { red[warp] = sq2; red[4 + warp] = sk2; }
      __syncthreads();
      const float qn = 1.0f / sqrtf(red[0] + red[1] + red[2] + red[3] + p.eps);
      const float kn = 1.0f / sqrtf(red[4] + red[5] + red[6] + red[7] + p.eps);
      float* out = dn_pre_qk(p, hd, row);
      out[tid] = va * qn;
      out[128 + tid] = vb * kn;
    } else {
      dn_pre_v(p, hd, row)[tid] = va;
      if (tid == 0) {
        const float alpha = __ldcg(p.ab + (size_t)row * 2 * p.Hv + hd), betar = __ldcg(p.ab + (size_t)row * 2 * p.Hv + p.Hv + hd);
        float* gb = dn_pre_gb(p, hd, row);
        gb[0] = expf(softplus_ref(alpha + dtb) * a_h); gb[1] = sigmoid_acc(betar);
      }
    }
  }
}

// The recurrence itself. A thread owns a quarter (32 of the 128 key dims) of one of the CTA's 32 state
// rows, in registers; per token it needs that quarter of k and q (fetched one token ahead), 32-term dot
// products as four interleaved partial sums, and two shuffles over the four lanes of a row. No shared
// memory and no barrier: every group of four lanes advances on its own. (The summation order differs from
// dn_step_kernel's, so the two forms agree to rounding, not to the bit.)
__global__ void __launch_bounds__(128) dn_scan_kernel(DnStepParams p) {
  const int D = 128, RB = 4;
  const int h = blockIdx.x / RB, rb = blockIdx.x % RB;
  const SeqDesc sq = p.seqs[blockIdx.y];
  const int tid = threadIdx.x, jl = tid >> 2, part = tid & 3;
  const int j = rb * 32 + jl;
  float* Srow = p.state + (size_t)sq.slot * p.state_slot_stride + (size_t)h * D * D + (size_t)j * D + 32 * part;
  float s[32];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const float4 v = *reinterpret_cast<const float4*>(Srow + 4 * i);
    s[4 * i] = v.x; s[4 * i + 1] = v.y; s[4 * i + 2] = v.z; s[4 * i + 3] = v.w;
  }
  const float oscale = 1.0f / sqrtf((float)D);
  pdl_wait();
  pdl_launch();
  const float* pqk = dn_pre_qk(p, h % p.Hk, sq.row0);
  const float* pv = dn_pre_v(p, h, sq.row0) + rb * 32;
  const float* pgb = dn_pre_gb(p, h, sq.row0);
  float4 kq[16], nkq[16];  // k quarter (8 float4) then q quarter
  float vv, nvv = 0.f; float2 gb, ngb = make_float2(0.f, 0.f);
  auto fetch = [&](int i, float4 (&dst)[16], float& v, float2& g) {
    const float* t = pqk + (size_t)i * 256;
#pragma unroll
    for (int u = 0; u < 8; u++) {
      dst[u] = __ldcg(reinterpret_cast<const float4*>(t + 128 + 32 * part + 4 * u));
      dst[8 + u] = __ldcg(reinterpret_cast<const float4*>(t + 32 * part + 4 * u));
    }
    v = __ldcg(pv + (size_t)i * 128 + jl);
    g = __ldcg(reinterpret_cast<const float2*>(pgb + (size_t)i * 2));
  };
  fetch(0, kq, vv, gb);
  for (int i = 0; i < sq.n; i++) {
    if (i + 1 < sq.n) fetch(i + 1, nkq, nvv, ngb);
    const float g = gb.x, beta = gb.y;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
    for (int u = 0; u < 8; u++) {
      a0 = fmaf(s[4 * u], kq[u].x, a0); a1 = fmaf(s[4 * u + 1], kq[u].y, a1);
      a2 = fmaf(s[4 * u + 2], kq[u].z, a2); a3 = fmaf(s[4 * u + 3], kq[u].w, a3);
    }
    float kv = (a0 + a1) + (a2 + a3);
    kv += __shfl_xor_sync(0xffffffffu, kv, 1);
    kv += __shfl_xor_sync(0xffffffffu, kv, 2);
    // S *= g; u = (v - S^T k) * beta; S += k u^T   (llm/deltanet.go:365-418), with g factored out of the dot
    const float dj = (vv - g * kv) * beta;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int u = 0; u < 8; u++) {
      s[4 * u] = fmaf(dj, kq[u].x, s[4 * u] * g); s[4 * u + 1] = fmaf(dj, kq[u].y, s[4 * u + 1] * g);
      s[4 * u + 2] = fmaf(dj, kq[u].z, s[4 * u + 2] * g); s[4 * u + 3] = fmaf(dj, kq[u].w, s[4 * u + 3] * g);
      o0 = fmaf(s[4 * u], kq[8 + u].x, o0); o1 = fmaf(s[4 * u + 1], kq[8 + u].y, o1);
      o2 = fmaf(s[4 * u + 2], kq[8 + u].z, o2); o3 = fmaf(s[4 * u + 3], kq[8 + u].w, o3);
    }
    float ov = (o0 + o1) + (o2 + o3);
    ov += __shfl_xor_sync(0xffffffffu, ov, 1);
    ov += __shfl_xor_sync(0xffffffffu, ov, 2);
    if (part == 0) p.o_raw[(size_t)(sq.row0 + i) * (p.Hv * D) + h * D + j] = ov * oscale;
#pragma unroll
    for (int u = 0; u < 16; u++) kq[u] = nkq[u];
    vv = nvv; gb = ngb;
  }
#pragma unroll
  for (int i = 0; i < 8; i++) *reinterpret_cast<float4*>(Srow + 4 * i) = make_float4(s[4 * i], s[4 * i + 1], s[4 * i + 2], s[4 * i + 3]);
  // the ring keeps the last positions' conv inputs (written here, after every read of the old ring)
  {
    const int hk = h % p.Hk, qk = p.Hk * D;
    const int ch_q = hk * D + tid, ch_k = qk + hk * D + tid, ch_v = 2 * qk + h * D + rb * 32 + (tid & 31);
    float* ring = p.ring + (size_t)sq.slot * p.ring_slot_stride + (size_t)blockIdx.x * (DN_RING * DN_RING_W);
    for (int i = max(0, sq.n - DN_RING); i < sq.n; i++) {
      const float* pr = p.proj + (size_t)(sq.row0 + i) * p.ldp;
      float* rw = ring + (size_t)((sq.pos0 + i) & (DN_RING - 1)) * DN_RING_W;
      rw[tid] = pr[ch_q]; rw[128 + tid] = pr[ch_k];
      if (tid < 32) rw[256 + tid] = pr[ch_v];
    }
  }
}

// -----------------------------------------------------------------------------------------
// The recurrence in chunks of 64 tokens (the chunked form of the gated delta rule). Within a chunk the per-token
// updates  s_j <- g_t s_j + beta_t (v_t[j] - g_t s_j . k_t) k_t  are solved for all tokens at once: with
// L_t = sum_{r<=t} log g_r and ratio(t, r) = exp(L_t - L_r),
//   A[t][r] = beta_t ratio(t, r) (k_t . k_r)  (r < t),      W[t][r] = ratio(t, r) (q_t . k_r)  (r <= t),
//   R[t][j] = beta_t (v_t[j] - exp(L_t) (S0 k_t)[j]),       D[t][j] = R[t][j] - sum_{r<t} A[t][r] D[r][j],
//   o_t[j]  = (exp(L_t) (S0 q_t)[j] + sum_{r<=t} W[t][r] D[r][j]) / sqrt(128),
//   S_C     = exp(L_C) S0 + sum_r ratio(C, r) D[r] k_r^T,
// which is the token-by-token recurrence re-associated (llm/deltanet.go:365-418 is the sequential form; the
// reference has no chunked one, llm/gpu_deltanet.go:48-52). Everything stays f32 (the state and the recurrence
// are f32 throughout in the reference's device path), so the matrix products run on the FMA pipe, register-tiled,
// from shared memory; only the forward substitution for D is sequential (32 columns wide, solved in four blocks of
// 16 tokens). A CTA owns 32 state rows of one head, as dn_scan_kernel does, and reads the same inputs.
// grid (Hv * 4, n_seq), block 512, dynamic shared memory DN_CHUNK_SMEM.
// -----------------------------------------------------------------------------------------
constexpr int DN_C = 64;                       // tokens per chunk
constexpr int DN_KP = 132;                     // pitch of the K and Q rows (floats): 16-byte reads of rows tx, tx+16, .. fall on distinct banks
constexpr int DN_AP = 68;                      // pitch of A and W rows
constexpr int DN_DP = 68;                      // pitch of the solved deltas, kept transposed: DT[j][r]
constexpr size_t DN_CHUNK_SMEM = sizeof(float) * (2 * DN_C * DN_KP + 32 * DN_KP + DN_C * 32 + 32 * DN_DP + 2 * DN_C * DN_AP + 4 * DN_C);

__global__ void __launch_bounds__(512, 1) dn_chunk_kernel(DnStepParams p) {
  const int D = 128, RB = 4;
  const int h = blockIdx.x / RB, rb = blockIdx.x % RB;
  const SeqDesc sq = p.seqs[blockIdx.y];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Two halves of eight warps work side by side: the first on what the forward substitution needs (A, then K S0^T
  // and the right-hand sides) and later on the state, the second on what only the outputs need (Q S0^T, W, then the
  // outputs). w8 / t2 are a thread's warp and thread index inside its half.
  const bool second = warp >= 8;
  const int w8 = warp & 7, t2 = tid & 255;
  // products of token rows with the state block or the deltas: a lane takes four of the 32 columns j (j8 + 8m) and a
  // quarter of the contraction range (cq), eight tokens (w8 + 8u) - 128 multiply-adds per twelve 16-byte reads -
  // and the four lanes of a column add their quarters with two shuffles
  const int j8 = lane & 7, cq = lane >> 3;
  extern __shared__ __align__(16) float dc_smem[];
  float* Ks = dc_smem;                          // [64][DN_KP]
  float* Qs = Ks + DN_C * DN_KP;                // [64][DN_KP]
  float* ST = Qs + DN_C * DN_KP;                // [32 j][DN_KP]: the CTA's 32 state rows
  float* Vs = ST + 32 * DN_KP;                  // [64][32] values, then R
  float* DT = Vs + DN_C * 32;                   // [32 j][DN_DP] the solved deltas, transposed
  float* Am = DT + 32 * DN_DP;                  // [64][DN_AP]
  float* Wm = Am + DN_C * DN_AP;                // [64][DN_AP]
  float* Lg = Wm + DN_C * DN_AP;                // [64] cumulative log decay
  float* Bt = Lg + DN_C;                        // [64] beta
  float* Gm = Bt + DN_C;                        // [64] exp(L_t)
  float* Cr = Gm + DN_C;                        // [64] exp(L_C - L_r)
  float* Sg = p.state + (size_t)sq.slot * p.state_slot_stride + (size_t)h * D * D + (size_t)(rb * 32) * D;
  // the state block does not depend on the producer kernel
  for (int idx = tid; idx < 32 * D; idx += 512) { const int j = idx >> 7, i = idx & 127; ST[j * DN_KP + i] = Sg[idx]; }
  const float oscale = 1.0f / sqrtf((float)D);
  pdl_wait();
  pdl_launch();
  const float* pqk = dn_pre_qk(p, h % p.Hk, sq.row0);
  const float* pv = dn_pre_v(p, h, sq.row0) + rb * 32;
  const float* pgb = dn_pre_gb(p, h, sq.row0);
  const int ty = t2 >> 4, tx = t2 & 15;
  for (int c0 = 0; c0 < sq.n; c0 += DN_C) {
    const int n = min(DN_C, sq.n - c0);
    __syncthreads();                            // the previous chunk's readers are done with every buffer
    // ---- inputs: q, k rows (zero past the end), values, decay and beta ----
    for (int idx = tid; idx < DN_C * 64; idx += 512) {
      const int t = idx >> 6, c = idx & 63;     // 64 float4 per token: 32 of q, 32 of k
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (t < n) v = __ldcg(reinterpret_cast<const float4*>(pqk + (size_t)(c0 + t) * 256 + 4 * c));
      float* dst = (c < 32 ? Qs : Ks) + t * DN_KP + 4 * (c & 31);
      *reinterpret_cast<float4*>(dst) = v;
    }
    for (int idx = tid; idx < DN_C * 32; idx += 512) {
      const int t = idx >> 5, j = idx & 31;
      Vs[idx] = t < n ? __ldcg(pv + (size_t)(c0 + t) * 128 + j) : 0.f;
    }
    if (warp == 0) {                            // cumulative log decay of the chunk: two tokens per lane
      const int t0 = 2 * lane, t1 = t0 + 1;
      const float g0 = t0 < n ? __ldcg(pgb + (size_t)(c0 + t0) * 2) : 1.f, g1 = t1 < n ? __ldcg(pgb + (size_t)(c0 + t1) * 2) : 1.f;
      Bt[t0] = t0 < n ? __ldcg(pgb + (size_t)(c0 + t0) * 2 + 1) : 0.f;
      Bt[t1] = t1 < n ? __ldcg(pgb + (size_t)(c0 + t1) * 2 + 1) : 0.f;
      const float l0 = fmaxf(logf(g0), -87.f), l1 = fmaxf(logf(g1), -87.f);
      float run = l0 + l1;                      // inclusive scan over the lanes' pair sums
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const float up = __shfl_up_sync(0xffffffffu, run, o); if (lane >= o) run += up; }
      Lg[t0] = run - l1; Lg[t1] = run;
      const float total = __shfl_sync(0xffffffffu, run, 31);
      Gm[t0] = expf(run - l1); Gm[t1] = expf(run);
      Cr[t0] = expf(total - (run - l1)); Cr[t1] = expf(total - run);
    }
    __syncthreads();
    // ---- a 64 x 64 product of token rows against the key rows, 4 x 4 per thread: the first half forms
    //      A = beta ratio (K K^T) below the diagonal, the second W = ratio (Q K^T) on and below it ----
    auto gram = [&](const float* Xs, float* Out, bool is_a) {
      float aa[4][4];
#pragma unroll
      for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) aa[a][b] = 0.f;
      for (int i = 0; i < D; i += 4) {
        float4 xt[4], kr[4];
#pragma unroll
        for (int a = 0; a < 4; a++) {
          xt[a] = *reinterpret_cast<const float4*>(Xs + (ty + 16 * a) * DN_KP + i);
          kr[a] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * a) * DN_KP + i);
        }
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
          for (int b = 0; b < 4; b++) aa[a][b] += xt[a].x * kr[b].x + xt[a].y * kr[b].y + xt[a].z * kr[b].z + xt[a].w * kr[b].w;
      }
#pragma unroll
      for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) {
          const int t = ty + 16 * a, r = tx + 16 * b;
          const float ratio = r <= t ? expf(Lg[t] - Lg[r]) : 0.f;
          Out[t * DN_AP + r] = is_a ? (r < t ? Bt[t] * ratio * aa[a][b] : 0.f) : ratio * aa[a][b];
        }
    };
    // ---- out[m][u] = sum_c X[w8 + 8u][c] * Y[j8 + 8m][c] over `len` values of c: X rows of pitch xp (token rows
    //      or W rows), Y rows of pitch yp (the state block or the transposed deltas) ----
    auto rows_times = [&](const float* X, int xp, const float* Y, int yp, int len, float (&out)[4][8]) {
#pragma unroll
      for (int m = 0; m < 4; m++)
#pragma unroll
        for (int u = 0; u < 8; u++) out[m][u] = 0.f;
      const int cbeg = cq * (len / 4);
      for (int c = cbeg; c < cbeg + len / 4; c += 4) {
        float4 yv[4];
#pragma unroll
        for (int m = 0; m < 4; m++) yv[m] = *reinterpret_cast<const float4*>(Y + (j8 + 8 * m) * yp + c);
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const float4 xx = *reinterpret_cast<const float4*>(X + (w8 + 8 * u) * xp + c);
#pragma unroll
          for (int m = 0; m < 4; m++) out[m][u] += xx.x * yv[m].x + xx.y * yv[m].y + xx.z * yv[m].z + xx.w * yv[m].w;
        }
      }
#pragma unroll
      for (int m = 0; m < 4; m++)
#pragma unroll
        for (int u = 0; u < 8; u++) {
          out[m][u] += __shfl_xor_sync(0xffffffffu, out[m][u], 8);
          out[m][u] += __shfl_xor_sync(0xffffffffu, out[m][u], 16);
        }
    };
    float qs[4][8];
    if (!second) {
      gram(Ks, Am, true);
      float ks[4][8];
      rows_times(Ks, DN_KP, ST, DN_KP, D, ks);
      // right-hand sides R; of a column's four lanes, lane cq writes the tokens u = cq and cq + 4
#pragma unroll
      for (int m = 0; m < 4; m++)
#pragma unroll
        for (int u = 0; u < 8; u++)
          if ((u & 3) == cq) {
            const int t = w8 + 8 * u, j = j8 + 8 * m;
            Vs[t * 32 + j] = Bt[t] * (Vs[t * 32 + j] - Gm[t] * ks[m][u]);
          }
      asm volatile("bar.sync 1, 256;" ::: "memory");   // A and R are complete (the first half wrote them)
      // ---- forward substitution D[t] = R[t] - sum_{r<t} A[t][r] D[r] in four blocks of 16 tokens: the part of the sum
      //      that comes from the blocks already solved is taken off the block's right-hand sides by the whole half
      //      (thread -> token t, columns j0 and j0 + 16), then one warp solves the 16 x 16 triangle with the block's
      //      deltas in registers (lane = column j; every index is a compile-time constant, so the loads run ahead of
      //      the chain of dependent multiply-adds) ----
      for (int b = 0; b < DN_C / 16; b++) {
        if (b > 0) {
          const int t = 16 * b + (t2 >> 4), j0 = t2 & 15;
          float s0 = 0.f, s1 = 0.f;
          for (int r = 0; r < 16 * b; r += 4) {
            const float4 a = *reinterpret_cast<const float4*>(Am + t * DN_AP + r);
            const float4 d0 = *reinterpret_cast<const float4*>(DT + j0 * DN_DP + r), d1 = *reinterpret_cast<const float4*>(DT + (j0 + 16) * DN_DP + r);
            s0 += a.x * d0.x + a.y * d0.y + a.z * d0.z + a.w * d0.w;
            s1 += a.x * d1.x + a.y * d1.y + a.z * d1.z + a.w * d1.w;
          }
          Vs[t * 32 + j0] -= s0; Vs[t * 32 + j0 + 16] -= s1;
          asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        if (warp == 0) {
          float d[16];
#pragma unroll
          for (int tl = 0; tl < 16; tl++) {
            const int t = 16 * b + tl;
            float acc = Vs[t * 32 + lane];
            float av[16];
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++)
              if (4 * q4 < tl) {
                const float4 a = *reinterpret_cast<const float4*>(Am + t * DN_AP + 16 * b + 4 * q4);
                av[4 * q4] = a.x; av[4 * q4 + 1] = a.y; av[4 * q4 + 2] = a.z; av[4 * q4 + 3] = a.w;
              }
#pragma unroll
            for (int r = 0; r < 16; r++)
              if (r < tl) acc -= av[r] * d[r];
            d[tl] = acc;
          }
          float* dl = DT + lane * DN_DP + 16 * b;
#pragma unroll
          for (int q4 = 0; q4 < 4; q4++) *reinterpret_cast<float4*>(dl + 4 * q4) = make_float4(d[4 * q4], d[4 * q4 + 1], d[4 * q4 + 2], d[4 * q4 + 3]);
        }
        if (b + 1 < DN_C / 16) asm volatile("bar.sync 1, 256;" ::: "memory");   // the block's deltas are there for the next update
      }
    } else {
      rows_times(Qs, DN_KP, ST, DN_KP, D, qs);
#pragma unroll
      for (int m = 0; m < 4; m++)
#pragma unroll
        for (int u = 0; u < 8; u++) qs[m][u] *= Gm[w8 + 8 * u];
      gram(Qs, Wm, false);
    }
    __syncthreads();
    if (second) {
      // ---- outputs: o_t[j] = (Gamma_t QS + W D) / sqrt(D) ----
      float wd[4][8];
      rows_times(Wm, DN_AP, DT, DN_DP, DN_C, wd);
#pragma unroll
      for (int m = 0; m < 4; m++)
#pragma unroll
        for (int u = 0; u < 8; u++)
          if ((u & 3) == cq) {
            const int t = w8 + 8 * u;
            if (t < n) p.o_raw[(size_t)(sq.row0 + c0 + t) * (p.Hv * D) + h * D + rb * 32 + j8 + 8 * m] = (qs[m][u] + wd[m][u]) * oscale;
          }
    } else {
      // ---- state: S[j][i] = Gamma_C S[j][i] + sum_r Cr[r] D[r][j] K[r][i]: a thread owns columns j = jp, jp + 16 and
      //      the i in [i0, i0 + 4) and [i0 + 64, i0 + 68), and nobody else reads or writes them now (the products with the
      //      old state are done) ----
      const int jp = t2 >> 4, i0 = 4 * (t2 & 15);
      float acc[2][8];
      const float gc = Gm[DN_C - 1];
#pragma unroll
      for (int jj = 0; jj < 2; jj++) {
        const float4 s0 = *reinterpret_cast<const float4*>(ST + (jp + 16 * jj) * DN_KP + i0), s1 = *reinterpret_cast<const float4*>(ST + (jp + 16 * jj) * DN_KP + i0 + 64);
        acc[jj][0] = gc * s0.x; acc[jj][1] = gc * s0.y; acc[jj][2] = gc * s0.z; acc[jj][3] = gc * s0.w;
        acc[jj][4] = gc * s1.x; acc[jj][5] = gc * s1.y; acc[jj][6] = gc * s1.z; acc[jj][7] = gc * s1.w;
      }
      for (int r = 0; r < DN_C; r += 4) {
        const float4 cr = *reinterpret_cast<const float4*>(Cr + r);
        const float4 d0 = *reinterpret_cast<const float4*>(DT + jp * DN_DP + r), d1 = *reinterpret_cast<const float4*>(DT + (jp + 16) * DN_DP + r);
        const float c0v[4] = {cr.x * d0.x, cr.y * d0.y, cr.z * d0.z, cr.w * d0.w}, c1v[4] = {cr.x * d1.x, cr.y * d1.y, cr.z * d1.z, cr.w * d1.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const float4 k0 = *reinterpret_cast<const float4*>(Ks + (r + e) * DN_KP + i0), k1 = *reinterpret_cast<const float4*>(Ks + (r + e) * DN_KP + i0 + 64);
          acc[0][0] += k0.x * c0v[e]; acc[0][1] += k0.y * c0v[e]; acc[0][2] += k0.z * c0v[e]; acc[0][3] += k0.w * c0v[e];
          acc[0][4] += k1.x * c0v[e]; acc[0][5] += k1.y * c0v[e]; acc[0][6] += k1.z * c0v[e]; acc[0][7] += k1.w * c0v[e];
          acc[1][0] += k0.x * c1v[e]; acc[1][1] += k0.y * c1v[e]; acc[1][2] += k0.z * c1v[e]; acc[1][3] += k0.w * c1v[e];
          acc[1][4] += k1.x * c1v[e]; acc[1][5] += k1.y * c1v[e]; acc[1][6] += k1.z * c1v[e]; acc[1][7] += k1.w * c1v[e];
        }
      }
#pragma unroll
      for (int jj = 0; jj < 2; jj++) {
        *reinterpret_cast<float4*>(ST + (jp + 16 * jj) * DN_KP + i0) = make_float4(acc[jj][0], acc[jj][1], acc[jj][2], acc[jj][3]);
        *reinterpret_cast<float4*>(ST + (jp + 16 * jj) * DN_KP + i0 + 64) = make_float4(acc[jj][4], acc[jj][5], acc[jj][6], acc[jj][7]);
      }
    }
  }
  __syncthreads();
  for (int idx = tid; idx < 32 * D; idx += 512) { const int j = idx >> 7, i = idx & 127; Sg[idx] = ST[j * DN_KP + i]; }
  // the ring keeps the last positions' conv inputs (written here, after every read of the old ring by the pre-pass)
  if (tid < 128) {
    const int hk = h % p.Hk, qk = p.Hk * D;
    const int ch_q = hk * D + tid, ch_k = qk + hk * D + tid, ch_v = 2 * qk + h * D + rb * 32 + (tid & 31);
    float* ring = p.ring + (size_t)sq.slot * p.ring_slot_stride + (size_t)blockIdx.x * (DN_RING * DN_RING_W);
    for (int i = max(0, sq.n - DN_RING); i < sq.n; i++) {
      const float* pr = p.proj + (size_t)(sq.row0 + i) * p.ldp;
      float* rw = ring + (size_t)((sq.pos0 + i) & (DN_RING - 1)) * DN_RING_W;
      rw[tid] = pr[ch_q]; rw[128 + tid] = pr[ch_k];
      if (tid < 32) rw[256 + tid] = pr[ch_v];
    }
  }
}

// gated RMSNorm of one token's head: sums of squares grouped as the step kernel groups them (eight rows
// per warp in order, four warps per row block, four row blocks)
__global__ void __launch_bounds__(128) dn_post_kernel(DnStepParams p, int M) {
  const int D = 128, row = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  __shared__ float sq[128], wss[16], tot_sm;
  pdl_wait();
  pdl_launch();
  const float ov = p.o_raw[(size_t)row * (p.Hv * D) + h * D + j];
  sq[j] = ov * ov;
  __syncthreads();
  if (j < 16) {
    float ss = 0.f;
    for (int r = 0; r < 8; r++) ss += sq[j * 8 + r];
    wss[j] = ss;
  }
  __syncthreads();
  if (j == 0) {
    float tot = 0.f;
    for (int rb = 0; rb < 4; rb++) tot += wss[4 * rb] + wss[4 * rb + 1] + wss[4 * rb + 2] + wss[4 * rb + 3];
    tot_sm = tot;
  }
  __syncthreads();
  const float nsc = 1.0f / sqrtf(tot_sm / (float)D + p.eps);
  const float zz = p.proj[(size_t)row * p.ldp + 2 * p.Hk * D + p.Hv * D + h * D + j];
  p.y16[(size_t)row * (p.Hv * D) + h * D + j] = __float2half_rn(ov * nsc * p.norm_w[j] * sigmoid_acc(zz));
}

int launch_dn_scan(const DnStepParams& p, int M, int max_n, bool pdl, cudaStream_t st) {
  if (p.D != 128 || p.conv != 4) { set_error("dn_scan: head dim must be 128 and conv kernel 4"); return EINVAL_; }
  if (p.mid != nullptr || p.pre == nullptr || p.o_raw == nullptr) { set_error("dn_scan: not available for speculative passes"); return EINVAL_; }
  if (p.ab == nullptr || p.H % 128 != 0 || (size_t)DN_AB_ROWS * p.H * 2 > 200 * 1024) { set_error("dn_scan: row length must be a multiple of 128 (at most 6400)"); return EINVAL_; }
  const int ab_smem = DN_AB_ROWS * p.H * 2;
  B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(dn_ab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  B200_TRY(launch_k(dn_ab_kernel, dim3((M + DN_AB_ROWS - 1) / DN_AB_ROWS), dim3(256), ab_smem, pdl, st, p, M));
  B200_TRY(launch_k(dn_pre_kernel, dim3(p.Hk + p.Hv, p.n_seq, (max_n + DN_PRE_TOKENS - 1) / DN_PRE_TOKENS), dim3(128), 0, true, st, p));
  if (max_n >= DN_CHUNK_FROM) {
    // long sequences: the recurrence in chunks of 64 tokens
    B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(dn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DN_CHUNK_SMEM));
    B200_TRY(launch_k(dn_chunk_kernel, dim3(p.Hv * 4, p.n_seq), dim3(512), DN_CHUNK_SMEM, true, st, p));
  } else {
    B200_TRY(launch_k(dn_scan_kernel, dim3(p.Hv * 4, p.n_seq), dim3(128), 0, true, st, p));
  }
  return launch_k(dn_post_kernel, dim3(M, p.Hv), dim3(128), 0, true, st, p, M);
}

int launch_dn_step(const DnStepParams& p, bool pdl, cudaStream_t st) {
  if (p.D != 128 || p.conv != 4) { set_error("dn_step: head dim must be 128 and conv kernel 4"); return EINVAL_; }
  // (passes of at most 8 sequences stay on dn_step_kernel: they give every row the single-row pass's bits)
  if (p.n_seq >= 16) return launch_k(dn_head_kernel, dim3(p.Hv, p.n_seq), dim3(512), 0, pdl, st, p);
  return launch_k(dn_step_kernel, dim3(p.Hv * 4, p.n_seq), dim3(128), 0, pdl, st, p);
}

// =========================================================================================
// Attention pre-pass: per-head RMSNorm of q and k, NeoX partial rotary from a host-built
// table, fp16 K/V into the cache (reference: llm/attn.go:144-184, 510-586;
// shaders/llm_attn_pack.comp). grid (Hq + 2*Hkv, M), block hd.
// =========================================================================================
__global__ void attn_pack_kernel(AttnParams p) {
  const int hd = p.hd, d = threadIdx.x, n = blockIdx.y, which = blockIdx.x;
  __shared__ float buf[256], red[8];
  tl_mark(p.tl, 0);
  // what the producer kernel does not write (position, slot, norm weight, rotary entry) is fetched before waiting for it
  const int pos = p.row_pos[n], slot = p.row_slot[n];
  const float* gamma = which < p.Hq ? p.q_norm : which < p.Hq + p.Hkv ? p.k_norm : nullptr;
  const float gamma_d = gamma != nullptr ? gamma[d] : 0.f;
  const int half = p.rope_dims / 2;
  float2 cs = make_float2(1.f, 0.f);
  if (gamma != nullptr && d < p.rope_dims) cs = *reinterpret_cast<const float2*>(p.rope + ((size_t)(pos + p.rope_off) * half + (d < half ? d : d - half)) * 2);
  pdl_wait();
  pdl_launch();
  tl_mark(p.tl, 1);
  const float* pr = p.proj + (size_t)n * p.ldp;
  const int kv_off = p.Hq * 2 * hd;
  float x;
  if (which < p.Hq) x = pr[which * 2 * hd + d];
  else if (which < p.Hq + p.Hkv) x = pr[kv_off + (which - p.Hq) * hd + d];
  else x = pr[kv_off + p.Hkv * hd + (which - p.Hq - p.Hkv) * hd + d];
  if (gamma != nullptr) {
    float ss = warp_sum(x * x);
    if ((d & 31) == 0) red[d >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < hd / 32; w++) tot += red[w];
    x = x * (1.0f / sqrtf(tot / (float)hd + p.eps)) * gamma_d;
    buf[d] = x;
    __syncthreads();
    if (d < p.rope_dims) {
      const int i = d < half ? d : d - half;
      const float x0 = buf[i], x1 = buf[i + half];
      x = d < half ? x0 * cs.x - x1 * cs.y : x0 * cs.y + x1 * cs.x;
    }
  }
  if (which < p.Hq) p.q16[((size_t)n * p.Hq + which) * hd + d] = __float2half_rn(x);
  else {
    const bool isk = which < p.Hq + p.Hkv;
    const int kh = isk ? which - p.Hq : which - p.Hq - p.Hkv;
    __half* c = (isk ? p.kcache : p.vcache) + (size_t)slot * p.slot_stride + ((size_t)pos * p.Hkv + kh) * hd;
    c[d] = __float2half_rn(x);
  }
}
int launch_attn_pack(const AttnParams& p, bool pdl, cudaStream_t st) {
  if (p.hd > 256 || p.hd % 32) { set_error("attn_pack: head dim must be a multiple of 32, at most 256"); return EINVAL_; }
  return launch_k(attn_pack_kernel, dim3(p.Hq + 2 * p.Hkv, p.M), dim3(p.hd), 0, pdl, st, p);
}

// =========================================================================================
// Split-KV decode attention (reference: llm/attn.go:190-217, 444-496;
// shaders/llm_attn_wmma.comp -DSPLITK, llm_attn_combine.comp). grid (nsplit, Hkv, M):
// a CTA of 4 warps covers `split_cells` cells of one KV head for the G query heads that
// share it.
// =========================================================================================
// -----------------------------------------------------------------------------------------
// Tensor-core form of the same split-KV decode attention. A warp walks 16 cells at a time:
//   S = Q K^T   as mma.m16n8k16 with the G query heads of the KV group on the M axis (the reference's
//               HROWS idea, shaders/llm_attn_wmma.comp:161-190) and 8 cells on N; a lane reads 16 bytes
//               of a K row (the dot product does not care which head dims share a k-slot, so the k-slots
//               are assigned to whatever 8 dims a lane's load covers, in Q and K alike);
//   P = exp(S * scale - m), rounded to fp16 (reference: shaders/llm_attn_wmma.comp:860);
//   O += P V    with the score tile's C registers reused as the A fragment, and V pairs of two cells
//               packed per dim with byte permutes (an in-register transpose; no shared-memory staging).
// Online softmax per warp, warps merged in shared memory, splits merged by attn_merge_kernel.
// -----------------------------------------------------------------------------------------

template <int HD, int G>
__global__ void __launch_bounds__(128) attn_mma_kernel(AttnParams p) {
  constexpr int KS = HD / 16;   // k-steps of the score mma
  constexpr int NB = HD / 64;   // 64-dim blocks of the value mma
  const int split = blockIdx.x, kvh = blockIdx.y, n = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  __shared__ float sm_m[4][G], sm_l[4][G], sm_f[4][G];
  __shared__ __align__(16) float sm_o[4][G][HD + 4];  // padded: the 16-byte stores of a quarter warp spread over the banks
  tl_mark(p.tl, 0);
  // The row's position and slot were written before this pass began. When every sequence has one row in the pass,
  // every cell but the newest was written by earlier passes too: both can be read before the producer kernel
  // (which writes the newest cell and the query) is known to be complete. A warp whose first block lies wholly
  // below the newest cell fetches its keys now.
  const int pos = p.row_pos[n], slot = p.row_slot[n];
  const int ncell = pos + 1;
  const int c0 = split * p.split_cells, c1 = min(ncell, c0 + p.split_cells);
  const float scale = 1.0f / sqrtf((float)HD);
  const size_t cell_stride = (size_t)p.Hkv * HD;
  const __half* kbase = p.kcache + (size_t)slot * p.slot_stride + (size_t)kvh * HD;
  const __half* vbase = p.vcache + (size_t)slot * p.slot_stride + (size_t)kvh * HD;
  uint4 ka4[KS / 2], kb4[KS / 2];
  auto fetch_k = [&](int cb) {
    const int ka = min(cb + g, c1 - 1), kb = min(cb + 8 + g, c1 - 1);  // clamped rows are masked below
    const __half* kra = kbase + (size_t)ka * cell_stride;
    const __half* krb = kbase + (size_t)kb * cell_stride;
#pragma unroll
    for (int j = 0; j < KS / 2; j++) {
      ka4[j] = ldg_stream(kra + 8 * (t + 4 * j));
      kb4[j] = ldg_stream(krb + 8 * (t + 4 * j));
    }
  };
  const int cb_first = c0 + warp * 16;
  const bool early = p.one_row_per_seq && cb_first + 16 <= pos;   // (then also cb_first < c1)
  if (early) fetch_k(cb_first);
  pdl_wait();
  pdl_launch();
  tl_mark(p.tl, 1);
  // query A fragments: head g of the group on row g; rows 8..15 stay zero
  uint32_t qa[KS][2];
#pragma unroll
  for (int j = 0; j < KS / 2; j++) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (g < G) v = *reinterpret_cast<const uint4*>(p.q16 + ((size_t)n * p.Hq + kvh * G + g) * HD + 8 * (t + 4 * j));
    qa[2 * j][0] = v.x; qa[2 * j][1] = v.y; qa[2 * j + 1][0] = v.z; qa[2 * j + 1][1] = v.w;
  }
  float o[HD / 8][2];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) { o[i][0] = 0.f; o[i][1] = 0.f; }
  float m = -INFINITY, l = 0.f;
  for (int cb = c0 + warp * 16; cb < c1; cb += 64) {
    // ---- scores of 16 cells ----
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    if (!(early && cb == cb_first)) fetch_k(cb);
    // the value rows do not depend on the scores: the first two 64-dim blocks are fetched while the score mma
    // runs, the rest as soon as the key registers are free, so every value load is in flight before the softmax
    const int cell_a = cb + 2 * t, cell_c = cb + 8 + 2 * t;
    const int va_c = min(cell_a, c1 - 1), vb_c = min(cell_a + 1, c1 - 1), vc_c = min(cell_c, c1 - 1), vd_c = min(cell_c + 1, c1 - 1);
    uint4 vv[NB][4];
    auto fetch_v = [&](int b) {
      const int doff = 8 * (g + 8 * b);
      vv[b][0] = ldg_stream(vbase + (size_t)va_c * cell_stride + doff); vv[b][1] = ldg_stream(vbase + (size_t)vb_c * cell_stride + doff);
      vv[b][2] = ldg_stream(vbase + (size_t)vc_c * cell_stride + doff); vv[b][3] = ldg_stream(vbase + (size_t)vd_c * cell_stride + doff);
    };
#pragma unroll
    for (int b = 0; b < NB && b < 2; b++) fetch_v(b);
#pragma unroll
    for (int j = 0; j < KS / 2; j++) {
      const uint32_t a0[4] = {qa[2 * j][0], 0u, qa[2 * j][1], 0u}, a1[4] = {qa[2 * j + 1][0], 0u, qa[2 * j + 1][1], 0u};
      mma16816(s0, a0, ka4[j].x, ka4[j].y);
      mma16816(s0, a1, ka4[j].z, ka4[j].w);
      mma16816(s1, a0, kb4[j].x, kb4[j].y);
      mma16816(s1, a1, kb4[j].z, kb4[j].w);
    }
#pragma unroll
    for (int b = 2; b < NB; b++) fetch_v(b);
    // row g, cells cb + 2t, +1 (tile 0) and cb + 8 + 2t, +1 (tile 1)
    float sc[4] = {s0[0] * scale, s0[1] * scale, s1[0] * scale, s1[1] * scale};
    const int cell[4] = {cb + 2 * t, cb + 2 * t + 1, cb + 8 + 2 * t, cb + 9 + 2 * t};
#pragma unroll
    for (int i = 0; i < 4; i++) if (cell[i] >= c1) sc[i] = -INFINITY;
    float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m, mx);                       // finite: a block always holds at least one live cell
    const float corr = expf(m - mn);
    float pv[4];
#pragma unroll
    for (int i = 0; i < 4; i++) pv[i] = expf(sc[i] - mn);
    l = l * corr + ((pv[0] + pv[1]) + (pv[2] + pv[3]));
    m = mn;
    const uint32_t pa[4] = {pack_half2(pv[0], pv[1]), 0u, pack_half2(pv[2], pv[3]), 0u};
    // ---- O = O * corr + P V ----
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const uint4 wa = vv[b][0], wb = vv[b][1], wc = vv[b][2], wd = vv[b][3];
      const uint32_t ra[4] = {wa.x, wa.y, wa.z, wa.w}, rb[4] = {wb.x, wb.y, wb.z, wb.w}, rc[4] = {wc.x, wc.y, wc.z, wc.w}, rd[4] = {wd.x, wd.y, wd.z, wd.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float acc_e[4] = {o[b * 8 + 2 * j][0] * corr, o[b * 8 + 2 * j][1] * corr, 0.f, 0.f};
        float acc_o[4] = {o[b * 8 + 2 * j + 1][0] * corr, o[b * 8 + 2 * j + 1][1] * corr, 0.f, 0.f};
        mma16816(acc_e, pa, __byte_perm(ra[j], rb[j], 0x5410), __byte_perm(rc[j], rd[j], 0x5410));
        mma16816(acc_o, pa, __byte_perm(ra[j], rb[j], 0x7632), __byte_perm(rc[j], rd[j], 0x7632));
        o[b * 8 + 2 * j][0] = acc_e[0]; o[b * 8 + 2 * j][1] = acc_e[1];
        o[b * 8 + 2 * j + 1][0] = acc_o[0]; o[b * 8 + 2 * j + 1][1] = acc_o[1];
      }
    }
  }
  // row sums live as per-lane partials over the four t lanes
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  // n-tile (b, i) column n' holds dim 8 * (n' + 8b) + i; this lane has columns 2t and 2t + 1 of head g
  if (g < G) {
    if (t == 0) { sm_m[warp][g] = m; sm_l[warp][g] = l; }
#pragma unroll
    for (int b = 0; b < NB; b++) {
      float* d0 = &sm_o[warp][g][8 * (2 * t + 8 * b)];
      float* d1 = &sm_o[warp][g][8 * (2 * t + 1 + 8 * b)];
      *reinterpret_cast<float4*>(d0) = make_float4(o[b * 8 + 0][0], o[b * 8 + 1][0], o[b * 8 + 2][0], o[b * 8 + 3][0]);
      *reinterpret_cast<float4*>(d0 + 4) = make_float4(o[b * 8 + 4][0], o[b * 8 + 5][0], o[b * 8 + 6][0], o[b * 8 + 7][0]);
      *reinterpret_cast<float4*>(d1) = make_float4(o[b * 8 + 0][1], o[b * 8 + 1][1], o[b * 8 + 2][1], o[b * 8 + 3][1]);
      *reinterpret_cast<float4*>(d1 + 4) = make_float4(o[b * 8 + 4][1], o[b * 8 + 5][1], o[b * 8 + 6][1], o[b * 8 + 7][1]);
    }
  }
  __syncthreads();
  // the warps' factors exp(m_w - m*) once per head, not once per output element
  if (tid < 4 * G) {
    const int w = tid / G, hh = tid - w * G;
    const float mm = fmaxf(fmaxf(sm_m[0][hh], sm_m[1][hh]), fmaxf(sm_m[2][hh], sm_m[3][hh]));
    sm_f[w][hh] = sm_m[w][hh] == -INFINITY ? 0.f : expf(sm_m[w][hh] - mm);
  }
  __syncthreads();
  const int PW = HD + 2;
  for (int i = tid; i < G * HD; i += 128) {
    const int hh = i / HD, d = i - hh * HD;
    float ov = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) ov += sm_o[w][hh][d] * sm_f[w][hh];
    float* part = p.partial + (((size_t)n * p.Hq + kvh * G + hh) * p.nsplit + split) * PW;
    part[d] = ov;
    if (d == 0) {
      float lv = 0.f;
#pragma unroll
      for (int w = 0; w < 4; w++) lv += sm_l[w][hh] * sm_f[w][hh];
      part[HD] = fmaxf(fmaxf(sm_m[0][hh], sm_m[1][hh]), fmaxf(sm_m[2][hh], sm_m[3][hh]));
      part[HD + 1] = lv;
    }
  }
  tl_mark(p.tl, 4);
}

// -----------------------------------------------------------------------------------------
// Long-split form of the same kernel: eight warps, and the key and value rows reach shared memory by
// bulk copies (one per 16-cell tile row, completing on an mbarrier) instead of passing through registers.
// A warp owns a ring of three tile slots and keeps a whole block (16 keys + 16 values) in flight ahead of
// the block it computes on, so the bytes in flight per SM no longer depend on registers or on which phase
// the warps are in. Row pitches are padded (keys +64 bytes, values +16) so the 16-byte fragment reads of
// a quarter warp fall on distinct banks. Arithmetic and fragment layout are those of attn_mma_kernel.
// -----------------------------------------------------------------------------------------
template <int HD, int G>
__global__ void __launch_bounds__(256, 1) attn_ring_kernel(AttnParams p) {
  constexpr int KS = HD / 16, NB = HD / 64, NW = 8, NSLOT = 3;
  constexpr int KP = HD * 2 + 64, VP = HD * 2 + 16;  // row pitches in bytes
  constexpr int SLOT = 16 * KP;                      // a slot holds the key or the value rows of 16 cells
  extern __shared__ __align__(128) uint8_t ar_ring[];  // [NW][NSLOT][SLOT]; reused for the warps' outputs at the end
  __shared__ uint64_t bars[NW][NSLOT];
  __shared__ float sm_m[NW][G], sm_l[NW][G], sm_f[NW][G];
  const int split = blockIdx.x, kvh = blockIdx.y, n = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  tl_mark(p.tl, 0);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NSLOT; s++) mbar_init(&bars[warp][s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  pdl_wait();
  pdl_launch();
  tl_mark(p.tl, 1);
  const int pos = p.row_pos[n], slot = p.row_slot[n];
  const int ncell = pos + 1;
  const int c0 = split * p.split_cells, c1 = min(ncell, c0 + p.split_cells);
  const float scale = 1.0f / sqrtf((float)HD);
  const size_t cell_stride = (size_t)p.Hkv * HD;
  const __half* kbase = p.kcache + (size_t)slot * p.slot_stride + (size_t)kvh * HD;
  const __half* vbase = p.vcache + (size_t)slot * p.slot_stride + (size_t)kvh * HD;
  uint8_t* ring = ar_ring + (size_t)warp * NSLOT * SLOT;
  const int cb0 = c0 + warp * 16;
  // tile j of this warp: keys (j even) or values (j odd) of block j / 2, in slot j % 3
  auto issue = [&](int j) {
    const int cb = cb0 + (NW * 16) * (j >> 1);
    if (cb >= c1) return;
    const bool isv = j & 1;
    uint64_t* bar = &bars[warp][j % NSLOT];
    uint8_t* dst = ring + (j % NSLOT) * SLOT;
    if (lane == 0) mbar_expect_tx(bar, 16 * HD * 2);
    __syncwarp();  // every lane is done with the slot's previous tile, and the byte count is posted
    if (lane < 16) {
      const int row = min(cb + lane, c1 - 1);  // clamped rows are masked below
      bulk_copy_g2s(dst + lane * (isv ? VP : KP), (isv ? vbase : kbase) + (size_t)row * cell_stride, HD * 2, bar);
    }
  };
  issue(0); issue(1); issue(2);
  uint32_t qa[KS][2];
#pragma unroll
  for (int j = 0; j < KS / 2; j++) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (g < G) v = *reinterpret_cast<const uint4*>(p.q16 + ((size_t)n * p.Hq + kvh * G + g) * HD + 8 * (t + 4 * j));
    qa[2 * j][0] = v.x; qa[2 * j][1] = v.y; qa[2 * j + 1][0] = v.z; qa[2 * j + 1][1] = v.w;
  }
  float o[HD / 8][2];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) { o[i][0] = 0.f; o[i][1] = 0.f; }
  float m = -INFINITY, l = 0.f;
  bool lost = false;
  for (int i = 0, cb = cb0; cb < c1; i++, cb += NW * 16) {
    // ---- scores of 16 cells ----
    const int jk = 2 * i, jv = 2 * i + 1;
    if (!mbar_wait(&bars[warp][jk % NSLOT], (jk / NSLOT) & 1)) { lost = true; break; }
    const uint8_t* kt = ring + (jk % NSLOT) * SLOT + g * KP + t * 16;
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < KS / 2; j++) {
      const uint4 ka = lds128(kt + j * 64), kb = lds128(kt + 8 * KP + j * 64);
      const uint32_t a0[4] = {qa[2 * j][0], 0u, qa[2 * j][1], 0u}, a1[4] = {qa[2 * j + 1][0], 0u, qa[2 * j + 1][1], 0u};
      mma16816(s0, a0, ka.x, ka.y);
      mma16816(s0, a1, ka.z, ka.w);
      mma16816(s1, a0, kb.x, kb.y);
      mma16816(s1, a1, kb.z, kb.w);
    }
    issue(jk + 3);  // the next block's values, into the slot the keys just left
    // row g, cells cb + 2t, +1 (tile 0) and cb + 8 + 2t, +1 (tile 1)
    float sc[4] = {s0[0] * scale, s0[1] * scale, s1[0] * scale, s1[1] * scale};
    const int cell[4] = {cb + 2 * t, cb + 2 * t + 1, cb + 8 + 2 * t, cb + 9 + 2 * t};
#pragma unroll
    for (int u = 0; u < 4; u++) if (cell[u] >= c1) sc[u] = -INFINITY;
    float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m, mx);                       // finite: a block always holds at least one live cell
    const float corr = expf(m - mn);
    float pv[4];
#pragma unroll
    for (int u = 0; u < 4; u++) pv[u] = expf(sc[u] - mn);
    l = l * corr + ((pv[0] + pv[1]) + (pv[2] + pv[3]));
    m = mn;
    const uint32_t pa[4] = {pack_half2(pv[0], pv[1]), 0u, pack_half2(pv[2], pv[3]), 0u};
    // ---- O = O * corr + P V ----
    if (!mbar_wait(&bars[warp][jv % NSLOT], (jv / NSLOT) & 1)) { lost = true; break; }
    const uint8_t* vt = ring + (jv % NSLOT) * SLOT + (2 * t) * VP + g * 16;
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const uint4 wa = lds128(vt + b * 128), wb = lds128(vt + VP + b * 128), wc = lds128(vt + 8 * VP + b * 128), wd = lds128(vt + 9 * VP + b * 128);
      const uint32_t ra[4] = {wa.x, wa.y, wa.z, wa.w}, rb[4] = {wb.x, wb.y, wb.z, wb.w}, rc[4] = {wc.x, wc.y, wc.z, wc.w}, rd[4] = {wd.x, wd.y, wd.z, wd.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float acc_e[4] = {o[b * 8 + 2 * j][0] * corr, o[b * 8 + 2 * j][1] * corr, 0.f, 0.f};
        float acc_o[4] = {o[b * 8 + 2 * j + 1][0] * corr, o[b * 8 + 2 * j + 1][1] * corr, 0.f, 0.f};
        mma16816(acc_e, pa, __byte_perm(ra[j], rb[j], 0x5410), __byte_perm(rc[j], rd[j], 0x5410));
        mma16816(acc_o, pa, __byte_perm(ra[j], rb[j], 0x7632), __byte_perm(rc[j], rd[j], 0x7632));
        o[b * 8 + 2 * j][0] = acc_e[0]; o[b * 8 + 2 * j][1] = acc_e[1];
        o[b * 8 + 2 * j + 1][0] = acc_o[0]; o[b * 8 + 2 * j + 1][1] = acc_o[1];
      }
    }
    issue(jv + 3);  // the keys two blocks ahead, into the slot the values just left
  }
  if (lost && p.err != nullptr && lane == 0) atomicExch(p.err, 1);  // a copy never landed: report; the result is void
  // row sums live as per-lane partials over the four t lanes
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  __syncthreads();  // every warp has consumed what it issued: the ring becomes the warps' output buffer
  float (*sm_o)[G][HD + 4] = reinterpret_cast<float (*)[G][HD + 4]>(ar_ring);  // padded like attn_mma_kernel's
  if (g < G) {
    if (t == 0) { sm_m[warp][g] = m; sm_l[warp][g] = l; }
#pragma unroll
    for (int b = 0; b < NB; b++) {
      float* d0 = &sm_o[warp][g][8 * (2 * t + 8 * b)];
      float* d1 = &sm_o[warp][g][8 * (2 * t + 1 + 8 * b)];
      *reinterpret_cast<float4*>(d0) = make_float4(o[b * 8 + 0][0], o[b * 8 + 1][0], o[b * 8 + 2][0], o[b * 8 + 3][0]);
      *reinterpret_cast<float4*>(d0 + 4) = make_float4(o[b * 8 + 4][0], o[b * 8 + 5][0], o[b * 8 + 6][0], o[b * 8 + 7][0]);
      *reinterpret_cast<float4*>(d1) = make_float4(o[b * 8 + 0][1], o[b * 8 + 1][1], o[b * 8 + 2][1], o[b * 8 + 3][1]);
      *reinterpret_cast<float4*>(d1 + 4) = make_float4(o[b * 8 + 4][1], o[b * 8 + 5][1], o[b * 8 + 6][1], o[b * 8 + 7][1]);
    }
  }
  __syncthreads();
  // the warps' factors exp(m_w - m*) once per head, not once per output element
  if (tid < NW * G) {
    const int w = tid / G, hh = tid - w * G;
    float mm = -INFINITY;
#pragma unroll
    for (int v = 0; v < NW; v++) mm = fmaxf(mm, sm_m[v][hh]);
    sm_f[w][hh] = sm_m[w][hh] == -INFINITY ? 0.f : expf(sm_m[w][hh] - mm);
  }
  __syncthreads();
  const int PW = HD + 2;
  for (int i = tid; i < G * HD; i += 256) {
    const int hh = i / HD, d = i - hh * HD;
    float ov = 0.f;
#pragma unroll
    for (int w = 0; w < NW; w++) ov += sm_o[w][hh][d] * sm_f[w][hh];
    float* part = p.partial + (((size_t)n * p.Hq + kvh * G + hh) * p.nsplit + split) * PW;
    part[d] = ov;
    if (d == 0) {
      float mm = -INFINITY, lv = 0.f;
#pragma unroll
      for (int w = 0; w < NW; w++) { mm = fmaxf(mm, sm_m[w][hh]); lv += sm_l[w][hh] * sm_f[w][hh]; }
      part[HD] = mm; part[HD + 1] = lv;
    }
  }
  tl_mark(p.tl, 4);
}

// -----------------------------------------------------------------------------------------
// Causal attention of a many-row pass of ONE sequence (prefill): query tiles x key/value tiles with an online
// softmax, no per-row split partials and no merge launch (the reference's flash form:
// shaders/llm_attn_wmma.comp:102-117 QT/BM query tiles, :161-190 HROWS). A CTA of eight warps owns 8 * 16 / G
// consecutive query rows of one KV head; a warp takes 16 / G of them with the G query heads of the group, which
// fills the sixteen rows of the mma's M axis (G = 8: rows 2w and 2w + 1 with heads 0..7). Key and value tiles of 32 cells
// reach shared memory by bulk copies (one per cache row, both tensors on one mbarrier, two stages) and are shared
// by the eight warps; the query tile is staged once. Fragment layout, fp16 probabilities and the order of the
// arithmetic are those of the split-KV kernels above; a cell past a row's own position scores -inf.
// The result goes straight to the gated fp16 context rows. grid (ceil(M / (128 / G)), Hkv), block 256.
// -----------------------------------------------------------------------------------------
template <int HD, int G>
__global__ void __launch_bounds__(256, 1) attn_prefill_kernel(AttnParams p) {
  static_assert(G == 8 || G == 4, "the sixteen M rows are 16 / G query rows of G heads");
  constexpr int KS = HD / 16, NB = HD / 64, TC = 32;
  constexpr int RW = 16 / G, QT = 8 * RW;                      // query rows per warp and per CTA
  constexpr int KP = HD * 2 + 64, VP = HD * 2 + 16;           // row pitches in bytes (bank-conflict-free 16-byte reads)
  extern __shared__ __align__(128) uint8_t pf_smem[];          // Q [QT][G][KP] | K [2][TC][KP] | V [2][TC][VP]
  __shared__ __align__(8) uint64_t full[2];
  uint8_t* qs = pf_smem;
  uint8_t* ks = qs + (size_t)QT * G * KP;
  uint8_t* vs = ks + (size_t)2 * TC * KP;
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;      // long rows first
  const int kvh = blockIdx.y, n0 = tile * QT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  if (tid == 0) { mbar_init(&full[0], 1); mbar_init(&full[1], 1); mbar_fence_init(); }
  __syncthreads();
  pdl_wait();
  pdl_launch();
  const int slot = p.row_slot[n0], pos0 = p.row_pos[n0];       // rows of one sequence at consecutive positions
  const int rows = min(QT, p.M - n0);
  const int ncell = pos0 + rows;                                // cells the tile's last row sees
  const int ntile = (ncell + TC - 1) / TC;
  const size_t cell_stride = (size_t)p.Hkv * HD;
  const __half* kbase = p.kcache + (size_t)slot * p.slot_stride + (size_t)kvh * HD;
  const __half* vbase = p.vcache + (size_t)slot * p.slot_stride + (size_t)kvh * HD;
  auto issue = [&](int k) {   // warp 0: key and value rows of tile k into stage k & 1
    if (k >= ntile) return;
    const int s = k & 1;
    if (lane == 0) mbar_expect_tx(&full[s], 2u * TC * HD * 2);
    __syncwarp();
    const int row = min(k * TC + lane, ncell - 1);             // rows past the end repeat the last one and are masked
    bulk_copy_g2s(ks + ((size_t)s * TC + lane) * KP, kbase + (size_t)row * cell_stride, HD * 2, &full[s]);
    bulk_copy_g2s(vs + ((size_t)s * TC + lane) * VP, vbase + (size_t)row * cell_stride, HD * 2, &full[s]);
  };
  if (warp == 0) { issue(0); issue(1); }
  // the query tile: row r, head h at qs + (r * G + h) * KP
  for (int i = tid; i < QT * G * (HD / 8); i += 256) {
    const int d8 = i % (HD / 8), rh = i / (HD / 8), r = rh / G, h = rh - r * G;
    const int n = n0 + min(r, rows - 1);
    *reinterpret_cast<uint4*>(qs + (size_t)rh * KP + d8 * 16) = *reinterpret_cast<const uint4*>(p.q16 + ((size_t)n * p.Hq + kvh * G + h) * HD + d8 * 8);
  }
  __syncthreads();
  // M row g is query row rA with head g % G, M row g + 8 is query row rB with the same head
  const int rA = RW * warp + g / G, rB = rA + 8 / G, hh = g % G;
  const int posA = pos0 + min(rA, rows - 1), posB = pos0 + min(rB, rows - 1);
  const int pos_warp = pos0 + min(RW * warp + RW - 1, rows - 1);   // the warp's last row
  const uint8_t* qa_row = qs + (size_t)(rA * G + hh) * KP + t * 16;
  const uint8_t* qb_row = qs + (size_t)(rB * G + hh) * KP + t * 16;
  const float scale = 1.0f / sqrtf((float)HD);
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) { o[i][0] = 0.f; o[i][1] = 0.f; o[i][2] = 0.f; o[i][3] = 0.f; }
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
  bool lost = false;
  for (int k = 0; k < ntile; k++) {
    const int s = k & 1;
    if (!mbar_wait(&full[s], (uint32_t)((k >> 1) & 1))) { lost = true; break; }
#pragma unroll 1
    for (int blk = 0; blk < TC / 16; blk++) {
      const int cb = k * TC + blk * 16;
      if (cb > pos_warp) break;                                // every cell of the block lies past all of the warp's rows
      // ---- scores of 16 cells for both rows ----
      const uint8_t* kt = ks + ((size_t)s * TC + blk * 16 + g) * KP + t * 16;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < KS / 2; j++) {
        const uint4 qa = lds128(qa_row + j * 64), qb = lds128(qb_row + j * 64);
        const uint4 ka = lds128(kt + j * 64), kb = lds128(kt + 8 * KP + j * 64);
        const uint32_t a0[4] = {qa.x, qb.x, qa.y, qb.y}, a1[4] = {qa.z, qb.z, qa.w, qb.w};
        mma16816(s0, a0, ka.x, ka.y);
        mma16816(s0, a1, ka.z, ka.w);
        mma16816(s1, a0, kb.x, kb.y);
        mma16816(s1, a1, kb.z, kb.w);
      }
      // rows g (A) and g + 8 (B); cells cb + 2t, +1 (tile 0) and cb + 8 + 2t, +1 (tile 1)
      const int cell[4] = {cb + 2 * t, cb + 2 * t + 1, cb + 8 + 2 * t, cb + 9 + 2 * t};
      float sa[4] = {s0[0] * scale, s0[1] * scale, s1[0] * scale, s1[1] * scale};
      float sb[4] = {s0[2] * scale, s0[3] * scale, s1[2] * scale, s1[3] * scale};
#pragma unroll
      for (int u = 0; u < 4; u++) { if (cell[u] > posA) sa[u] = -INFINITY; if (cell[u] > posB) sb[u] = -INFINITY; }
      float mxA = fmaxf(fmaxf(sa[0], sa[1]), fmaxf(sa[2], sa[3])), mxB = fmaxf(fmaxf(sb[0], sb[1]), fmaxf(sb[2], sb[3]));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1)); mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1)); mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      // cell 0 lies at or before every row's position, so the running maxima are finite from the first block on
      const float mnA = fmaxf(mA, mxA), mnB = fmaxf(mB, mxB);
      const float corrA = expf(mA - mnA), corrB = expf(mB - mnB);
      float pa_[4], pb_[4];
#pragma unroll
      for (int u = 0; u < 4; u++) { pa_[u] = expf(sa[u] - mnA); pb_[u] = expf(sb[u] - mnB); }
      lA = lA * corrA + ((pa_[0] + pa_[1]) + (pa_[2] + pa_[3]));
      lB = lB * corrB + ((pb_[0] + pb_[1]) + (pb_[2] + pb_[3]));
      mA = mnA; mB = mnB;
      const uint32_t pa[4] = {pack_half2(pa_[0], pa_[1]), pack_half2(pb_[0], pb_[1]), pack_half2(pa_[2], pa_[3]), pack_half2(pb_[2], pb_[3])};
      // ---- O = O * corr + P V ----
      const uint8_t* vt = vs + ((size_t)s * TC + blk * 16 + 2 * t) * VP + g * 16;
#pragma unroll
      for (int b = 0; b < NB; b++) {
        const uint4 wa = lds128(vt + b * 128), wb = lds128(vt + VP + b * 128), wc = lds128(vt + 8 * VP + b * 128), wd = lds128(vt + 9 * VP + b * 128);
        const uint32_t ra[4] = {wa.x, wa.y, wa.z, wa.w}, rb[4] = {wb.x, wb.y, wb.z, wb.w}, rc[4] = {wc.x, wc.y, wc.z, wc.w}, rd[4] = {wd.x, wd.y, wd.z, wd.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float* oe = o[b * 8 + 2 * j];
          float* oo = o[b * 8 + 2 * j + 1];
          float acc_e[4] = {oe[0] * corrA, oe[1] * corrA, oe[2] * corrB, oe[3] * corrB};
          float acc_o[4] = {oo[0] * corrA, oo[1] * corrA, oo[2] * corrB, oo[3] * corrB};
          mma16816(acc_e, pa, __byte_perm(ra[j], rb[j], 0x5410), __byte_perm(rc[j], rd[j], 0x5410));
          mma16816(acc_o, pa, __byte_perm(ra[j], rb[j], 0x7632), __byte_perm(rc[j], rd[j], 0x7632));
          oe[0] = acc_e[0]; oe[1] = acc_e[1]; oe[2] = acc_e[2]; oe[3] = acc_e[3];
          oo[0] = acc_o[0]; oo[1] = acc_o[1]; oo[2] = acc_o[2]; oo[3] = acc_o[3];
        }
      }
    }
    __syncthreads();                       // every warp is done with stage s
    if (warp == 0) { fence_proxy_async(); issue(k + 2); }
  }
  if (lost && p.err != nullptr && lane == 0) atomicExch(p.err, 1);  // a copy never landed: report; the result is void
  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  // out = O / l * sigmoid(gate) -> fp16 context rows (reference: shaders/llm_attn_combine.comp:100-102)
#pragma unroll
  for (int half = 0; half < 2; half++) {
    const int r = half ? rB : rA;
    if (r >= rows) continue;
    const int n = n0 + r, head = kvh * G + hh;
    const float inv = 1.0f / (half ? lB : lA);
    const float* gate = p.proj + (size_t)n * p.ldp + (size_t)head * 2 * HD + HD;
    __half* dst = p.ctx16 + (size_t)n * p.Hq * HD + (size_t)head * HD;
#pragma unroll
    for (int b = 0; b < NB; b++) {
#pragma unroll
      for (int par = 0; par < 2; par++) {            // o[..][0] and o[..][1] are dims 8 * (2t + par + 8b) + i
        const int d0 = 8 * (2 * t + par + 8 * b);
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const float v0 = o[b * 8 + 2 * i][2 * half + par] * inv * sigmoid_acc(gate[d0 + 2 * i]);
          const float v1 = o[b * 8 + 2 * i + 1][2 * half + par] * inv * sigmoid_acc(gate[d0 + 2 * i + 1]);
          w[i] = pack_half2(v0, v1);
        }
        *reinterpret_cast<uint4*>(dst + d0) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

// Merge of the splits: O = sum_s O_s * exp(m_s - m*), divide by the merged row sum, times
// sigmoid(gate), to fp16 (reference: shaders/llm_attn_combine.comp:43-102). grid (Hq, M), block hd.
__global__ void attn_merge_kernel(AttnParams p) {
  const int head = blockIdx.x, n = blockIdx.y, d = threadIdx.x, hd = p.hd, PW = hd + 2;
  extern __shared__ float mg_f[];  // [nsplit] factors exp(m_s - m*), then [nsplit] row sums
  __shared__ float mg_red[8];
  tl_mark(p.tl, 0);
  // the row's position and its gate (written by the in-projection, three kernels back) do not wait for the splits
  const int nlive = (p.row_pos[n] + 1 + p.split_cells - 1) / p.split_cells;
  const float gate = p.proj[(size_t)n * p.ldp + head * 2 * hd + hd + d];
  pdl_wait();
  pdl_launch();
  tl_mark(p.tl, 1);
  const float* part = p.partial + ((size_t)n * p.Hq + head) * p.nsplit * PW;
  // one round of loads for every split's maximum and row sum, shared through shared memory
  float mloc = -INFINITY;
  for (int sp = d; sp < nlive; sp += blockDim.x) {
    const float ms = __ldcg(part + (size_t)sp * PW + hd);
    mg_f[sp] = ms; mg_f[p.nsplit + sp] = __ldcg(part + (size_t)sp * PW + hd + 1);
    mloc = fmaxf(mloc, ms);
  }
  mloc = warp_max(mloc);
  if ((d & 31) == 0) mg_red[d >> 5] = mloc;
  __syncthreads();
  float mm = -INFINITY;
  for (int w = 0; w < (int)(blockDim.x + 31) / 32; w++) mm = fmaxf(mm, mg_red[w]);
  float ov = 0.f, lv = 0.f;
  int sp = 0;
  for (; sp + 16 <= nlive; sp += 16) {  // sixteen independent loads in flight, summed in split order
    float a[16];
#pragma unroll
    for (int u = 0; u < 16; u++) a[u] = __ldcg(part + (size_t)(sp + u) * PW + d);
#pragma unroll
    for (int u = 0; u < 16; u++) {
      const float ms = mg_f[sp + u];
      const float e = ms == -INFINITY ? 0.f : expf(ms - mm);
      ov += a[u] * e; lv += mg_f[p.nsplit + sp + u] * e;
    }
  }
  for (; sp < nlive; sp++) {
    const float ms = mg_f[sp];
    const float e = ms == -INFINITY ? 0.f : expf(ms - mm);
    ov += __ldcg(part + (size_t)sp * PW + d) * e; lv += mg_f[p.nsplit + sp] * e;
  }
  p.ctx16[(size_t)n * p.Hq * hd + head * hd + d] = __float2half_rn(ov / lv * sigmoid_acc(gate));
  tl_mark(p.tl, 6, true);
}

int launch_attn_decode(const AttnParams& p, bool pdl, cudaStream_t st) {
  const int G = p.Hq / p.Hkv;
  dim3 grid(p.nsplit, p.Hkv, p.M), block(128);
  int s;
  if (p.split_cells >= 256 && ((p.hd == 256 && G == 8) || (p.hd == 128 && G == 4))) {
    // long splits: eight warps fed by bulk copies
    const size_t smem = (size_t)8 * 3 * 16 * (p.hd * 2 + 64);
    B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(attn_ring_kernel<256, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 16 * (256 * 2 + 64)));
    B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(attn_ring_kernel<128, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * 3 * 16 * (128 * 2 + 64)));
    return p.hd == 256 ? launch_k(attn_ring_kernel<256, 8>, grid, dim3(256), smem, pdl, st, p)
                       : launch_k(attn_ring_kernel<128, 4>, grid, dim3(256), smem, pdl, st, p);
  }
  if (p.hd == 256 && G == 8) s = launch_k(attn_mma_kernel<256, 8>, grid, block, 0, pdl, st, p);
  else if (p.hd == 128 && G == 4) s = launch_k(attn_mma_kernel<128, 4>, grid, block, 0, pdl, st, p);
  else if (p.hd == 128 && G == 8) s = launch_k(attn_mma_kernel<128, 8>, grid, block, 0, pdl, st, p);
  else if (p.hd == 256 && G == 4) s = launch_k(attn_mma_kernel<256, 4>, grid, block, 0, pdl, st, p);
  else { set_error("attn_decode: unsupported head_dim / group size (128 or 256 dims, 4 or 8 query heads per KV head)"); return EINVAL_; }
  return s;
}
// many rows of one sequence: the tiled causal kernel (rows [0, M) sit at consecutive positions of one slot)
bool attn_prefill_fits(const AttnParams& p) {
  const int G = p.Hkv > 0 ? p.Hq / p.Hkv : 0;
  return ((G == 8 && p.hd == 256) || (G == 4 && p.hd == 128)) && p.M >= 16;
}
int launch_attn_prefill(const AttnParams& p, bool pdl, cudaStream_t st) {
  if (!attn_prefill_fits(p)) { set_error("attn_prefill: 8 query heads per KV head of 256 dims, or 4 of 128"); return EINVAL_; }
  const int G = p.Hq / p.Hkv, QT = 128 / G;
  const dim3 grid((p.M + QT - 1) / QT, p.Hkv);
  auto smem = [](int hd) { return (size_t)128 * (hd * 2 + 64) + (size_t)2 * 32 * (hd * 2 + 64) + (size_t)2 * 32 * (hd * 2 + 16); };
  B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(attn_prefill_kernel<256, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem(256)));
  B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(attn_prefill_kernel<128, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem(128)));
  return p.hd == 256 ? launch_k(attn_prefill_kernel<256, 8>, grid, dim3(256), smem(256), pdl, st, p)
                     : launch_k(attn_prefill_kernel<128, 4>, grid, dim3(256), smem(128), pdl, st, p);
}
int launch_attn_merge(const AttnParams& p, bool pdl, cudaStream_t st) {
  return launch_k(attn_merge_kernel, dim3(p.Hq, p.M), dim3(p.hd), (size_t)2 * p.nsplit * sizeof(float), pdl, st, p);
}

// =========================================================================================
// Greedy sampling: argmax with ties to the lowest id (reference: llm/sample.go:359-367)
// =========================================================================================
__global__ void __launch_bounds__(1024) argmax_kernel(const float* logits, int V, int32_t* out) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  pdl_wait();
  pdl_launch();
  const float* lg = logits + (size_t)blockIdx.x * V;
  float v = -INFINITY; int idx = 0x7fffffff;
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(lg) & 15) == 0) {
    // four independent 16-byte loads in flight per thread; a thread's indices still rise, so `>` keeps the lowest
    const float4* lg4 = reinterpret_cast<const float4*>(lg);
    const int V4 = V >> 2;
    for (int i0 = threadIdx.x; i0 < V4; i0 += 4 * 1024) {
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; u++) { const int i = i0 + u * 1024; x[u] = i < V4 ? __ldcg(lg4 + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY); }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int e = 4 * (i0 + u * 1024);
        if (x[u].x > v) { v = x[u].x; idx = e; }
        if (x[u].y > v) { v = x[u].y; idx = e + 1; }
        if (x[u].z > v) { v = x[u].z; idx = e + 2; }
        if (x[u].w > v) { v = x[u].w; idx = e + 3; }
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += 1024) {
      float x = lg[i];
      if (x > v) { v = x; idx = i; }
    }
  }
  auto better = [](float a, int ai, float b, int bi2) { return a > b || (a == b && ai < bi2); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, v, o);
    int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (better(ov, oi, v, idx)) { v = ov; idx = oi; }
  }
  if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = v; bi[threadIdx.x >> 5] = idx; }
  __syncthreads();
  if (threadIdx.x < 32) {
    v = bv[threadIdx.x]; idx = bi[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, v, o);
      int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (better(ov, oi, v, idx)) { v = ov; idx = oi; }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
  }
}
int launch_argmax(const float* logits, int M, int V, int32_t* out, bool pdl, cudaStream_t st) {
  return launch_k(argmax_kernel, dim3(M), dim3(1024), 0, pdl, st, logits, V, out);
}

__global__ void advance_kernel(int32_t* ids, const int32_t* next, int* row_pos, SeqDesc* seqs, int M, int32_t* history, int* hist_len) {
  const int i = threadIdx.x;
  if (i < M) {
    ids[i] = next[i];
    row_pos[i] += 1;
    seqs[i].pos0 += 1;
    if (history != nullptr) history[(size_t)(*hist_len) * M + i] = next[i];
  }
  __syncthreads();
  if (i == 0 && hist_len != nullptr) *hist_len += 1;
}
int launch_advance(int32_t* ids, const int32_t* next, int* row_pos, SeqDesc* seqs, int M, int32_t* history, int* hist_len, cudaStream_t st) {
  if (M > 1024) { set_error("advance: too many rows"); return ECAPACITY; }
  advance_kernel<<<1, 1024, 0, st>>>(ids, next, row_pos, seqs, M, history, hist_len);
  B200_CUDA(cudaGetLastError());
  return OK;
}

// =========================================================================================
// Failure-detection probe: a bounded wait that nothing can satisfy. The barrier expects 16 bytes of
// copies and none is issued, so the wait runs out, the error word is set and the kernel returns; no
// copy is in flight and nothing faults. The host then sees the word exactly as it would after a real
// copy that never landed.
// =========================================================================================
__global__ void wait_timeout_probe_kernel(int* err, uint32_t limit) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    mbar_expect_tx(&bar, 16);
    if (!mbar_wait(&bar, 0, limit)) atomicExch(err, 1);
  }
}
int launch_wait_timeout_probe(int* err, cudaStream_t st) {
  wait_timeout_probe_kernel<<<1, 32, 0, st>>>(err, 1u << 16);
  B200_CUDA(cudaGetLastError());
  return OK;
}

}  // namespace b200
