// tcgen05 / TMEM GEMM for many-row K-quant projections (see qgemm.cuh).
#include <cuda.h>

#include <algorithm>
#include <cstring>
#include <string>
#include <type_traits>

#include "qgemm.cuh"

namespace b200 {

namespace {

constexpr int GM_THREADS = 320;   // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..9: dequant + epilogue
constexpr int GM_ROWS = 128;      // weight rows per tile = UMMA M = TMEM lanes
constexpr int GM_KSTEP = 64;      // fp16 elements per K step = one 128-byte swizzle row
constexpr int A_BYTES = GM_ROWS * 128;
constexpr int GM_SPROB = 1024;    // most problems (experts) of a grouped launch: the list lives in shared memory

__host__ __device__ constexpr int gm_stages(int tn, bool dual) { return tn >= 256 ? (dual ? 3 : 4) : tn >= 128 ? (dual ? 4 : 6) : (dual ? 5 : 8); }
__host__ __device__ constexpr int gm_stage_bytes(int tn, bool dual) { return A_BYTES * (dual ? 2 : 1) + tn * 128; }

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory"); }
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tm, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)), "l"(tm), "r"(c0),
               "r"(c1), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], fp16 x fp16 -> f32
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// 32 consecutive f32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile of 128-byte rows, 128-byte swizzle: rows 128 bytes
// apart, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: f32 accumulate, fp16 A and B, both K-major, M 128, N tn
__host__ __device__ constexpr uint32_t idesc_f16(int tn) { return (1u << 4) | ((uint32_t)(tn >> 3) << 17) | ((uint32_t)(GM_ROWS >> 4) << 24); }

// Weight loads keep their place in the instruction stream (volatile): a block is asked for one whole block of work
// before its first use, and a compiler free to sink the loads next to their uses would undo that.
__device__ __forceinline__ uint4 ldg128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ---- dequantisation of 64 consecutive elements of one weight row ------------------------------
// Each returns the values as eight 16-byte chunks of fp16 (chunk c = elements 8c..8c+7 of the K step).
// Arithmetic follows gguf/dequant.go (unfused multiply, subtract), then one rounding to fp16.
// What a thread holds of its row: one whole super-block (four K steps), fetched one super-block ahead
// of its use so that a block's bytes are requested together (whole DRAM lines, many loads in flight).
template <int TYPE>
struct RawBlock {
  // Q4_K: header, 8 x 16 nibble bytes. Q5_K: header, 2 x 16 fifth-bit bytes, 8 x 16 nibble bytes.
  // Q6_K (row planes): 8 x 16 ql bytes, 4 x 16 qh bytes, 16 int8 scales; d apart.
  // Q8_0 (row planes): 16 x 16 int8 bytes (eight 32-element blocks), their eight fp16 d.
  uint4 q[TYPE == T_Q4_K ? 9 : TYPE == T_Q5_K ? 11 : TYPE == T_Q8_0 ? 17 : 13];
  uint32_t d;
};

// (scale, min) of sub-block 2 * pair + half (gguf/dequant.go:238-243). The twelve packed bytes are the words y, z, w
// of the header quad; `pair` is a compile-time constant at every call, `half` may be a run-time value, so the byte
// inside a word is picked by a shift and no array is indexed.
__device__ __forceinline__ void k4_scale_min_dev(int pair, int half, const uint4& hdr, int& sc, int& m) {
  const int sh = 8 * (2 * (pair & 1) + half);
  if (pair < 2) {
    sc = (int)((hdr.y >> sh) & 63);
    m = (int)((hdr.z >> sh) & 63);
  } else {
    const uint32_t hi = (hdr.w >> sh) & 0xFF;
    sc = (int)((hi & 0xF) | ((((hdr.y >> sh) & 0xFF) >> 6) << 4));
    m = (int)((hi >> 4) | ((((hdr.z >> sh) & 0xFF) >> 6) << 4));
  }
}

template <int TYPE>
__device__ __forceinline__ void load_raw(const uint8_t* row, int nb, int blk, RawBlock<TYPE>& r) {
  if constexpr (TYPE == T_Q4_K || TYPE == T_Q5_K) {
    constexpr int NQ = TYPE == T_Q4_K ? 9 : 11;
    const uint8_t* b = row + (size_t)blk * (16 * NQ);
#pragma unroll
    for (int i = 0; i < NQ; i++) r.q[i] = ldg128(b + 16 * i);
  } else if constexpr (TYPE == T_Q8_0) {  // row planes: qs[K] | d[K/32] fp16
    const uint8_t* qs = row + (size_t)blk * 256;
#pragma unroll
    for (int i = 0; i < 16; i++) r.q[i] = ldg128(qs + 16 * i);
    r.q[16] = ldg128(row + (size_t)nb * 256 + (size_t)blk * 16);
  } else {  // Q6_K row planes: ql[nb][128] | qh[nb][64] | scales[nb][16] | d[nb]
    const uint8_t* ql = row + (size_t)blk * 128;
    const uint8_t* qh = row + (size_t)nb * 128 + (size_t)blk * 64;
#pragma unroll
    for (int i = 0; i < 8; i++) r.q[i] = ldg128(ql + 16 * i);
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[8 + i] = ldg128(qh + 16 * i);
    r.q[12] = ldg128(row + (size_t)nb * 192 + (size_t)blk * 16);
    r.d = __ldg(reinterpret_cast<const unsigned short*>(row + (size_t)nb * 208 + (size_t)blk * 2));
  }
}

// 64 weights -> eight 16-byte chunks of fp16. The quants become exact fp16 integers through the
// 0x6400 exponent trick (1024 + q, minus 1024). The f32 factors d*sc and dmin*m are carried as fp16
// hi + lo pairs, so that the value q*(d*sc) - dmin*m is formed as fma(q, hi, -mhi) + fma(q, lo, -mlo):
// the first term is rounded once, the second is a correction far below its ulp. Against rounding the f32
// value once (the reference's prefill GEMM) this differs by at most one fp16 ulp, independently per weight
// (a single fp16 factor would put the same rounding error on all 32 weights of a sub-block).
__device__ __forceinline__ uint32_t h2_bcast(float v) {
  __half2 h = __float2half2_rn(v);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void h2_split(float v, uint32_t& hi, uint32_t& lo) {
  const __half h = __float2half_rn(v);
  hi = h2_bcast(__half2float(h));
  lo = h2_bcast(v - __half2float(h));
}
// bytes (b0, b1) and (b2, b3) of a word of 0..63 values -> half2 pairs of the exact integers
__device__ __forceinline__ void bytes_to_h2(uint32_t w, uint32_t off, uint32_t& p01, uint32_t& p23) {
  p01 = hadd2_u(__byte_perm(w, 0x64646464u, 0x4140), off);
  p23 = hadd2_u(__byte_perm(w, 0x64646464u, 0x4342), off);
}

// `half` selects which 32 of the K step's 64 elements a thread forms: chunks 4*half .. 4*half+3. It may be a run-time
// value (the two halves of a row then share one instruction stream); j is a compile-time constant at every call.
template <int TYPE>
__device__ __forceinline__ void dequant32(const RawBlock<TYPE>& r, int j, int half, uint4 (&out)[4]) {
  if constexpr (TYPE == T_Q4_K || TYPE == T_Q5_K) {
    // low nibbles are sub-block 2j (half 0), high nibbles sub-block 2j+1 (half 1); word w holds bytes 4w..4w+3
    constexpr int QS = TYPE == T_Q4_K ? 1 : 3;  // first nibble quad
    const uint32_t m1024 = h2_bcast(-1024.f);
    const float d = h2f_lo(r.q[0].x), dmin = h2f_hi(r.q[0].x);
    int sc, m;
    k4_scale_min_dev(j, half, r.q[0], sc, m);
    uint32_t dh, dl, nh, nl;
    h2_split(__fmul_rn(d, (float)sc), dh, dl);
    h2_split(-__fmul_rn(dmin, (float)m), nh, nl);
    const uint4 qa = r.q[QS + 2 * j], qb = r.q[QS + 2 * j + 1];
    const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    uint32_t hb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if constexpr (TYPE == T_Q5_K) {
      hb[0] = r.q[1].x; hb[1] = r.q[1].y; hb[2] = r.q[1].z; hb[3] = r.q[1].w; hb[4] = r.q[2].x; hb[5] = r.q[2].y; hb[6] = r.q[2].z; hb[7] = r.q[2].w;
    }
#pragma unroll
    for (int c = 0; c < 4; c++) {
      uint32_t o[4];
#pragma unroll
      for (int h = 0; h < 2; h++) {
        uint32_t w = (qw[2 * c + h] >> (4 * half)) & 0x0F0F0F0Fu;
        if constexpr (TYPE == T_Q5_K) w |= ((hb[2 * c + h] >> (2 * j + half)) & 0x01010101u) << 4;  // fifth bit -> bit 4
        uint32_t a, b;
        bytes_to_h2(w, m1024, a, b);
        o[2 * h] = hadd2_u(hfma2_u(a, dh, nh), hfma2_u(a, dl, nl));
        o[2 * h + 1] = hadd2_u(hfma2_u(b, dh, nh), hfma2_u(b, dl, nl));
      }
      out[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else if constexpr (TYPE == T_Q8_0) {
    // bytes are int8: flip the sign bit (b + 128 as unsigned), ride the exponent trick, take 1152 off
    const uint32_t m1152 = h2_bcast(-1152.f);
    const uint32_t dw[4] = {r.q[16].x, r.q[16].y, r.q[16].z, r.q[16].w};
    const float dv = half ? h2f_hi(dw[j]) : h2f_lo(dw[j]);  // 32-element block 2j + half of the super-block
    uint32_t ds, dsl;
    h2_split(dv, ds, dsl);
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const uint4 qlo = r.q[4 * j + (c >> 1)], qhi = r.q[4 * j + 2 + (c >> 1)];
      const uint4 qv = half ? qhi : qlo;
      const uint32_t w0 = ((c & 1) ? qv.z : qv.x) ^ 0x80808080u, w1 = ((c & 1) ? qv.w : qv.y) ^ 0x80808080u;
      uint32_t a, b, e, f;
      bytes_to_h2(w0, m1152, a, b);
      bytes_to_h2(w1, m1152, e, f);
      out[c] = make_uint4(hfma2_u(a, ds, hmul2_u(a, dsl)), hfma2_u(b, ds, hmul2_u(b, dsl)), hfma2_u(e, ds, hmul2_u(e, dsl)), hfma2_u(f, ds, hmul2_u(f, dsl)));
    }
  } else {
    const int hf = j >> 1, up = j & 1, quarter = 2 * up + half;  // half hf, quarter: elements l = 0..31
    const float dd = __half2float(__ushort_as_half((unsigned short)r.d));
    const uint4 l0 = half ? r.q[4 * hf + 2] : r.q[4 * hf], l1 = half ? r.q[4 * hf + 3] : r.q[4 * hf + 1], g0 = r.q[8 + 2 * hf], g1 = r.q[9 + 2 * hf];
    const uint32_t lw[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
    const uint32_t hw[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const uint32_t scw[4] = {r.q[12].x, r.q[12].y, r.q[12].z, r.q[12].w};
    const uint32_t m1056 = h2_bcast(-1056.f);  // the 1024 of the exponent trick and the format's centre 32
#pragma unroll
    for (int c = 0; c < 4; c++) {         // l = 8c .. 8c+7: words 2c, 2c+1; scale index 8*hf + l/16 + 2*quarter
      // = 4 * (2*hf + up) + (c >> 1) + 2 * half: the word is fixed at compile time, the byte inside it is not
      const uint32_t scword = scw[2 * hf + up];
      uint32_t ds, dsl;
      h2_split(__fmul_rn(dd, (float)(int)(int8_t)((scword >> (8 * ((c >> 1) + 2 * half))) & 0xFF)), ds, dsl);
      uint32_t o[4];
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const uint32_t w = lw[2 * c + h];
        const uint32_t nib = up ? (w >> 4) & 0x0F0F0F0Fu : w & 0x0F0F0F0Fu;
        const uint32_t v = nib | (((hw[2 * c + h] >> (2 * quarter)) & 0x03030303u) << 4);
        uint32_t a, b;
        bytes_to_h2(v, m1056, a, b);
        o[2 * h] = hfma2_u(a, ds, hmul2_u(a, dsl)); o[2 * h + 1] = hfma2_u(b, ds, hmul2_u(b, dsl));
      }
      out[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// chunks 4*half .. 4*half+3 of row r of a [rows][128-byte] tile under the 128-byte swizzle
__device__ __forceinline__ void store_swizzled(uint8_t* tile, int r, int half, const uint4 (&v)[4]) {
#pragma unroll
  for (int c = 0; c < 4; c++) *reinterpret_cast<uint4*>(tile + r * 128 + (((4 * half + c) ^ (r & 7)) << 4)) = v[c];
}

template <int TYPE, int TN, int EPI>
__global__ void __launch_bounds__(GM_THREADS) qgemm_kernel(const __grid_constant__ CUtensorMap tmx, const QGemmParams p) {
  constexpr bool DUAL = EPI == GEMM_SWIGLU;
  constexpr int NS = gm_stages(TN, DUAL), STAGE = gm_stage_bytes(TN, DUAL), B_OFF = A_BYTES * (DUAL ? 2 : 1);
  constexpr uint32_t TCOLS = (DUAL ? 2 : 1) * TN < 32 ? 32 : (DUAL ? 2 : 1) * TN;  // 64, 128, 256 or 512: a power of two
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_a[NS], full_b[NS], empty[NS], acc_full, acc_empty;
  __shared__ uint32_t tmem_base_sm;
  __shared__ volatile int failed;
  __shared__ GemmProblem sprob[GM_SPROB];
  __shared__ int stile[GM_SPROB + 1];   // activation tiles before each problem (exclusive scan)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < NS; s++) { mbar_init(&full_a[s], 8); mbar_init(&full_b[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(&acc_full, 1); mbar_init(&acc_empty, 8);
    mbar_fence_init();
    failed = 0;
  }
  if (warp == 1) tmem_alloc(&tmem_base_sm, TCOLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_sm;
  pdl_wait();
  pdl_launch();

  const int n_prob = p.n_problems != nullptr ? min(*p.n_problems, p.max_problems) : 1;
  const int K = p.K, nb = K / 256, ksteps = K / GM_KSTEP;
  // Work items: (problem, activation-row tile, weight-row tile), the weight tile fastest, over the tiles the problems
  // really have: a scan of ceil(count / TN) per problem, made once per CTA, turns an item index into its problem by
  // bisection. CTAs next to each other work on the same activation tile (read through L2 once).
  const int n_tiles = (p.N + GM_ROWS - 1) / GM_ROWS;
  if (p.problems != nullptr) {
    for (int e = tid; e < n_prob; e += GM_THREADS) sprob[e] = p.problems[e];
  } else if (tid == 0) {
    sprob[0] = p.one;
  }
  __syncthreads();
  if (warp == 0) {
    const int per = (n_prob + 31) / 32;
    int c = 0;
    for (int i = 0; i < per; i++) { const int e = lane * per + i; if (e < n_prob) c += (sprob[e].count + TN - 1) / TN; }
    int cs = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int up = __shfl_up_sync(0xffffffffu, cs, o); if (lane >= o) cs += up; }
    int run = cs - c;
    for (int i = 0; i < per; i++) { const int e = lane * per + i; if (e < n_prob) { stile[e] = run; run += (sprob[e].count + TN - 1) / TN; } }
    if (lane == 31) stile[n_prob] = cs;
  }
  __syncthreads();
  const int total = stile[n_prob] * n_tiles;
  auto item = [&](int idx, GemmProblem& pr, int& nt, int& tt) {
    const int tile = idx / n_tiles;
    nt = idx - tile * n_tiles;
    int lo = 0, hi = n_prob - 1;          // the last problem whose first tile is not after `tile`
    while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (stile[mid] <= tile) lo = mid; else hi = mid - 1; }
    pr = sprob[lo];
    tt = tile - stile[lo];
    return true;
  };
  auto give_up = [&]() { if (p.err != nullptr) atomicExch(p.err, 1); failed = 1; };

  if (warp == 0) {
    // ---- activation tiles by TMA -----------------------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int idx = blockIdx.x; idx < total && !failed; idx += gridDim.x) {
        GemmProblem pr; int nt, tt;
        if (!item(idx, pr, nt, tt)) continue;
        for (int ks = 0; ks < ksteps; ks++, it++) {
          const int s = it % NS;
          if (!mbar_wait(&empty[s], ((it / NS) & 1) ^ 1)) { give_up(); break; }
          mbar_expect_tx(&full_b[s], TN * 128);
          tma_load_2d(smem + (size_t)s * STAGE + B_OFF, &tmx, ks * GM_KSTEP, pr.x_row0 + tt * TN, &full_b[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue ---------------------------------------------------------------------------
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      constexpr uint32_t idesc = idesc_f16(TN);
      for (int idx = blockIdx.x; idx < total && !failed; idx += gridDim.x) {
        GemmProblem pr; int nt, tt;
        if (!item(idx, pr, nt, tt)) continue;
        if (!mbar_wait(&acc_empty, (tcount & 1) ^ 1)) { give_up(); break; }  // the epilogue has drained the accumulator
        tc_fence_after();
        bool ok = true;
        for (int ks = 0; ks < ksteps; ks++, it++) {
          const int s = it % NS;
          const uint32_t ph = (it / NS) & 1;
          if (!mbar_wait(&full_a[s], ph) || !mbar_wait(&full_b[s], ph)) { give_up(); ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE), b_addr = a_addr + B_OFF;
          const uint64_t adesc = smem_desc_sw128(a_addr), bdesc = smem_desc_sw128(b_addr);
#pragma unroll
          for (int k4 = 0; k4 < GM_KSTEP / 16; k4++) {  // 32 bytes along K per instruction: +2 in the address field
            tc_mma_f16(tmem_base, adesc + 2 * k4, bdesc + 2 * k4, idesc, (ks | k4) != 0);
            if constexpr (DUAL) tc_mma_f16(tmem_base + TN, smem_desc_sw128(a_addr + A_BYTES) + 2 * k4, bdesc + 2 * k4, idesc, (ks | k4) != 0);
          }
          tc_commit(&empty[s]);  // arrives when the instructions above have read the stage
        }
        if (!ok) break;
        tc_commit(&acc_full);
        tcount++;
      }
    }
  } else {
    // ---- dequantisation, then the epilogue ------------------------------------------------------
    // warps 2..5 form the first 32 elements of every row's K step and drain the first half of the
    // accumulator's columns, warps 6..9 the second halves: two warps per scheduler hide each other's latencies.
    // Both halves run the same instructions (`half` is data), and the loop over a row's super-blocks is not
    // unrolled, so the loop body stays small enough for the instruction caches.
    const int half = warp >= 6 ? 1 : 0;
    const int r = ((warp - 2) & 3) * 32 + lane;    // weight row of the tile this thread dequantises
    const int q = warp & 3;                        // TMEM lane quarter this warp may read
    uint32_t it = 0, tcount = 0;
    RawBlock<TYPE> cur, nxt;
    bool primed = false;                           // cur already holds the first block of the item about to start
    for (int idx = blockIdx.x; idx < total && !failed; idx += gridDim.x) {
      GemmProblem pr; int nt, tt;
      if (!item(idx, pr, nt, tt)) continue;
      const int wrow = min(nt * GM_ROWS + r, p.N - 1);
      // Gated pair: warps 2..5 form the whole K step of the gate tensor, warps 6..9 that of the up tensor
      // (a thread then holds super-blocks of one tensor only).
      const uint8_t* myrow = (DUAL && half ? p.w2 : p.w) + (size_t)pr.expert * p.expert_stride + (size_t)wrow * p.stride;
      bool ok = true;
      // one K step: dequantise, wait for the stage to be free, store the swizzled tile, signal the MMA warp
      auto step = [&](const RawBlock<TYPE>& ra, int j) {
        const int s = it % NS;
        uint4 v[4], v2[4];
        if constexpr (DUAL) { dequant32<TYPE>(ra, j, 0, v); dequant32<TYPE>(ra, j, 1, v2); }
        else dequant32<TYPE>(ra, j, half, v);
        if (!mbar_wait(&empty[s], ((it / NS) & 1) ^ 1)) { give_up(); ok = false; return; }
        uint8_t* a = smem + (size_t)s * STAGE;
        if constexpr (DUAL) { store_swizzled(a + half * A_BYTES, r, 0, v); store_swizzled(a + half * A_BYTES, r, 1, v2); }
        else store_swizzled(a, r, half, v);
        fence_proxy_async();                       // make the generic-proxy stores visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_a[s]);
        it++;
      };
      if (!primed) load_raw<TYPE>(myrow, nb, 0, cur);
#pragma unroll 1
      for (int blk = 0; blk < nb && ok; blk++) {
        if (blk + 1 < nb) load_raw<TYPE>(myrow, nb, blk + 1, nxt);
#pragma unroll
        for (int j = 0; j < 4; j++) if (ok) step(cur, j);
        cur = nxt;
      }
      if (!ok) break;
      // the first block of this thread's row in the CTA's next item is asked for now and arrives under the epilogue
      primed = false;
      if (idx + (int)gridDim.x < total) {
        GemmProblem npr; int nnt, ntt;
        item(idx + gridDim.x, npr, nnt, ntt);
        const uint8_t* nrow = (DUAL && half ? p.w2 : p.w) + (size_t)npr.expert * p.expert_stride + (size_t)min(nnt * GM_ROWS + r, p.N - 1) * p.stride;
        load_raw<TYPE>(nrow, nb, 0, cur);
        primed = true;
      }
      if (!mbar_wait(&acc_full, tcount & 1)) { give_up(); break; }
      tc_fence_after();
      const int orow = nt * GM_ROWS + q * 32 + lane;  // TMEM lane = weight row
      const int t0 = tt * TN;
#pragma unroll 1
      for (int c0 = half * (TN / 2); c0 < (half + 1) * (TN / 2); c0 += 32) {
        // output row of column c0 + lane (-1: past the problem's rows), fetched by the lanes side by side and handed
        // round by shuffles: no store below waits for a load of its own
        int my_row = -1;
        if (t0 + c0 + lane < pr.count) my_row = p.y_rows != nullptr ? __ldg(p.y_rows + pr.y_row0 + t0 + c0 + lane) : pr.y_row0 + t0 + c0 + lane;
        uint32_t acc[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c0, acc);
        if constexpr (DUAL) {
          uint32_t up[32];
          tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + TN + c0, up);
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const int yr = __shfl_sync(0xffffffffu, my_row, i);
            if (yr >= 0 && orow < p.N) {
              const float g = __uint_as_float(acc[i]), u = __uint_as_float(up[i]);
              p.y16[(int64_t)yr * p.ldy + orow] = __float2half_rn(g * sigmoid_acc(g) * u);  // shaders/llm_moe_gemv.comp:777-781
            }
          }
        } else if constexpr (EPI == GEMM_RESID) {
          // the old values first, all of them in flight together, then the sums
          float old[32];
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const int yr = __shfl_sync(0xffffffffu, my_row, i);
            old[i] = 0.f;
            if (yr >= 0 && orow < p.N) asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(old[i]) : "l"(p.y + (int64_t)yr * p.ldy + orow));
          }
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const int yr = __shfl_sync(0xffffffffu, my_row, i);
            if (yr >= 0 && orow < p.N) p.y[(int64_t)yr * p.ldy + orow] = old[i] + __uint_as_float(acc[i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) {
            const int yr = __shfl_sync(0xffffffffu, my_row, i);
            if (yr >= 0 && orow < p.N) p.y[(int64_t)yr * p.ldy + orow] = __uint_as_float(acc[i]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty);
      tcount++;
    }
  }
  // ---- teardown: every thread arrives; tensor memory is released by the warp that took it -------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TCOLS);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

template <int TYPE, int TN, int EPI>
int launch_t(const QGemmParams& p, const CUtensorMap& tm, bool pdl, cudaStream_t st) {
  constexpr bool DUAL = EPI == GEMM_SWIGLU;
  auto kernel = qgemm_kernel<TYPE, TN, EPI>;
  const size_t smem = (size_t)gm_stages(TN, DUAL) * gm_stage_bytes(TN, DUAL) + 1024;
  B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int sm_count = sm_count_current();
  if (sm_count <= 0) return ECUDA;
  const int n_tiles = (p.N + GM_ROWS - 1) / GM_ROWS;
  if (p.problems != nullptr && p.max_problems > GM_SPROB) { set_error("qgemm: more problems than the kernel's shared-memory list holds (1024)"); return ECAPACITY; }
  // upper bound of the items: every problem's tiles, each problem rounding up at most once
  const int64_t total = ((int64_t)(p.max_count + TN - 1) / TN + (p.problems != nullptr ? p.max_problems : 0)) * n_tiles;
  const int gx = (int)std::max<int64_t>(1, std::min<int64_t>(total, sm_count)), gy = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(gx, gy); cfg.blockDim = dim3(GM_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  B200_CUDA(cudaLaunchKernelEx(&cfg, kernel, tm, p));
  return OK;
}

template <int TYPE, int TN>
int launch_epi(int epi, const QGemmParams& p, const CUtensorMap& tm, bool pdl, cudaStream_t st) {
  switch (epi) {
    case GEMM_STORE: return launch_t<TYPE, TN, GEMM_STORE>(p, tm, pdl, st);
    case GEMM_RESID: return launch_t<TYPE, TN, GEMM_RESID>(p, tm, pdl, st);
    case GEMM_SWIGLU: return launch_t<TYPE, TN, GEMM_SWIGLU>(p, tm, pdl, st);
  }
  set_error("qgemm: unknown epilogue");
  return EINVAL_;
}
template <int TYPE>
int launch_tn(int epi, int tn, const QGemmParams& p, const CUtensorMap& tm, bool pdl, cudaStream_t st) {
  if (tn == 64) return launch_epi<TYPE, 64>(epi, p, tm, pdl, st);
  if (tn == 128) return launch_epi<TYPE, 128>(epi, p, tm, pdl, st);
  if (tn == 256 && epi != GEMM_SWIGLU) return launch_epi<TYPE, 256>(epi, p, tm, pdl, st);
  set_error("qgemm: activation tile must be 64, 128 or 256 rows (128 at most for the gated pair)");
  return EINVAL_;
}

}  // namespace

int make_x_tensor_map(const __half* x, int64_t rows, int K, int tn, void* out) {
  static EncodeTiledFn encode = nullptr;
  if (encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    B200_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (fn == nullptr || qres != cudaDriverEntryPointSuccess) { set_error("qgemm: the driver does not export cuTensorMapEncodeTiled"); return ECUDA; }
    encode = (EncodeTiledFn)fn;
  }
  if (K % GM_KSTEP != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) { set_error("qgemm: activations must be 16-byte aligned with a row length that is a multiple of 64"); return EINVAL_; }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(__half)};
  const cuuint32_t box[2] = {(cuuint32_t)GM_KSTEP, (cuuint32_t)tn};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("qgemm: cuTensorMapEncodeTiled failed with code " + std::to_string((int)r)); return ECUDA; }
  return OK;
}

int launch_qgemm(uint32_t type, int epi, int tn, const QGemmParams& p, const void* tmap_host, bool pdl, cudaStream_t st) {
  if (p.K % 256 != 0 || p.K <= 0) { set_error("qgemm: row length must be a multiple of 256"); return EINVAL_; }
  CUtensorMap tm;
  memcpy(&tm, tmap_host, sizeof(tm));
  switch (type) {
    case T_Q4_K: return launch_tn<T_Q4_K>(epi, tn, p, tm, pdl, st);
    case T_Q5_K: return launch_tn<T_Q5_K>(epi, tn, p, tm, pdl, st);
    case T_Q6_K: return launch_tn<T_Q6_K>(epi, tn, p, tm, pdl, st);
    case T_Q8_0:
      if (epi == GEMM_STORE && tn == 64) return launch_t<T_Q8_0, 64, GEMM_STORE>(p, tm, pdl, st);
      break;
  }
  set_error("qgemm: weight type has no tensor-core projection kernel (Q4_K, Q5_K, Q6_K; Q8_0 with 64-row tiles and a plain store)");
  return EINVAL_;
}

}  // namespace b200
