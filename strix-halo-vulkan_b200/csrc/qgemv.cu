#include <algorithm>
// Instantiations and launcher of the fused K-quant projection kernel (qgemv.cuh).
#include "kernels.cuh"

namespace b200 {

// max_entries: grid.y of a launch whose CTAs route for themselves (one per row and slot). Launches over a work list
// ignore it: their grid is the device's resident CTAs, which share the list evenly whatever its length.
template <int TYPE, int PRO, int EPI, bool DUAL, bool GROUPED>
static int launch_one(const QGemvParams& p, int max_entries, bool pdl, cudaStream_t st) {
  auto kernel = qgemv_kernel<TYPE, PRO, EPI, DUAL, GROUPED>;
  const int g_sm_count = sm_count_current();
  if (g_sm_count <= 0) return ECUDA;
  const int nb = p.K / 256;
  const int wpt = nb >= 8 ? 8 : nb >= 4 ? 4 : nb >= 2 ? 2 : 1;
  const int tpc = QG_WARPS / wpt;
  const int tiles = (p.N + 15) / 16;
  const int groups = (tiles + tpc - 1) / tpc;
  const int ny = GROUPED ? max_entries : 1, nz = GROUPED ? 1 : (p.M + QG_MAXCOLS - 1) / QG_MAXCOLS;
  // As many CTAs per SM (up to three: 80 registers per thread) as still leave each a ring of two stages, or of
  // one when it has a single group to walk: more resident warps hide the dequantisation's latencies, and a
  // grid that fits at once needs no second round. Three per SM only for the expert kernels and the Q6_K ones (the head's long walk): elsewhere the register cap costs more than
  // the extra warps give, and every CTA of a projection reads the same activation rows out of L2 - the more
  // CTAs ask at once the longer each waits. Persistent CTAs share the device between the y / z slices.
  const size_t fixed = qg_fixed_smem(p.K, p.xcols, DUAL), stage = qg_stage_bytes(p.K, p.stride, DUAL);
  const size_t budgets[4] = {0, 220 * 1024, 110 * 1024, 72 * 1024};
  if (fixed + stage > budgets[1]) { set_error("qgemv: row length too large for shared memory"); return ECAPACITY; }
  int occ = 1, rounds = 1, gx = 1, ns = 1;
  dim3 grid;
  if (GROUPED && !p.route_here) {
    // A work list: persistent CTAs, each with an equal contiguous share of the list's (entry, group) units. The
    // walk is bound by the instructions that turn quants into fragments, so the resident warps count for more than
    // the ring's depth: three CTAs per SM with a single stage beat two with two stages when three fit.
    occ = fixed + stage <= budgets[3] ? 3 : fixed + stage <= budgets[2] ? 2 : 1;
    ns = (int)((budgets[occ] - fixed) / stage);
    if (ns > QG_MAX_STAGES) ns = QG_MAX_STAGES;
    grid = dim3(g_sm_count * occ, 1, 1);
  } else {
    for (int o = 3; o >= 1; o--) {
      if (o == 3 && !GROUPED && TYPE != T_Q6_K) continue;  // the other plain kernels are compiled for two CTAs per SM
      int cap = g_sm_count * o / (ny * nz);
      if (cap < 1) cap = 1;
      // every CTA walks the same number of groups (a ragged last round leaves most SMs idle)
      rounds = (groups + cap - 1) / cap;
      gx = (groups + rounds - 1) / rounds;
      occ = o;
      if (fixed + (size_t)std::min(rounds, 2) * stage <= budgets[o]) break;
    }
    ns = (int)((budgets[occ] - fixed) / stage);
    if (ns > QG_MAX_STAGES) ns = QG_MAX_STAGES;
    if (ns > rounds) ns = rounds;
    if (ns < 1) ns = 1;
    grid = dim3(gx, ny, nz);
  }
  const size_t smem = fixed + (size_t)ns * stage;
  B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(220 * 1024 + 4096)));
  QGemvParams pp = p;
  pp.nstage = ns;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = dim3(QG_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  B200_CUDA(cudaLaunchKernelEx(&cfg, kernel, pp));
  return OK;
}

template <int TYPE>
static int launch_type(int pro, int epi, bool dual, bool grouped, const QGemvParams& p, int max_entries, bool pdl, cudaStream_t st) {
  if (!grouped && !dual) {
    if (pro == PRO_NORM && epi == EPI_STORE) return launch_one<TYPE, PRO_NORM, EPI_STORE, false, false>(p, 0, pdl, st);
    if (pro == PRO_COMBINE && epi == EPI_STORE) return launch_one<TYPE, PRO_COMBINE, EPI_STORE, false, false>(p, 0, pdl, st);
    if (pro == PRO_F16 && epi == EPI_STORE) return launch_one<TYPE, PRO_F16, EPI_STORE, false, false>(p, 0, pdl, st);
    if (pro == PRO_F16 && epi == EPI_RESID) return launch_one<TYPE, PRO_F16, EPI_RESID, false, false>(p, 0, pdl, st);
  } else if (grouped && pro == PRO_F16) {
    if (dual && epi == EPI_SWIGLU) return launch_one<TYPE, PRO_F16, EPI_SWIGLU, true, true>(p, max_entries, pdl, st);
    if (!dual && epi == EPI_STORE) return launch_one<TYPE, PRO_F16, EPI_STORE, false, true>(p, max_entries, pdl, st);
  }
  set_error("qgemv: this prologue / epilogue combination is not built");
  return EINVAL_;
}

// tile groups a projection of N rows of length K is cut into (= partial sums of squares it leaves per row)
int qgemv_groups(int K, int N) {
  const int nb = K / 256;
  const int wpt = nb >= 8 ? 8 : nb >= 4 ? 4 : nb >= 2 ? 2 : 1;
  const int tpc = QG_WARPS / wpt;
  return ((N + 15) / 16 + tpc - 1) / tpc;
}

// CTAs per tile so that every warp has one (slot, super-block) unit, at most 4
int moe_down1_split(int used, int K) {
  const int units = (used + 1) * (K / 256);
  return std::max(1, std::min(4, (units + QG_WARPS - 1) / QG_WARPS));
}

template <int TYPE>
static int launch_md(const MoeDown1Params& p, int rows, bool pdl, cudaStream_t st) {
  auto kernel = moe_down1_kernel<TYPE>;
  const int slots1 = p.used + 1, cl = p.split;
  const size_t smem = md_smem(p.K, (slots1 + cl - 1) / cl, p.stride);
  if (smem > 200 * 1024) { set_error("moe_down1: tiles too large for shared memory"); return ECAPACITY; }
  B200_ONCE_PER_DEVICE(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(((p.N + 15) / 16) * cl, rows); cfg.blockDim = dim3(QG_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  B200_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return OK;
}

int launch_moe_down1(uint32_t type, const MoeDown1Params& p, int rows, bool pdl, cudaStream_t st) {
  if (p.K % 256 != 0 || p.K <= 0 || p.used + 1 > MD_MAXSLOTS || p.split < 1 || p.split > 4 || p.part == nullptr || rows < 1 || rows > QG_FUSED_ROWS) { set_error("moe_down1: shape outside kernel limits"); return EINVAL_; }
  switch (type) {
    case T_Q4_K: return launch_md<T_Q4_K>(p, rows, pdl, st);
    case T_Q5_K: return launch_md<T_Q5_K>(p, rows, pdl, st);
    case T_Q6_K: return launch_md<T_Q6_K>(p, rows, pdl, st);
  }
  set_error("moe_down1: weight type has no fused projection kernel (Q4_K, Q5_K, Q6_K only)");
  return EINVAL_;
}

int launch_qgemv(uint32_t type, int pro, int epi, bool dual, bool grouped, const QGemvParams& p, int max_entries, bool pdl, cudaStream_t st) {
  if (p.K % 256 != 0 || p.K <= 0) { set_error("qgemv: row length must be a multiple of 256"); return EINVAL_; }
  if (p.xcols < 1 || p.xcols > QG_MAXCOLS) { set_error("qgemv: xcols out of range"); return EINVAL_; }
  if (p.ss_out != nullptr && qgemv_groups(p.K, p.N) > SS_LD) { set_error("qgemv: more tile groups than partial-sum slots"); return ECAPACITY; }
  if (pro == PRO_COMBINE && (p.K > QG_COMBINE_MAX_K || p.used < 0 || p.used > 32 || p.M > QG_MAXCOLS || p.h_out == nullptr || p.h_out == p.hsrc)) { set_error("qgemv: combine prologue outside its limits"); return EINVAL_; }
  if (pro == PRO_NORM && (p.ss_n < 1 || p.ss_n > SS_LD)) { set_error("qgemv: bad partial-sum count"); return EINVAL_; }
  switch (type) {
    case T_Q4_K: return launch_type<T_Q4_K>(pro, epi, dual, grouped, p, max_entries, pdl, st);
    case T_Q5_K: return launch_type<T_Q5_K>(pro, epi, dual, grouped, p, max_entries, pdl, st);
    case T_Q6_K: return launch_type<T_Q6_K>(pro, epi, dual, grouped, p, max_entries, pdl, st);
  }
  set_error("qgemv: weight type has no fused projection kernel (Q4_K, Q5_K, Q6_K only)");
  return EINVAL_;
}

}  // namespace b200
