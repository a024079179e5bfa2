// Instantiations and launcher of the fused K-quant projection kernel (qgemv.cuh).
#include "kernels.cuh"

namespace b200 {

template <int TYPE, int PRO, int EPI, bool DUAL, bool GROUPED>
static int launch_one(const QGemvParams& p, int max_entries, bool pdl, cudaStream_t st) {
  auto kernel = qgemv_kernel<TYPE, PRO, EPI, DUAL, GROUPED>;
  const size_t smem = qg_smem_bytes(p.K, p.xcols, DUAL);
  static size_t configured = 0;
  if (smem > configured) {
    if (smem > 220 * 1024) { set_error("qgemv: row length too large for shared memory"); return ECAPACITY; }
    B200_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  const int nb = p.K / 256;
  const int wpt = nb >= 8 ? 8 : nb >= 4 ? 4 : nb >= 2 ? 2 : 1;
  const int tpc = QG_WARPS / wpt;
  const int tiles = (p.N + 15) / 16;
  dim3 grid((tiles + tpc - 1) / tpc, GROUPED ? max_entries : 1, GROUPED ? 1 : (p.M + QG_MAXCOLS - 1) / QG_MAXCOLS);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = dim3(QG_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  B200_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return OK;
}

template <int TYPE>
static int launch_type(int pro, int epi, bool dual, bool grouped, const QGemvParams& p, int max_entries, bool pdl, cudaStream_t st) {
  if (!grouped && !dual) {
    if (pro == PRO_RMSNORM && epi == EPI_STORE) return launch_one<TYPE, PRO_RMSNORM, EPI_STORE, false, false>(p, 0, pdl, st);
    if (pro == PRO_DN_GATED && epi == EPI_RESID) return launch_one<TYPE, PRO_DN_GATED, EPI_RESID, false, false>(p, 0, pdl, st);
    if (pro == PRO_F16 && epi == EPI_RESID) return launch_one<TYPE, PRO_F16, EPI_RESID, false, false>(p, 0, pdl, st);
    if (pro == PRO_F16 && epi == EPI_STORE) return launch_one<TYPE, PRO_F16, EPI_STORE, false, false>(p, 0, pdl, st);
    if (pro == PRO_CONCAT_NORM && epi == EPI_STORE) return launch_one<TYPE, PRO_CONCAT_NORM, EPI_STORE, false, false>(p, 0, pdl, st);
  } else if (grouped) {
    if (dual && pro == PRO_RMSNORM && epi == EPI_SWIGLU) return launch_one<TYPE, PRO_RMSNORM, EPI_SWIGLU, true, true>(p, max_entries, pdl, st);
    if (!dual && pro == PRO_F16 && epi == EPI_STORE) return launch_one<TYPE, PRO_F16, EPI_STORE, false, true>(p, max_entries, pdl, st);
  }
  set_error("qgemv: this prologue/epilogue combination is not built");
  return EINVAL_;
}

int launch_qgemv(uint32_t type, int pro, int epi, bool dual, bool grouped, const QGemvParams& p, int max_entries, bool pdl, cudaStream_t st) {
  if (p.K % 256 != 0 || p.K <= 0) { set_error("qgemv: row length must be a multiple of 256"); return EINVAL_; }
  if (p.xcols < 1 || p.xcols > QG_MAXCOLS) { set_error("qgemv: xcols out of range"); return EINVAL_; }
  switch (type) {
    case T_Q4_K: return launch_type<T_Q4_K>(pro, epi, dual, grouped, p, max_entries, pdl, st);
    case T_Q5_K: return launch_type<T_Q5_K>(pro, epi, dual, grouped, p, max_entries, pdl, st);
    case T_Q6_K: return launch_type<T_Q6_K>(pro, epi, dual, grouped, p, max_entries, pdl, st);
  }
  set_error("qgemv: weight type has no fused projection kernel (Q4_K, Q5_K, Q6_K only)");
  return EINVAL_;
}

}  // namespace b200
