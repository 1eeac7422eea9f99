// Instantiates the tiled fused kernels for one (element type, kernel size) pair; each
// fused_tiled_*.cu includes this with DWBNQ_INST_T / DWBNQ_INST_K defined so the four
// families compile in parallel.
#include "dwbnq_fused.cuh"

namespace dwbnq {

namespace {

template <typename T, int K, int STRIDE, int QM, bool USE_TMA>
cudaError_t launch_one(const CUtensorMap &tmap, const FusedArgs &a, const TileCfg &c,
                       long long ctas, int threads, size_t smem, cudaStream_t stream) {
  auto kern = fused_tiled_kernel<T, K, STRIDE, kRowsPerPatch, QM, USE_TMA>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned int)ctas, threads, smem, stream>>>(tmap, a, c);
  return cudaGetLastError();
}

template <typename T, int K, int STRIDE, bool USE_TMA>
cudaError_t launch_qm(int qm, const CUtensorMap &tmap, const FusedArgs &a, const TileCfg &c,
                      long long ctas, int threads, size_t smem, cudaStream_t stream) {
  switch (qm) {
    case QM_NONE: return launch_one<T, K, STRIDE, QM_NONE, USE_TMA>(tmap, a, c, ctas, threads, smem, stream);
    case QM_FPQ: return launch_one<T, K, STRIDE, QM_FPQ, USE_TMA>(tmap, a, c, ctas, threads, smem, stream);
    case QM_POW2: return launch_one<T, K, STRIDE, QM_POW2, USE_TMA>(tmap, a, c, ctas, threads, smem, stream);
    case QM_MM_APPLY: return launch_one<T, K, STRIDE, QM_MM_APPLY, USE_TMA>(tmap, a, c, ctas, threads, smem, stream);
    case QM_MM_REDUCE: return launch_one<T, K, STRIDE, QM_MM_REDUCE, USE_TMA>(tmap, a, c, ctas, threads, smem, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

template <>
cudaError_t launch_tiled<DWBNQ_INST_T, DWBNQ_INST_K>(int stride, int qm, bool use_tma,
                                                     const CUtensorMap &tmap, const FusedArgs &a,
                                                     const TileCfg &c, long long ctas, int threads,
                                                     size_t smem, cudaStream_t stream) {
  using T = DWBNQ_INST_T;
  constexpr int K = DWBNQ_INST_K;
  if (stride == 1) {
    return use_tma ? launch_qm<T, K, 1, true>(qm, tmap, a, c, ctas, threads, smem, stream)
                   : launch_qm<T, K, 1, false>(qm, tmap, a, c, ctas, threads, smem, stream);
  }
  if (stride == 2) {
    return use_tma ? launch_qm<T, K, 2, true>(qm, tmap, a, c, ctas, threads, smem, stream)
                   : launch_qm<T, K, 2, false>(qm, tmap, a, c, ctas, threads, smem, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace dwbnq
