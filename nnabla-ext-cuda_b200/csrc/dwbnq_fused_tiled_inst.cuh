// Instantiates the tiled fused kernels for one (element type, kernel size) pair; each
// fused_tiled_*.cu includes this with DWBNQ_INST_T / DWBNQ_INST_K defined so the four
// families compile in parallel.
#include "dwbnq_fused.cuh"

namespace dwbnq {

namespace {

typedef void (*TiledKernel)(const CUtensorMap, const FusedArgs, const TileCfg);

template <typename T, int K, int STRIDE, int MODE>
TiledKernel pick_qm(int qm) {
  switch (qm) {
    case QM_NONE: return fused_tiled_kernel<T, K, STRIDE, kRowsPerPatch, QM_NONE, MODE>;
    case QM_FPQ: return fused_tiled_kernel<T, K, STRIDE, kRowsPerPatch, QM_FPQ, MODE>;
    case QM_POW2: return fused_tiled_kernel<T, K, STRIDE, kRowsPerPatch, QM_POW2, MODE>;
    case QM_MM_APPLY: return fused_tiled_kernel<T, K, STRIDE, kRowsPerPatch, QM_MM_APPLY, MODE>;
    case QM_MM_REDUCE: return fused_tiled_kernel<T, K, STRIDE, kRowsPerPatch, QM_MM_REDUCE, MODE>;
    case QM_FPQ_LEAN: return fused_tiled_kernel<T, K, STRIDE, kRowsPerPatch, QM_FPQ_LEAN, MODE>;
  }
  return nullptr;
}

template <typename T, int K, int STRIDE>
TiledKernel pick_mode(int qm, int mode) {
  switch (mode) {
    case TM_TMA: return pick_qm<T, K, STRIDE, TM_TMA>(qm);
    case TM_COOP: return pick_qm<T, K, STRIDE, TM_COOP>(qm);
    case TM_RAW: return pick_qm<T, K, STRIDE, TM_RAW>(qm);
  }
  return nullptr;
}

template <typename T, int K>
TiledKernel pick(int stride, int qm, int mode) {
  if (stride == 1) return pick_mode<T, K, 1>(qm, mode);
  if (stride == 2) return pick_mode<T, K, 2>(qm, mode);
  return nullptr;
}

}  // namespace

template <>
cudaError_t launch_tiled<DWBNQ_INST_T, DWBNQ_INST_K>(int stride, int qm, int mode, const CUtensorMap &tmap,
                                                     const FusedArgs &a, const TileCfg &c, int ctas,
                                                     int threads, size_t smem, cudaStream_t stream) {
  (void)threads;
  TiledKernel kern = pick<DWBNQ_INST_T, DWBNQ_INST_K>(stride, qm, mode);
  if (!kern) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  // block = (strips, planes, row blocks): one patch per thread
  kern<<<(unsigned int)ctas, dim3(c.n_strips, c.P, c.n_rb), smem, stream>>>(tmap, a, c);
  return cudaGetLastError();
}

}  // namespace dwbnq
