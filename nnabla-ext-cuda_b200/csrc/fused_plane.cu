// Instantiations and dispatch of the small-plane fused kernel (7x7 and 14x14 planes).
#include "dwbnq_internal.h"

namespace dwbnq {

namespace {

typedef void (*PlaneKernel)(const FusedArgs, const PlaneCfg);

template <typename T, int W, int NRB>
PlaneKernel pick_qm(int qm) {
  switch (qm) {
    case QM_NONE: return fused_plane_kernel<T, W, NRB, QM_NONE>;
    case QM_FPQ: return fused_plane_kernel<T, W, NRB, QM_FPQ>;
    case QM_POW2: return fused_plane_kernel<T, W, NRB, QM_POW2>;
    case QM_MM_APPLY: return fused_plane_kernel<T, W, NRB, QM_MM_APPLY>;
    case QM_MM_REDUCE: return fused_plane_kernel<T, W, NRB, QM_MM_REDUCE>;
    case QM_FPQ_LEAN: return fused_plane_kernel<T, W, NRB, QM_FPQ_LEAN>;
  }
  return nullptr;
}

template <typename T>
cudaError_t launch_t(int w, int qm, const FusedArgs &a, const PlaneCfg &c, cudaStream_t stream) {
  PlaneKernel kern = nullptr;
  size_t smem = 0;
  if (w == 7) {
    kern = pick_qm<T, 7, 1>(qm);
    smem = plane_smem_bytes(7, 1, sizeof(T));
  } else if (w == 14) {
    kern = pick_qm<T, 14, 2>(qm);
    smem = plane_smem_bytes(14, 2, sizeof(T));
  }
  if (!kern) return cudaErrorInvalidValue;
  // all of the unified L1 / shared memory as shared memory: the tiles are the working set
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned int)c.n_tiles, 32, smem, stream>>>(a, c);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_plane(int dtype, int w, int qm, const FusedArgs &a, const PlaneCfg &c,
                         cudaStream_t stream) {
  return dtype == DWBNQ_F32 ? launch_t<float>(w, qm, a, c, stream) : launch_t<__half>(w, qm, a, c, stream);
}

}  // namespace dwbnq
