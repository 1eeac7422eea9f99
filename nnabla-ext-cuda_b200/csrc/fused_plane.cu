// Instantiations and dispatch of the small-plane fused kernels (7x7, 14x14, 28x28 planes).
#include <cstdlib>

#include "dwbnq_internal.h"

namespace dwbnq {

namespace {

typedef void (*PlaneKernel)(const FusedArgs, const PlaneCfg);

template <typename T, int W, int NRB, int NCB, int NBND>
PlaneKernel pick_s1(int qm) {
  switch (qm) {
    case QM_NONE: return fused_plane_kernel<T, W, NRB, NCB, NBND, QM_NONE>;
    case QM_FPQ: return fused_plane_kernel<T, W, NRB, NCB, NBND, QM_FPQ>;
    case QM_POW2: return fused_plane_kernel<T, W, NRB, NCB, NBND, QM_POW2>;
    case QM_MM_APPLY: return fused_plane_kernel<T, W, NRB, NCB, NBND, QM_MM_APPLY>;
    case QM_MM_REDUCE: return fused_plane_kernel<T, W, NRB, NCB, NBND, QM_MM_REDUCE>;
    case QM_FPQ_LEAN: return fused_plane_kernel<T, W, NRB, NCB, NBND, QM_FPQ_LEAN>;
    case QM_MM_REDUCE_STORE: return fused_plane_kernel<T, W, NRB, NCB, NBND, QM_MM_REDUCE_STORE>;
  }
  return nullptr;
}

// 8-bit storage: FixedPointQuantize modes, fp32 arithmetic
template <int W, int NRB, int NCB, int NBND>
PlaneKernel pick_s1_code8(int qm) {
  if (qm == QM_FPQ) return fused_plane_kernel<float, W, NRB, NCB, NBND, QM_FPQ, true>;
  if (qm == QM_FPQ_LEAN) return fused_plane_kernel<float, W, NRB, NCB, NBND, QM_FPQ_LEAN, true>;
  return nullptr;
}
template <int NRB, int NCB, int NBND>
PlaneKernel pick_s2_code8(int qm) {
  if (qm == QM_FPQ) return fused_plane_s2_kernel<float, NRB, NCB, NBND, QM_FPQ, true>;
  if (qm == QM_FPQ_LEAN) return fused_plane_s2_kernel<float, NRB, NCB, NBND, QM_FPQ_LEAN, true>;
  return nullptr;
}
PlaneKernel pick_pair7_code8(int qm) {
  if (qm == QM_FPQ) return fused_plane_pair7_kernel<float, QM_FPQ, true>;
  if (qm == QM_FPQ_LEAN) return fused_plane_pair7_kernel<float, QM_FPQ_LEAN, true>;
  return nullptr;
}
PlaneKernel pick_code8(int k, int hw, int stride, int qm) {
  if (stride == 1 && k == 3) {
    if (hw == 7) return pick_pair7_code8(qm);
    if (hw == 14) return pick_s1_code8<14, 2, 1, 1>(qm);
    if (hw == 28) return pick_s1_code8<14, 4, 2, 1>(qm);
    if (hw == 56) return pick_s1_code8<14, 8, 4, 1>(qm);
    if (hw == 112) return pick_s1_code8<14, 4, 8, 4>(qm);
  } else if (stride == 2 && k == 3) {
    if (hw == 14) return pick_s2_code8<1, 1, 1>(qm);
    if (hw == 28) return pick_s2_code8<2, 2, 1>(qm);
    if (hw == 56) return pick_s2_code8<4, 4, 1>(qm);
    if (hw == 112) return pick_s2_code8<4, 8, 2>(qm);
  }
  return nullptr;
}

template <typename T, int K, int W, int NRB, int NCB, int NBND>
PlaneKernel pick_kxk(int qm) {
  switch (qm) {
    case QM_NONE: return fused_plane_kxk_kernel<T, K, W, NRB, NCB, NBND, QM_NONE>;
    case QM_FPQ: return fused_plane_kxk_kernel<T, K, W, NRB, NCB, NBND, QM_FPQ>;
    case QM_POW2: return fused_plane_kxk_kernel<T, K, W, NRB, NCB, NBND, QM_POW2>;
    case QM_MM_APPLY: return fused_plane_kxk_kernel<T, K, W, NRB, NCB, NBND, QM_MM_APPLY>;
    case QM_MM_REDUCE: return fused_plane_kxk_kernel<T, K, W, NRB, NCB, NBND, QM_MM_REDUCE>;
    case QM_FPQ_LEAN: return fused_plane_kxk_kernel<T, K, W, NRB, NCB, NBND, QM_FPQ_LEAN>;
    case QM_MM_REDUCE_STORE: return fused_plane_kxk_kernel<T, K, W, NRB, NCB, NBND, QM_MM_REDUCE_STORE>;
  }
  return nullptr;
}

template <typename T>
PlaneKernel pick_pair7(int qm) {
  switch (qm) {
    case QM_NONE: return fused_plane_pair7_kernel<T, QM_NONE>;
    case QM_FPQ: return fused_plane_pair7_kernel<T, QM_FPQ>;
    case QM_POW2: return fused_plane_pair7_kernel<T, QM_POW2>;
    case QM_MM_APPLY: return fused_plane_pair7_kernel<T, QM_MM_APPLY>;
    case QM_MM_REDUCE: return fused_plane_pair7_kernel<T, QM_MM_REDUCE>;
    case QM_FPQ_LEAN: return fused_plane_pair7_kernel<T, QM_FPQ_LEAN>;
    case QM_MM_REDUCE_STORE: return fused_plane_pair7_kernel<T, QM_MM_REDUCE_STORE>;
  }
  return nullptr;
}

template <typename T, int NRB, int NCB, int NBND>
PlaneKernel pick_s2(int qm) {
  switch (qm) {
    case QM_NONE: return fused_plane_s2_kernel<T, NRB, NCB, NBND, QM_NONE>;
    case QM_FPQ: return fused_plane_s2_kernel<T, NRB, NCB, NBND, QM_FPQ>;
    case QM_POW2: return fused_plane_s2_kernel<T, NRB, NCB, NBND, QM_POW2>;
    case QM_MM_APPLY: return fused_plane_s2_kernel<T, NRB, NCB, NBND, QM_MM_APPLY>;
    case QM_MM_REDUCE: return fused_plane_s2_kernel<T, NRB, NCB, NBND, QM_MM_REDUCE>;
    case QM_FPQ_LEAN: return fused_plane_s2_kernel<T, NRB, NCB, NBND, QM_FPQ_LEAN>;
    case QM_MM_REDUCE_STORE: return fused_plane_s2_kernel<T, NRB, NCB, NBND, QM_MM_REDUCE_STORE>;
  }
  return nullptr;
}

template <typename T>
cudaError_t launch_t(int k, int hw, int stride, int qm, const FusedArgs &a, const PlaneCfg &c,
                     cudaStream_t stream) {
  PlaneKernel kern = nullptr;
  if (a.code8) {
    kern = sizeof(T) == 4 ? pick_code8(k, hw, stride, qm) : nullptr;
  } else if (stride == 1 && k == 3) {
    if (hw == 7) kern = pick_pair7<T>(qm);
    else if (hw == 14) kern = pick_s1<T, 14, 2, 1, 1>(qm);
    else if (hw == 28) kern = pick_s1<T, 14, 4, 2, 1>(qm);
    else if (hw == 56) kern = pick_s1<T, 14, 8, 4, 1>(qm);
    else if (hw == 112) kern = pick_s1<T, 14, 4, 8, 4>(qm);
  } else if (stride == 1 && k == 5) {
    if (hw == 14) kern = pick_kxk<T, 5, 14, 2, 1, 1>(qm);
    else if (hw == 28) kern = pick_kxk<T, 5, 14, 4, 2, 1>(qm);
    else if (hw == 56) kern = pick_kxk<T, 5, 14, 8, 4, 1>(qm);
    else if (hw == 112) kern = pick_kxk<T, 5, 14, 4, 8, 4>(qm);
  } else if (stride == 2 && k == 3) {
    if (hw == 14) kern = pick_s2<T, 1, 1, 1>(qm);
    else if (hw == 28) kern = pick_s2<T, 2, 2, 1>(qm);
    else if (hw == 56) kern = pick_s2<T, 4, 4, 1>(qm);
    else if (hw == 112) kern = pick_s2<T, 4, 8, 2>(qm);
  }
  if (!kern) return cudaErrorInvalidValue;
  const size_t smem = plane_launch_smem(k, hw, stride, sizeof(T), a.code8 != 0);
  // all of the unified L1 / shared memory as shared memory: the tiles are the working set
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  return launch_pdl(kern, dim3((unsigned int)c.n_tiles), dim3(32), smem, stream, a, c);
}

}  // namespace

bool plane_has_code8(int dtype, int k, int hw, int stride, int qm) {
  return dtype == DWBNQ_F32 && pick_code8(k, hw, stride, qm) != nullptr;
}

cudaError_t launch_plane(int dtype, int k, int hw, int stride, int qm, const FusedArgs &a,
                         const PlaneCfg &c, cudaStream_t stream) {
  return dtype == DWBNQ_F32 ? launch_t<float>(k, hw, stride, qm, a, c, stream)
                            : launch_t<__half>(k, hw, stride, qm, a, c, stream);
}

}  // namespace dwbnq
