// Geometry, instantiations and dispatch of the general-geometry plane kernel.
#include <cstdlib>

#include "dwbnq_internal.h"
#include "dwbnq_plane_gen.cuh"

namespace dwbnq {

namespace {

// Geometry for one block shape; n_tiles == 0 when it does not apply.
PlaneGenCfg geometry_for(int wb, int r, int h, int w, long long n_planes, bool aligned, float *util) {
  PlaneGenCfg g;
  g.H = h;
  g.W = w;
  g.wb = wb;
  g.r = r;
  g.ncb = g.brb = g.bands = g.gmode = g.P = g.n_tiles = g.bulk = 0;
  *util = 0.0f;
  if (h < 1 || w < 2 || (w % 2) != 0 || w > wb * 32 || n_planes < 1) return g;
  g.ncb = (w + wb - 1) / wb;
  const int nrb_total = (h + r - 1) / r;
  int brb = 32 / g.ncb;
  if (h % r == 0 && n_planes * (long long)nrb_total < 0x7fffffffLL) {
    // row blocks line up across planes: bands of the whole image, every tile full
    const long long blocks = n_planes * (long long)nrb_total;
    if (brb > blocks) brb = (int)blocks;
    g.gmode = 1;
    g.brb = brb;
    g.bands = 1;
    g.P = 1;
    g.n_tiles = (int)((blocks + brb - 1) / brb);
    g.bulk = aligned ? 1 : 0;
    *util = (float)((double)w / ((double)g.ncb * wb) * (double)(g.brb * g.ncb) / 32.0);
    return g;
  }
  if (brb > nrb_total) brb = nrb_total;
  g.bands = (nrb_total + brb - 1) / brb;
  g.brb = (nrb_total + g.bands - 1) / g.bands;  // even out the bands
  g.P = g.bands == 1 ? 32 / (g.brb * g.ncb) : 1;
  if (g.P < 1) g.P = 1;
  const long long tiles = g.bands == 1 ? (n_planes + g.P - 1) / g.P : n_planes * g.bands;
  if (tiles > 0x7fffffffLL) return g;
  g.n_tiles = (int)tiles;
  g.bulk = aligned ? 1 : 0;
  // real outputs per tile-set of a plane / outputs the 32 lanes of its tiles could produce
  *util = (float)((double)h * w * g.P / ((double)g.bands * 32.0 * r * wb));
  return g;
}

}  // namespace

PlaneGenCfg plane_gen_geometry(int h, int w, long long n_planes, int elem_size, bool aligned, float *util) {
  (void)elem_size;
  float u14 = 0.0f, u8 = 0.0f;
  const PlaneGenCfg g14 = geometry_for(14, 7, h, w, n_planes, aligned, &u14);
  const PlaneGenCfg g8 = geometry_for(8, 8, h, w, n_planes, aligned, &u8);
  const bool take8 = g8.n_tiles > 0 && (g14.n_tiles == 0 || u8 > u14);
  if (util) *util = take8 ? u8 : u14;
  return take8 ? g8 : g14;
}

namespace {

typedef void (*GenKernel)(const FusedArgs, const PlaneGenCfg);

template <typename T, int WB, int R>
GenKernel pick(int qm) {
  switch (qm) {
    case QM_NONE: return fused_plane_gen_kernel<T, WB, R, QM_NONE>;
    case QM_FPQ: return fused_plane_gen_kernel<T, WB, R, QM_FPQ>;
    case QM_POW2: return fused_plane_gen_kernel<T, WB, R, QM_POW2>;
    case QM_MM_APPLY: return fused_plane_gen_kernel<T, WB, R, QM_MM_APPLY>;
    case QM_MM_REDUCE: return fused_plane_gen_kernel<T, WB, R, QM_MM_REDUCE>;
    case QM_FPQ_LEAN: return fused_plane_gen_kernel<T, WB, R, QM_FPQ_LEAN>;
    case QM_MM_REDUCE_STORE: return fused_plane_gen_kernel<T, WB, R, QM_MM_REDUCE_STORE>;
  }
  return nullptr;
}
template <typename T>
GenKernel pick_shape(int wb, int r, int qm) {
  if (wb == 14 && r == 7) return pick<T, 14, 7>(qm);
  if (wb == 8 && r == 8) return pick<T, 8, 8>(qm);
  return nullptr;
}

}  // namespace

cudaError_t launch_plane_gen(int dtype, int qm, const FusedArgs &a, const PlaneGenCfg &g, cudaStream_t stream) {
  GenKernel kern = dtype == DWBNQ_F32 ? pick_shape<float>(g.wb, g.r, qm) : pick_shape<__half>(g.wb, g.r, qm);
  if (!kern || g.n_tiles < 1) return cudaErrorInvalidValue;
  const size_t smem = plane_gen_smem_bytes(g, dtype == DWBNQ_F32 ? 4 : 2);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                       cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return e;
  return launch_pdl(kern, dim3((unsigned int)g.n_tiles), dim3(32), smem, stream, a, g);
}

}  // namespace dwbnq
