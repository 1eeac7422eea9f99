// The plane scheme of dwbnq_plane.cuh for ANY plane of even width (3x3, stride 1, pad 1):
// the geometry - plane size, blocks per tile, bands per plane - is a kernel argument instead
// of a template parameter, and the last column block / row block of a plane may be partly
// outside it. A thread owns a block of R rows x WB columns (two instantiations: 7 x 14, which
// tiles planes whose sides are multiples of 7, and 8 x 8, which tiles multiples of 8; the
// host picks the one that wastes fewer lanes) and streams its input rows through two
// accumulator rows; what changes is
//   * a per-thread valid width (pairs beyond it load zeros and are not stored: in the
//     in-place tile they belong to the next row) and valid height (rows beyond the plane
//     load zeros and are not stored: they belong to the next plane),
//   * lanes beyond the tile's blocks idle (they only take part in the warp barriers),
//   * tiles whose byte span is not a multiple of 16 are copied by the threads.
// The instantiations for the MobileNet plane sizes in dwbnq_plane.cuh are a few percent
// faster (no predicates, constant pitch); this kernel serves every other even width up to
// 14 * 32 columns. Arithmetic contract and in-place hazard discipline are the same.
#pragma once

#include "dwbnq_plane.cuh"

namespace dwbnq {

struct PlaneGenCfg {
  int H, W;     // plane size (W even)
  int wb, r;    // block width and height of the instantiation
  int ncb;      // column blocks per plane: ceil(W / wb)
  int brb;      // row blocks per tile (band): brb * ncb <= 32
  int bands;    // tiles per plane along rows; 1 = whole planes
  int gmode;    // H % r == 0: a tile is brb consecutive row blocks of the whole [planes * H, W]
                // image, across plane boundaries (planes are adjacent in memory), so no lane idles
  int P;        // planes per tile (1 when bands > 1 or gmode)
  int n_tiles;  // CTAs
  int bulk;     // x and y 16-byte aligned
};

constexpr int kGenMaxW = 16;  // widest block of any instantiation (stash sizing)

// tile (P planes x (brb * 7 + 2 halo rows when banded) rows x W) | stash | mbarrier
__host__ __device__ inline size_t plane_gen_smem_bytes(const PlaneGenCfg &g, int elem_size) {
  const int rows = (g.bands > 1 || g.gmode) ? g.brb * g.r + 2 : g.H;
  size_t s = (size_t)g.P * rows * g.W * elem_size;
  s = (s + 15) / 16 * 16;
  s += (size_t)32 * plane_stash_elems(g.wb) * elem_size;
  s = (s + 15) / 16 * 16;
  return s + 16;
}

// Pairs j < npairs of a row (8-byte / 4-byte aligned), zeros beyond and for !valid.
template <typename T, int WB>
__device__ __forceinline__ void gen_load_row(const T *p, bool valid, int npairs, float *xv) {
#pragma unroll
  for (int j = 0; j < WB / 2; ++j) {
    float2 t = make_float2(0.0f, 0.0f);
    if (valid && j < npairs) {
      if (sizeof(T) == 4) t = *reinterpret_cast<const float2 *>(p + 2 * j);
      else t = __half22float2(*reinterpret_cast<const __half2 *>(p + 2 * j));
    }
    xv[2 * j] = t.x;
    xv[2 * j + 1] = t.y;
  }
}
template <typename T, int WB>
__device__ __forceinline__ void gen_store_row(T *p, int npairs, const float *o) {
#pragma unroll
  for (int j = 0; j < WB / 2; ++j) {
    if (j < npairs) {
      if (sizeof(T) == 4) *reinterpret_cast<float2 *>(p + 2 * j) = make_float2(o[2 * j], o[2 * j + 1]);
      else *reinterpret_cast<__half2 *>(p + 2 * j) = __floats2half2_rn(o[2 * j], o[2 * j + 1]);
    }
  }
}

template <typename T, int WB, int R, int QM>
__global__ void __launch_bounds__(32, 16)
    fused_plane_gen_kernel(const __grid_constant__ FusedArgs a, const PlaneGenCfg g) {
  static_assert(WB % 2 == 0 && WB <= kGenMaxW && R % 2 == 0 || R == 7, "even block width; R + 2 steps run in pairs");
  constexpr int W = WB;
  constexpr int NP = W / 2;
  constexpr int SW = plane_stash_elems(W);
  const int PW = g.W, H = g.H;
  const int PE = H * PW;
  const bool banded = g.bands > 1 || g.gmode != 0;  // tile = a band of rows with a halo row each side
  const int TB = g.brb * R;                       // rows per band
  const int halo = banded ? 1 : 0;
  const int TE = (banded ? TB + 2 : H) * PW;      // shared-memory elements per plane of the tile
  const int tpp = g.brb * g.ncb;                  // threads per plane (band)

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *tile = reinterpret_cast<T *>(smem_raw);
  const size_t tile_bytes = ((size_t)g.P * TE * sizeof(T) + 15) / 16 * 16;
  T *stash = reinterpret_cast<T *>(smem_raw + tile_bytes);
  constexpr size_t stash_bytes = ((size_t)32 * SW * sizeof(T) + 15) / 16 * 16;
  unsigned long long *bar = reinterpret_cast<unsigned long long *>(smem_raw + tile_bytes + stash_bytes);

  const int lane = threadIdx.x;
  const int n_planes = (int)(a.n * a.OC);
  const int nrb = H / R;  // gmode: row blocks per plane
  // first / one-past-last row of the tile, of what is loaded, and of what is stored, as row
  // indices of the whole [n_planes * H, W] image
  const int plane0 = g.gmode ? 0 : (g.bands > 1 ? blockIdx.x / g.bands : blockIdx.x) * g.P;
  const int r0 = g.gmode ? 0 : (g.bands > 1 ? (blockIdx.x % g.bands) * TB : 0);  // first plane row (not gmode)
  const int pv = g.gmode ? 1 : min(g.P, n_planes - plane0);
  const long long grow0 = g.gmode ? (long long)blockIdx.x * TB : (long long)plane0 * H + r0;
  const long long glimit = g.gmode ? (long long)n_planes * H : (long long)plane0 * H + (banded ? H : pv * H);
  const long long gfloor = g.gmode ? 0 : (long long)plane0 * H;
  const long long in_first = banded ? max(grow0 - 1, gfloor) : grow0;
  const int in_rows = (int)((banded ? min(grow0 + TB + 1, glimit) : glimit) - in_first);
  const int out_rows = (int)(banded ? min((long long)TB, glimit - grow0) : glimit - grow0);
  T *y = static_cast<T *>(a.y);
  const T *in_src = static_cast<const T *>(a.x) + in_first * PW;
  T *in_dst = tile + (banded ? (int)(in_first - (grow0 - 1)) * PW : 0);
  T *dst = y + grow0 * PW;
  const unsigned int bytes = (unsigned int)((size_t)in_rows * PW * sizeof(T));
  const unsigned int obytes = (unsigned int)((size_t)out_rows * PW * sizeof(T));
  // the copy engine needs 16-byte aligned addresses and sizes on both sides
  const bool async_tile = g.bulk != 0 && (bytes % 16) == 0 && (obytes % 16) == 0 &&
                          (reinterpret_cast<uintptr_t>(in_src) % 16) == 0 &&
                          (reinterpret_cast<uintptr_t>(dst) % 16) == 0 &&
                          (((size_t)(in_dst - tile) * sizeof(T)) % 16) == 0 &&
                          (((size_t)halo * PW * sizeof(T)) % 16) == 0;

  pdl_launch_dependents();
  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  pdl_wait_for_predecessor();  // nothing global is read or written before this point
  if (lane == 0) {
    if (async_tile) {
      mbar_expect_tx(bar, bytes);
      bulk_load_1d(in_dst, in_src, bytes, bar);
    }
  }

  // ---- this thread's plane, block and per-channel operands ---------------------------------
  const int slot = lane < g.P * tpp ? lane : 0;  // idle lanes shadow block 0 and never store
  const int pl = slot / tpp;
  const int rem = slot - pl * tpp;
  const int rb = rem / g.ncb;
  const int cb = rem - rb * g.ncb;
  // the block's plane and its first row inside that plane
  const long long gb = (long long)blockIdx.x * g.brb + rb;  // gmode: row block of the whole image
  const bool in_range = lane < g.P * tpp && (g.gmode ? gb < (long long)n_planes * nrb : pl < pv);
  const int plane = !in_range ? n_planes - 1 : g.gmode ? (int)(gb / nrb) : plane0 + pl;
  const int row_first = g.gmode ? (int)(gb % nrb) * R : r0 + rb * R;
  const bool active = in_range && row_first < H;
  const int ch = plane % a.OC;
  const int vw = min(W, PW - cb * W);            // valid columns of the block (even)
  const int vp = vw / 2;                         // valid pairs
  const int vr = max(0, min(R, H - row_first));  // valid rows of the block
  const bool has_left = cb > 0;
  const bool has_right = cb + 1 < g.ncb;
  const bool has_below = rb + 1 < g.brb;         // another block of this tile below
  const f32x2 nz = negzero2();
  f32x2 w2[9];
  bool exact = false;
  {
    const T *w = static_cast<const T *>(a.w) + (long long)ch * 9;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      const float wv = Elem<T>::to_f32(w[tap_index(a, i, 9)]);
      exact = exact || !(fabsf(wv) <= 3.402823466e38f);
      w2[i] = splat2(wv);
      pin(w2[i]);
    }
  }
  const float bv = a.b ? Elem<T>::to_f32(static_cast<const T *>(a.b)[ch]) : 0.0f;
  exact = exact || __float_as_uint(bv) == 0x80000000u;
  f32x2 bias2 = splat2(bv);
  pin(bias2);
  BnPacked bnp;
  if (QM == QM_FPQ_LEAN || a.has_bn) bnp = make_bn_packed(load_bn<T>(a, ch), nz);
  const MmCoef mm = load_mm<QM>(a, ch);

  if (!async_tile) {
    const int n = in_rows * PW;
    for (int i = lane; i < n; i += 32) in_dst[i] = in_src[i];
  }
  __syncwarp();
  if (async_tile && !mbar_wait_bounded(bar, 0)) {
    if (a.flag) atomicExch(a.flag, 1);
    return;
  }

  T *rows = tile + pl * TE + (halo + rb * R) * PW + cb * W;
  T *my_stash = stash + lane * SW + 2;
  // the row below the block, when another block of the tile owns (and will overwrite) it
  if (has_below) {
    const T *below = rows + R * PW;
    const bool bvalid = row_first + R < H;
    float xv[2 * NP];
    gen_load_row<T, W>(below, bvalid, vp, xv);
    gen_store_row<T, W>(my_stash, NP, xv);
    my_stash[-1] = (bvalid && has_left) ? below[-1] : Elem<T>::from_f32(0.0f);
    my_stash[W] = (bvalid && has_right) ? below[W] : Elem<T>::from_f32(0.0f);
  }
  __syncwarp();

  float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
  f32x2 acc0[NP], acc1[NP];

  auto step = [&](int k, f32x2 *fin, f32x2 *mid) {
    const int gi = row_first - 1 + k;
    const bool valid = gi >= 0 && gi < H;
    const bool from_stash = k == R + 1 && has_below;
    const T *src = from_stash ? my_stash : rows + (k - 1) * PW;
    float xv[2 * NP];
    gen_load_row<T, W>(src, valid, from_stash ? NP : vp, xv);
    float xl = 0.0f, xr = 0.0f;
    if (valid && has_left) xl = Elem<T>::to_f32(src[-1]);
    if (valid && has_right) xr = Elem<T>::to_f32(src[W]);
    __syncwarp();  // reads of this step before any write of this step (see dwbnq_plane.cuh)
    f32x2 E[NP], L[NP + 1];
#pragma unroll
    for (int j = 0; j < NP; ++j) E[j] = pack2(xv[2 * j], xv[2 * j + 1]);
#pragma unroll
    for (int j = 0; j <= NP; ++j) L[j] = pack2(j == 0 ? xl : xv[2 * j - 1], j < NP ? xv[2 * j] : xr);

    auto taps = [&](f32x2 *acc, int ky, bool init) {
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        f32x2 v = init ? bias2 : acc[p];
        v = tap_add2<T>(v, w2[ky * 3 + 0], L[p], nz);
        v = tap_add2<T>(v, w2[ky * 3 + 1], E[p], nz);
        v = tap_add2<T>(v, w2[ky * 3 + 2], L[p + 1], nz);
        acc[p] = v;
      }
    };

    if (k >= 2) {
      taps(fin, 2, false);
      if (QM == QM_FPQ_LEAN || a.has_bn) bn_apply_packed<NP>(fin, bnp);
      float o[2 * NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) unpack2(fin[p], o[2 * p], o[2 * p + 1]);
      const bool row_ok = active && k - 2 < vr;
      if (qm_reduces(QM)) {
#pragma unroll
        for (int j = 0; j < W; ++j) {
          if (row_ok && j < vw) {
            lo = fminf(lo, o[j]);
            hi = fmaxf(hi, o[j]);
          }
        }
      }
      if (qm_stores(QM)) {
        plane_quant<QM, W>(o, a.q, mm);
        if (row_ok) gen_store_row<T, W>(rows + (k - 2) * PW, vp, o);
      }
    }
    if (k >= 1 && k <= R) taps(mid, 1, false);
    if (k <= R - 1) taps(fin, 0, true);
  };

#pragma unroll 1
  for (int k = 0; k < R + 2; k += 2) {
    step(k, acc0, acc1);
    if (k + 1 < R + 2) step(k + 1, acc1, acc0);
  }

  if (exact && active)
    plane_exact_block<T, QM>(a, plane, ch, row_first, cb * W, vr, vw, rows, PW, mm, &lo, &hi);

  if (qm_reduces(QM) && active) {
    // NaN never enters (fminf / fmaxf drop it), matching the element-wise reduction
    atomicMin(a.q.mm_enc_min + ch, enc_ordered(lo));
    atomicMax(a.q.mm_enc_max + ch, enc_ordered(hi));
  }
  if (!qm_stores(QM)) return;

  const T *out_src = tile + halo * PW;
  if (async_tile) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) bulk_store_1d_and_wait(dst, out_src, obytes);
  } else {
    __syncwarp();
    const int n = out_rows * PW;
    for (int i = lane; i < n; i += 32) dst[i] = out_src[i];
  }
}

// Host side (fused_plane_gen.cu): geometry for a plane, 0 CTAs when the kernel does not apply.
// (chooses between the instantiations; `util` receives the fraction of lane-work that lands
// on real outputs)
PlaneGenCfg plane_gen_geometry(int h, int w, long long n_planes, int elem_size, bool aligned, float *util);
cudaError_t launch_plane_gen(int dtype, int qm, const FusedArgs &a, const PlaneGenCfg &g, cudaStream_t stream);

}  // namespace dwbnq
