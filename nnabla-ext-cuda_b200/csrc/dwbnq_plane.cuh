// Fused dw-conv(3x3, stride 1, pad 1) -> BN -> quantizer for SMALL planes (7x7, 14x14),
// where a row is narrower than a warp's worth of 16-byte vectors and its pitch is not a
// multiple of 16 bytes, so neither the strip decomposition nor a padded TMA tile fits.
//
// One warp = one CTA = P consecutive (n, c) planes, which are contiguous in memory:
//   * lane 0 brings the whole tile in with ONE bulk async copy and, at the end, sends the
//     finished tile out with ONE bulk async store: global memory only ever sees full,
//     contiguous lines;
//   * a thread owns R = 7 full-width rows of one plane. Input rows stream through it one at
//     a time: the row is loaded from shared memory once, as pairs of horizontally adjacent
//     elements, and feeds the three output rows it touches (finishing row i-1, continuing
//     row i, starting row i+1 - which keeps every output's summation in the ky-major /
//     kx-minor order of the contract). Only two accumulator rows are live, the loop over
//     rows is rolled (two steps per trip), the code is a few KB and there is no per-element
//     halo test: the left / right zero columns are compile-time operands, the top / bottom
//     zero rows a predicated load;
//   * results overwrite the tile in place. The only rows read by one thread and written by
//     another are the neighbours' edge rows: the row below a thread's block is copied to a
//     private stash before anything is written, the row above is read in the first step,
//     and every step ends with a warp barrier.
// Arithmetic contract: the one of dwbnq_fused.cuh (bias-initialised accumulator, separately
// rounded product and sum, BN and quantizer of dwbnq_device.cuh). Halo taps enter as
// w * (+0.0); planes where that differs from skipping the tap (bias == -0.0, non-finite
// weights) are re-evaluated tap by tap by their threads after the fast pass.
#pragma once

#include "dwbnq_fused.cuh"

namespace dwbnq {

struct PlaneCfg {
  int P;        // planes per CTA = 32 / NRB
  int n_tiles;  // CTAs
  int bulk;     // x and y 16-byte aligned: the bulk copy engine may be used
};

constexpr int kPlaneRows = 7;  // rows per thread

__host__ __device__ constexpr int plane_stash_elems(int W) { return (W + 1) / 2 * 2; }
// tile | stash (NRB > 1) | mbarrier
__host__ __device__ constexpr size_t plane_smem_bytes(int W, int NRB, int elem_size) {
  size_t s = (size_t)(32 / NRB) * (kPlaneRows * NRB) * W * elem_size;
  s = (s + 15) / 16 * 16;
  if (NRB > 1) s += (size_t)32 * plane_stash_elems(W) * elem_size;
  s = (s + 15) / 16 * 16;
  return s + 16;
}

// Bulk async store shared -> global of `bytes` (multiple of 16, both sides 16-byte
// aligned); returns when the engine has read the shared-memory source.
__device__ __forceinline__ void bulk_store_1d_and_wait(void *dst, const void *src_smem,
                                                       unsigned int bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// One row of W elements at p (shared memory) as 2*NP floats, zeros beyond W and for
// !valid. Even W: pairs are 8-byte (float) / 4-byte (half) aligned and loaded whole.
template <typename T, int W>
__device__ __forceinline__ void plane_load_row(const T *p, bool valid, float *xv) {
  constexpr int NP = (W + 1) / 2;
  if (W % 2 == 0) {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      float2 t = make_float2(0.0f, 0.0f);
      if (valid) {
        if (sizeof(T) == 4) t = *reinterpret_cast<const float2 *>(p + 2 * j);
        else t = __half22float2(*reinterpret_cast<const __half2 *>(p + 2 * j));
      }
      xv[2 * j] = t.x;
      xv[2 * j + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j) xv[j] = valid ? Elem<T>::to_f32(p[j]) : 0.0f;
    xv[W] = 0.0f;
  }
}

template <typename T, int W>
__device__ __forceinline__ void plane_store_row(T *p, const float *o) {
  constexpr int NP = (W + 1) / 2;
  if (W % 2 == 0) {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      if (sizeof(T) == 4) *reinterpret_cast<float2 *>(p + 2 * j) = make_float2(o[2 * j], o[2 * j + 1]);
      else *reinterpret_cast<__half2 *>(p + 2 * j) = __floats2half2_rn(o[2 * j], o[2 * j + 1]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j) p[j] = Elem<T>::from_f32(o[j]);
  }
}

// Tap-by-tap evaluation of R full-width rows of one plane from global memory (the rare
// planes whose halo taps must be skipped rather than added as zeros). Kept out of line:
// it is cold and several times the size of the fast path.
template <typename T, int W, int QM>
__device__ __noinline__ void plane_exact_rows(const FusedArgs &a, int plane, int ch, int row0,
                                              T *rows, const MmCoef &mm, float *lo_out,
                                              float *hi_out) {
  float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
  const long long n = plane / a.OC;
#pragma unroll 1
  for (int r = 0; r < kPlaneRows; ++r) {
#pragma unroll 1
    for (int j = 0; j < W; ++j) {
      const float v = prequant_point<T>(a, n, ch, row0 + r, j);
      if (QM == QM_MM_REDUCE) {
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
      } else {
        rows[r * W + j] = Elem<T>::from_f32(quant_apply<QM>(v, a.q, mm));
      }
    }
  }
  *lo_out = lo;
  *hi_out = hi;
}

// Occupancy the kernel is compiled for: 16 one-warp CTAs per SM (128 registers).
template <typename T, int W, int NRB, int QM>
__global__ void __launch_bounds__(32, 16)
    fused_plane_kernel(const __grid_constant__ FusedArgs a, const PlaneCfg c) {
  constexpr int R = kPlaneRows;
  constexpr int H = R * NRB;
  constexpr int PE = H * W;          // elements per plane
  constexpr int NP = (W + 1) / 2;    // output pairs per row
  constexpr int P = 32 / NRB;        // planes per CTA
  constexpr int SW = plane_stash_elems(W);
  constexpr bool LEAN = QM == QM_FPQ_LEAN;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *tile = reinterpret_cast<T *>(smem_raw);
  constexpr size_t tile_bytes = ((size_t)P * PE * sizeof(T) + 15) / 16 * 16;
  T *stash = reinterpret_cast<T *>(smem_raw + tile_bytes);
  constexpr size_t stash_bytes = NRB > 1 ? ((size_t)32 * SW * sizeof(T) + 15) / 16 * 16 : 0;
  unsigned long long *bar = reinterpret_cast<unsigned long long *>(smem_raw + tile_bytes + stash_bytes);

  const int lane = threadIdx.x;
  const int n_planes = (int)(a.n * a.OC);
  const int plane0 = blockIdx.x * P;
  const int pv = min(P, n_planes - plane0);
  const T *x = static_cast<const T *>(a.x);
  T *y = static_cast<T *>(a.y);
  const unsigned int bytes = (unsigned int)(pv * PE * sizeof(T));
  const bool async_tile = c.bulk != 0 && (bytes % 16) == 0;

  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
    if (async_tile) {
      mbar_expect_tx(bar, bytes);
      bulk_load_1d(tile, x + (long long)plane0 * PE, bytes, bar);
    }
  }

  // ---- this thread's plane, rows and per-channel operands (the copy is in flight) --------
  const int pl = lane / NRB;
  const int rb = lane - pl * NRB;
  const bool active = pl < pv;
  const int plane = active ? plane0 + pl : n_planes - 1;
  const int ch = plane % a.OC;
  const f32x2 nz = negzero2();
  f32x2 w2[9];
  bool exact = false;
  {
    const T *w = static_cast<const T *>(a.w) + (long long)ch * 9;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      const float wv = Elem<T>::to_f32(w[i]);
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
  if (LEAN || a.has_bn) bnp = make_bn_packed(load_bn<T>(a, ch), nz);
  const MmCoef mm = load_mm<QM>(a, ch);

  if (!async_tile) {
    const int n = pv * PE;
    const T *src = x + (long long)plane0 * PE;
    for (int i = lane; i < n; i += 32) tile[i] = src[i];
  }
  __syncwarp();  // barrier initialisation and thread-copied data are visible
  if (async_tile && !mbar_wait_bounded(bar, 0)) {
    if (a.flag) atomicExch(a.flag, 1);
    return;
  }

  T *rows = tile + pl * PE + rb * (R * W);  // this thread's R rows, overwritten in place
  // the row below the block belongs to the next thread, which overwrites it early: keep a copy
  T *my_stash = stash + lane * SW;
  if (NRB > 1) {
    if (rb + 1 < NRB) {
      float xv[2 * NP];
      plane_load_row<T, W>(rows + R * W, true, xv);
      plane_store_row<T, W>(my_stash, xv);
    }
    __syncwarp();
  }

  float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
  f32x2 acc0[NP], acc1[NP];

  // One step = one input row k (plane row rb*R - 1 + k): finishes output row k-2 held in
  // `fin`, continues output row k-1 held in `mid`, starts output row k in `fin`.
  auto step = [&](int k, f32x2 *fin, f32x2 *mid) {
    const int gi = rb * R - 1 + k;
    const bool valid = gi >= 0 && gi < H;
    const T *src = (NRB > 1 && k == R + 1) ? my_stash : rows + (k - 1) * W;
    float xv[2 * NP];
    plane_load_row<T, W>(src, valid, xv);
    // The row above the block is the upper neighbour's last row, which it overwrites in its
    // last step; the barrier keeps every lane's first read ahead of any lane's last write.
    __syncwarp();
    // single-block planes: rows -1 and H are zero for every lane, their taps are skipped
    const bool zero_row = NRB == 1 && (k == 0 || k == R + 1);
    f32x2 E[NP], L[NP + 1];
#pragma unroll
    for (int j = 0; j < NP; ++j) E[j] = pack2(xv[2 * j], xv[2 * j + 1]);
#pragma unroll
    for (int j = 0; j <= NP; ++j)
      L[j] = pack2(j == 0 ? 0.0f : xv[2 * j - 1], j < NP ? xv[2 * j] : 0.0f);
    constexpr bool LAST_L_ZERO = (W % 2) != 0;  // odd W: L[NP] = (0, 0)

    auto taps = [&](f32x2 *acc, int ky, bool init) {
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        f32x2 v = init ? bias2 : acc[p];
        v = add2(v, mul2(w2[ky * 3 + 0], L[p], nz));
        v = add2(v, mul2(w2[ky * 3 + 1], E[p], nz));
        if (!(LAST_L_ZERO && p == NP - 1)) v = add2(v, mul2(w2[ky * 3 + 2], L[p + 1], nz));
        acc[p] = v;
      }
    };

    if (k >= 2) {
      if (!zero_row) taps(fin, 2, false);
      if (LEAN || a.has_bn) bn_apply_packed<NP>(fin, bnp);
      float o[2 * NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) unpack2(fin[p], o[2 * p], o[2 * p + 1]);
      if (QM == QM_MM_REDUCE) {
#pragma unroll
        for (int j = 0; j < W; ++j) {
          lo = fminf(lo, o[j]);
          hi = fmaxf(hi, o[j]);
        }
      } else {
        if (LEAN) {
#pragma unroll
          for (int j = 0; j < W; ++j) o[j] = fpq_apply_fast<false>(o[j], a.q);
        } else if (QM == QM_FPQ && a.q.fpq_fast) {
          if (a.q.fpq_min < 0.0f) {
#pragma unroll
            for (int j = 0; j < W; ++j) o[j] = fpq_apply_fast<true>(o[j], a.q);
          } else {
#pragma unroll
            for (int j = 0; j < W; ++j) o[j] = fpq_apply_fast<false>(o[j], a.q);
          }
        } else {
#pragma unroll
          for (int j = 0; j < W; ++j) o[j] = quant_apply<QM>(o[j], a.q, mm);
        }
        if (active) plane_store_row<T, W>(rows + (k - 2) * W, o);
      }
    }
    if (k >= 1 && k <= R) taps(mid, 1, false);
    if (k <= R - 1) {
      if (zero_row) {
#pragma unroll
        for (int p = 0; p < NP; ++p) fin[p] = bias2;
      } else {
        taps(fin, 0, true);
      }
    }
  };

#pragma unroll 1
  for (int k = 0; k < R + 2; k += 2) {
    step(k, acc0, acc1);
    if (k + 1 < R + 2) step(k + 1, acc1, acc0);
  }

  // ---- planes that need tap-skipping semantics: exact re-evaluation from global memory ----
  if (exact && active) plane_exact_rows<T, W, QM>(a, plane, ch, rb * R, rows, mm, &lo, &hi);

  if (QM == QM_MM_REDUCE) {
    if (NRB == 2) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, 1));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, 1));
    }
    if (active && (NRB != 2 || rb == 0)) {
      // NaN never enters (fminf / fmaxf drop it), matching the element-wise reduction
      atomicMin(a.q.mm_enc_min + ch, enc_ordered(lo));
      atomicMax(a.q.mm_enc_max + ch, enc_ordered(hi));
    }
    return;
  }

  // ---- the finished tile leaves in one piece ------------------------------------------------
  T *dst = y + (long long)plane0 * PE;
  if (async_tile) {
    fence_proxy_async_smem();  // this thread's shared-memory writes, for the copy engine
    __syncwarp();
    if (lane == 0) bulk_store_1d_and_wait(dst, tile, bytes);
  } else {
    __syncwarp();
    const int n = pv * PE;
    for (int i = lane; i < n; i += 32) dst[i] = tile[i];
  }
}

// Host-side entry (fused_plane.cu): launches fused_plane_kernel<T, W, H / 7, QM>.
cudaError_t launch_plane(int dtype, int w, int qm, const FusedArgs &a, const PlaneCfg &c,
                         cudaStream_t stream);
// Whether a (width, height) plane has an instantiation.
__host__ inline bool plane_shape_supported(int h, int w) {
  return (h == 7 && w == 7) || (h == 14 && w == 14);
}

}  // namespace dwbnq
