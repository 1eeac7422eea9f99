// Fused DepthwiseConvolution -> BatchNormalization(inference) -> quantizer kernels.
//
// The kernel families of the library share one arithmetic core. The plane kernels of
// dwbnq_plane.cuh / dwbnq_plane_gen.cuh serve 3x3 (stride 1 and 2) and 5x5 (stride 1) on the
// plane sizes they tile; this header holds the two families behind them:
//  * fused_generic_kernel: one thread per output element, taps read straight from global
//    memory, out-of-bounds taps skipped. Handles every geometry the reference accepts
//    (any kernel size, stride, pad, dilation, multiplier, 1-D) and is also the in-kernel
//    fall-back of the tiled family for the parameter values where "skip the tap" and
//    "add w * 0" differ (bias == -0.0, non-finite weights).
//  * fused_tiled_kernel: a CTA owns one tile of `P` (n, c) planes x a band of output rows.
//    The input of the tile is staged in shared memory by the copy engines - one TMA tiled
//    box load per plane (halo rows / columns arrive as zeros), or, where the row pitch is
//    not a multiple of 16 bytes (odd widths), one bulk async copy of the contiguous
//    planes with the halo masked when the window is read - while the threads build the
//    per-plane parameter records; several resident CTAs per SM overlap one tile's
//    arithmetic with the next tile's copy. Each thread computes R x VEC output patches
//    from a rolling register window on packed f32x2 pairs, applies BN and the quantizer in
//    registers and stores 16-byte vectors.
//
// Arithmetic contract (identical in every family): accumulator starts at the bias, taps in
// ky-major / kx-minor order, product and sum rounded separately (never contracted; for
// binary16 inputs the product is exact in fp32, so a fused multiply-add is the same
// operation), then the BN and quantizer steps of dwbnq_device.cuh.
#pragma once

#include <cuda.h>

#include "dwbnq_device.cuh"

namespace dwbnq {

struct FusedArgs {
  const void *x, *w, *b;                  // input, weights [OC,kh,kw], bias [OC] or null
  const void *beta, *gamma, *mean, *var;  // BN vectors [OC]; beta/gamma may be null
  void *y;
  float eps;
  int has_bn;
  long long n;  // batch
  int C, H, W, OC, Ho, Wo;
  int kh, kw, sh, sw, ph, pw, dh, dw, mult;
  QuantArgs q;
  int *flag;  // device word set when a bounded wait runs out
  // 8-bit storage (dwbnq_fused_fwd_code8): x and y hold FixedPointQuantize codes, one byte
  // per element, instead of T values. x = code * code_in_delta (int8 codes when
  // code_in_signed); y's code is the quantized value / q.fpq_delta (int8 when q.fpq_min < 0).
  // Weights, bias and the BN vectors stay T. 0 = off.
  int code8;
  int code_in_signed;
  float code_in_delta;
  // The taps are read back to front, w[kh*kw - 1 - i] for tap i: the convolution with the
  // kernel rotated by 180 degrees, which is the input gradient of a stride-1 convolution.
  int w_flip;
};

// Index of tap i of kk in the weight array.
__device__ __forceinline__ int tap_index(const FusedArgs &a, int i, int kk) { return a.w_flip ? kk - 1 - i : i; }

// One input element as fp32: a T value, or (8-bit storage) a code times its step.
template <typename T>
__device__ __forceinline__ float load_x(const FusedArgs &a, const void *base, long long idx) {
  if (a.code8) {
    const int c = a.code_in_signed ? (int)static_cast<const signed char *>(base)[idx]
                                   : (int)static_cast<const unsigned char *>(base)[idx];
    return __fmul_rn((float)c, a.code_in_delta);  // exact: a code has 8 bits
  }
  return Elem<T>::to_f32(static_cast<const T *>(base)[idx]);
}
// The code of a FixedPointQuantize output v = k * delta (delta a power of two: exact).
__device__ __forceinline__ int fpq_code(float v, const QuantArgs &q) {
  return __float2int_rn(__fmul_rn(v, q.fpq_inv_delta));
}

// Where the input tile of the tiled family comes from and how it is laid out.
enum TileMode : int {
  TM_TMA = 0,   // zero-padded tile, one TMA tiled box load per plane (async)
  TM_COOP = 1,  // zero-padded tile filled by cooperative loads (any alignment, synchronous)
  TM_RAW = 2    // whole planes copied verbatim by one bulk async copy; halo masked at load
};

// Geometry of the tiled family, fixed by the host planner.
struct TileCfg {
  int P;            // planes per tile
  int TH;           // output rows per tile (multiple of R)
  int n_row_tiles;  // ceil(Ho / TH); 1 in TM_RAW
  int n_strips;     // ceil(Wo / VEC)
  int n_rb;         // row blocks (items along y) per tile: TH / R
  int R;            // output rows per item
  int WS;           // padded modes: shared-memory row pitch in elements (multiple of VEC)
  int TR;           // input rows a tile needs: (TH - 1) * stride + K
  int box_rows;     // rows per TMA box (<= 256)
  int n_boxes;      // boxes per plane; a padded plane tile holds n_boxes * box_rows rows
  int tile_elems;   // elements per plane inside a stage (padded: multiple of 128 B; raw: H*W)
  int stage_elems;  // elements per stage buffer (multiple of 128 B), slack included
  int raw_lead;     // TM_RAW: slack elements in front of the first plane of a stage
  int vec_store;    // Wo % VEC == 0 and y 16-byte aligned
  int vec_fill;     // TM_COOP: 16-byte global loads allowed; TM_RAW: bulk copy allowed
  int n_tiles;
};

// ---- exact single-output evaluation (generic family and fall-back) -------------------

template <typename T>
__device__ __forceinline__ float conv_point(const FusedArgs &a, long long n, int oc, int oy,
                                            int ox) {
  const T *w = static_cast<const T *>(a.w);
  const T *b = static_cast<const T *>(a.b);
  const int ic = oc / a.mult;
  const long long xbase = (n * a.C + ic) * (long long)a.H * a.W;
  const T *wp = w + (long long)oc * a.kh * a.kw;
  float acc = b ? Elem<T>::to_f32(b[oc]) : 0.0f;
  for (int ky = 0; ky < a.kh; ++ky) {
    const int iy = oy * a.sh + ky * a.dh - a.ph;
    for (int kx = 0; kx < a.kw; ++kx) {
      const int ix = ox * a.sw + kx * a.dw - a.pw;
      if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W) {
        if (!DWBNQ_IN_BOUNDS(xbase + (long long)iy * a.W + ix, a.n * a.C * (long long)a.H * a.W, a.flag) ||
            !DWBNQ_IN_BOUNDS((long long)oc * a.kh * a.kw + tap_index(a, ky * a.kw + kx, a.kh * a.kw),
                             (long long)a.OC * a.kh * a.kw, a.flag))
          continue;
        const float xv = load_x<T>(a, a.x, xbase + (long long)iy * a.W + ix);
        const float wv = Elem<T>::to_f32(wp[tap_index(a, ky * a.kw + kx, a.kh * a.kw)]);
        acc = __fadd_rn(acc, __fmul_rn(wv, xv));
      }
    }
  }
  return acc;
}

template <typename T>
__device__ __forceinline__ BnCoef load_bn(const FusedArgs &a, int oc) {
  BnCoef c;
  c.mean = Elem<T>::to_f32(static_cast<const T *>(a.mean)[oc]);
  c.scale = a.gamma ? Elem<T>::to_f32(static_cast<const T *>(a.gamma)[oc]) : 1.0f;
  c.stdvar = bn_stdvar(Elem<T>::to_f32(static_cast<const T *>(a.var)[oc]), a.eps);
  c.beta = a.beta ? Elem<T>::to_f32(static_cast<const T *>(a.beta)[oc]) : 0.0f;
  return c;
}

// Pre-quantizer value of one output (conv, then BN when present).
template <typename T>
__device__ __forceinline__ float prequant_point(const FusedArgs &a, long long n, int oc, int oy,
                                                int ox) {
  float v = conv_point<T>(a, n, oc, oy, ox);
  if (a.has_bn) v = bn_apply(v, load_bn<T>(a, oc));
  return v;
}

template <int QM>
__device__ __forceinline__ MmCoef load_mm(const FusedArgs &a, int oc) {
  MmCoef m{1.0f, 0.0f, 0.0f};
  if (QM == QM_MM_APPLY) {
    m.scale = a.q.mm_scale[oc];
    m.lo = a.q.mm_lo[oc];
    m.hi = a.q.mm_hi[oc];
  }
  return m;
}

// Warp-cooperative min/max into the encoded per-channel slots: when the whole warp works
// on one channel (the common case) one lane issues the two atomics.
__device__ __forceinline__ void reduce_minmax_to_global(const QuantArgs &q, int oc, float v,
                                                        bool valid) {
  const unsigned int mask = __activemask();
  const int oc0 = __shfl_sync(mask, oc, __ffs(mask) - 1);
  const bool uniform = __all_sync(mask, oc == oc0);
  float lo = (valid && v == v) ? v : __uint_as_float(0x7f800000u);
  float hi = (valid && v == v) ? v : __uint_as_float(0xff800000u);
  if (uniform && mask == 0xffffffffu) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if ((threadIdx.x & 31) == 0) {
      atomicMin(q.mm_enc_min + oc, enc_ordered(lo));
      atomicMax(q.mm_enc_max + oc, enc_ordered(hi));
    }
  } else if (valid) {
    atomicMin(q.mm_enc_min + oc, enc_ordered(lo));
    atomicMax(q.mm_enc_max + oc, enc_ordered(hi));
  }
}

template <typename T, int QM>
__global__ void __launch_bounds__(256) fused_generic_kernel(const FusedArgs a,
                                                            const long long total) {
  T *y = static_cast<T *>(a.y);
  const long long step = (long long)gridDim.x * blockDim.x;
  // Whole warps iterate together (the bound is rounded up to a warp) so the shuffles in
  // the reduce mode always see a full warp.
  const long long total_w = (total + 31) / 32 * 32;
  for (long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x; o < total_w; o += step) {
    const bool valid = o < total;
    const long long oo = valid ? o : total - 1;
    const int ox = (int)(oo % a.Wo);
    long long t = oo / a.Wo;
    const int oy = (int)(t % a.Ho);
    t /= a.Ho;
    const int oc = (int)(t % a.OC);
    const long long n = t / a.OC;
    const float v = prequant_point<T>(a, n, oc, oy, ox);
    if (QM == QM_MM_REDUCE) {
      reduce_minmax_to_global(a.q, oc, v, valid);
    } else if (valid && DWBNQ_IN_BOUNDS(o, total, a.flag)) {
      const float r = quant_apply<QM>(v, a.q, load_mm<QM>(a, oc));
      if ((QM == QM_FPQ || QM == QM_FPQ_LEAN) && a.code8) static_cast<signed char *>(a.y)[o] = (signed char)fpq_code(r, a.q);
      else y[o] = Elem<T>::from_f32(r);
    }
  }
}

// ---- TMA / mbarrier wrappers (sm_100a PTX) ---------------------------------------------

__device__ __forceinline__ unsigned int smem_u32(const void *p) {
  return (unsigned int)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long *bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
               : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// One poll of the barrier phase. The suspend-time hint lets the hardware park the thread
// until the phase completes (or ~0.1 ms pass) instead of burning issue slots in a spin.
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned int parity) {
  unsigned int ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(100000u)
      : "memory");
  return ok != 0;
}
// Bounded wait. The limit is a TIME (2 s of the global nanosecond timer by default): a poll
// count alone would depend on how long the hardware parks a poll, and a healthy copy on a
// busy GPU must not be mistaken for a lost one. A poll cap (2^24, far beyond the time limit)
// backs the timer up. When the limit passes the caller records it in the device flag and
// returns, so a transfer that never lands cannot hang the GPU.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded_lane(unsigned long long *bar, unsigned int parity,
                                                       unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
#pragma unroll 1
  for (unsigned int i = 0; i < (1u << 24); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) break;
  }
  return false;
}
// Warp-uniform form (all 32 lanes call it): either every lane has observed the phase, or
// every lane gives up. A lane that ran out of time while another saw the phase complete
// polls once more (the phase stays complete), which also gives it the acquire it needs.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long *bar, unsigned int parity,
                                                  unsigned long long limit_ns = kWaitLimitNs) {
  bool ok = mbar_wait_bounded_lane(bar, parity, limit_ns);
  if (!__all_sync(0xffffffffu, ok)) {
    if (__any_sync(0xffffffffu, ok) && !ok) ok = mbar_try_wait(bar, parity);
    ok = __all_sync(0xffffffffu, ok);
  }
  return ok;
}
// CTA-uniform form (every thread of the block calls it): a block whose threads meet at
// barriers afterwards must leave as a whole.
__device__ __forceinline__ bool mbar_wait_bounded_cta(unsigned long long *bar, unsigned int parity,
                                                      unsigned long long limit_ns = kWaitLimitNs) {
  bool ok = mbar_wait_bounded_lane(bar, parity, limit_ns);
  if (__syncthreads_and(ok)) return true;
  if (!ok) ok = mbar_try_wait(bar, parity);  // completed meanwhile for a slower thread
  return __syncthreads_and(ok) != 0;
}
// One tiled 3-D box load {x, y, z} -> shared memory, completion counted on `bar`.
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *tm, int x, int y, int z,
                                            unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// ---- register window loader ----------------------------------------------------------
// Fills v[0..NV) with the NV consecutive elements that start L elements before `base`.
// `base` is 16-byte aligned (shared memory); the window is assembled from the widest
// aligned pieces: a single / pair on the left, 16-byte vectors, then a pair / single.
template <typename T> struct Pair;
template <> struct Pair<float> {
  static __device__ __forceinline__ void load(const float *p, float *v) {
    const float2 t = *reinterpret_cast<const float2 *>(p);
    v[0] = t.x; v[1] = t.y;
  }
};
template <> struct Pair<__half> {
  static __device__ __forceinline__ void load(const __half *p, float *v) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(p));
    v[0] = t.x; v[1] = t.y;
  }
};

template <typename T, int L, int NV>
__device__ __forceinline__ void load_window(const T *base, float *v) {
  constexpr int S = Elem<T>::VEC;
  static_assert(L >= 0 && L <= 2, "left halo of 0..2 elements");
  if (L == 1) v[0] = Elem<T>::to_f32(base[-1]);
  if (L == 2) Pair<T>::load(base - 2, v);
  constexpr int NRIGHT = NV - L;
  constexpr int NFULL = NRIGHT / S;
  constexpr int REM = NRIGHT % S;
#pragma unroll
  for (int i = 0; i < NFULL; ++i) Vec16<T>::load(base + i * S, v + L + i * S);
  constexpr int NPAIR = REM / 2;
#pragma unroll
  for (int i = 0; i < NPAIR; ++i) Pair<T>::load(base + NFULL * S + 2 * i, v + L + NFULL * S + 2 * i);
  if (REM % 2) v[NV - 1] = Elem<T>::to_f32(base[NRIGHT - 1]);
}


// Compile-time counted loop: f(IntC<0>{}), ..., f(IntC<N-1>{}).
template <int V> struct IntC { static constexpr int value = V; };
template <int N, int I = 0, typename F>
__device__ __forceinline__ void static_loop(F &&f) {
  if constexpr (I < N) {
    f(IntC<I>{});
    static_loop<N, I + 1>(f);
  }
}

// ---- the tiled kernel ----------------------------------------------------------------

// Per-plane parameter record in shared memory, built once per CTA by one thread per plane
// and laid out so the consumer fetches packed operands with 8/16-byte loads and no register
// shuffling:
//   [0, 2*KK)  weight pairs (w, w)
//   PAIRS + 0  (bias, bias)      + 2 (-mean, -mean)     + 4 (scale, scale)
//         + 6  (rcp, rcp)        + 8 (-stdvar, -stdvar) + 10 (beta, beta)
//   SCAL  + 0  stdvar  1 guard_lo  2 mm_scale  3 mm_lo  4 mm_hi  5 exact-evaluation flag
template <int K> struct ParamLayout {
  static constexpr int KK = K * K;
  static constexpr int PAIRS = 2 * KK + (2 * KK) % 4;  // 16-byte aligned
  static constexpr int SCAL = PAIRS + 12;
  static constexpr int COUNT = SCAL + 8;
};

// Shared-memory carve-up, also used by the host planner to size the launch.
__host__ __device__ inline size_t tiled_smem_bytes(int P, int stage_elems, int elem_size, int K) {
  const int kk2 = 2 * K * K;
  const int count = kk2 + kk2 % 4 + 20;
  size_t s = (size_t)stage_elems * elem_size;       // the tile (128 B multiple)
  s += (size_t)P * count * sizeof(float);           // parameter records
  s += (size_t)P * 2 * sizeof(unsigned int);        // per-plane encoded min / max
  s = (s + 15) / 16 * 16;
  s += 16;                                          // mbarrier
  return s;
}

// One bulk async copy global -> shared (16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(void *dst, const void *src, unsigned int bytes,
                                             unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Window of NV elements starting at p (any alignment), halo positions forced to +0.0 by
// per-position bit masks.
template <typename T, int NV>
__device__ __forceinline__ void load_window_raw(const T *p, const unsigned int *mask, float *v) {
#pragma unroll
  for (int i = 0; i < NV; ++i)
    v[i] = __uint_as_float(__float_as_uint(Elem<T>::to_f32(p[i])) & mask[i]);
}

// Resident CTAs per SM the kernel is compiled for: the 3x3 float kernels fit 64 registers
// (4 x 256 threads), the wider windows of the other instantiations get twice as many.
__host__ __device__ constexpr int tiled_min_blocks(int elem_size, int K, int mode) {
  return (elem_size == 4 && K == 3 && mode != TM_RAW) ? 3 : 2;
}

// One CTA = one tile: P planes x R*n_rb output rows. The tile copy (TMA / bulk) is issued
// first and flies while the per-plane parameter records are built; several CTAs per SM give
// the overlap between one tile's arithmetic and the next tile's copy.
template <typename T, int K, int STRIDE, int R, int QM, int MODE>
__global__ void __launch_bounds__(256, tiled_min_blocks(sizeof(T), K, MODE))
    fused_tiled_kernel(const __grid_constant__ CUtensorMap tmap, const FusedArgs a,
                       const TileCfg c) {
  constexpr int S = Elem<T>::VEC;  // outputs per thread and patch row = one 16-byte vector
  constexpr int PAD = K / 2;
  constexpr int NV = (S - 1) * STRIDE + K;  // window elements per row
  constexpr bool ASYNC = MODE != TM_COOP;
  using PL = ParamLayout<K>;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *tiles = reinterpret_cast<T *>(smem_raw);
  float *prm = reinterpret_cast<float *>(smem_raw + (size_t)c.stage_elems * sizeof(T));
  unsigned int *red = reinterpret_cast<unsigned int *>(prm + c.P * PL::COUNT);
  unsigned long long *bar = reinterpret_cast<unsigned long long *>(
      (reinterpret_cast<uintptr_t>(red + 2 * c.P) + 15) / 16 * 16);

  const int tid = (threadIdx.z * blockDim.y + threadIdx.y) * blockDim.x + threadIdx.x;
  const int nthr = blockDim.x * blockDim.y * blockDim.z;
  const int n_planes = (int)(a.n * a.OC);  // multiplier == 1; the planner keeps it below 2^31
  const T *x = static_cast<const T *>(a.x);
  T *y = static_cast<T *>(a.y);
  const int plane_elems = a.H * a.W;

  // this CTA's tile
  const int grp = blockIdx.x / c.n_row_tiles;
  const int plane0 = grp * c.P;
  const int pv = min(c.P, n_planes - plane0);
  const int oy0 = (blockIdx.x - grp * c.n_row_tiles) * c.TH;
  // TM_RAW: a tile whose byte span is not a multiple of 16 (the ragged last group, or an
  // unaligned tensor) is copied by the threads instead of by the bulk engine.
  const bool async_tile = MODE == TM_TMA || (MODE == TM_RAW && c.vec_fill != 0 &&
                                            ((pv * plane_elems * (int)sizeof(T)) % 16) == 0);

  if (ASYNC && tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
    if (async_tile) {
      if (MODE == TM_TMA) {
        const int rows_alloc = c.box_rows * c.n_boxes;
        mbar_expect_tx(bar, (unsigned int)((size_t)pv * rows_alloc * c.WS * sizeof(T)));
        const int iy0 = oy0 * STRIDE - PAD;
        for (int pl = 0; pl < pv; ++pl)
          for (int bx = 0; bx < c.n_boxes; ++bx)
            tma_load_3d(tiles + (size_t)pl * c.tile_elems + (size_t)bx * c.box_rows * c.WS, &tmap, -S,
                        iy0 + bx * c.box_rows, plane0 + pl, bar);
      } else {
        const unsigned int bytes = (unsigned int)(pv * plane_elems * sizeof(T));
        mbar_expect_tx(bar, bytes);
        bulk_load_1d(tiles + c.raw_lead, x + (long long)plane0 * plane_elems, bytes, bar);
      }
    }
  }

  // ---- per-plane parameter records: one thread per plane (the copy above is in flight) -----
  for (int pl = tid; pl < pv; pl += nthr) {
    const T *w = static_cast<const T *>(a.w);
    const int ch = (plane0 + pl) % a.OC;
    float *rec = prm + pl * PL::COUNT;
    // The tile treats out-of-bounds taps as w * (+0.0) added to the accumulator, the
    // contract is "skip the tap". They differ only when w * 0 is not +-0 (non-finite
    // weight) or when the accumulator can be -0.0 (bias == -0.0): flag the plane for exact
    // evaluation.
    bool exact = false;
#pragma unroll
    for (int i = 0; i < PL::KK; ++i) {
      const float wv = Elem<T>::to_f32(w[ch * PL::KK + tap_index(a, i, PL::KK)]);
      rec[2 * i] = wv;
      rec[2 * i + 1] = wv;
      exact = exact || !(fabsf(wv) <= 3.402823466e38f);
    }
    const float bv = a.b ? Elem<T>::to_f32(static_cast<const T *>(a.b)[ch]) : 0.0f;
    exact = exact || __float_as_uint(bv) == 0x80000000u;
    rec[PL::PAIRS] = rec[PL::PAIRS + 1] = bv;
    if (a.has_bn) {
      const BnCoef bc = load_bn<T>(a, ch);
      const float rcp = __frcp_rn(bc.stdvar);
      const bool safe = bc.stdvar >= 9.31322574615478515625e-10f && bc.stdvar <= 1073741824.0f;
      float *pr = rec + PL::PAIRS + 2;
      pr[0] = pr[1] = -bc.mean;
      pr[2] = pr[3] = bc.scale;
      pr[4] = pr[5] = rcp;
      pr[6] = pr[7] = -bc.stdvar;
      pr[8] = pr[9] = bc.beta;
      rec[PL::SCAL] = bc.stdvar;
      rec[PL::SCAL + 1] = safe ? DWBNQ_DIV_GUARD_LO : __uint_as_float(0x7f800000u);
    }
    if (QM == QM_MM_APPLY) {
      rec[PL::SCAL + 2] = a.q.mm_scale[ch];
      rec[PL::SCAL + 3] = a.q.mm_lo[ch];
      rec[PL::SCAL + 4] = a.q.mm_hi[ch];
    }
    rec[PL::SCAL + 5] = exact ? 1.0f : 0.0f;
    if (QM == QM_MM_REDUCE) {
      red[2 * pl] = DWBNQ_ENC_POS_INF;
      red[2 * pl + 1] = DWBNQ_ENC_NEG_INF;
    }
  }

  // ---- tiles the copy engines do not take -----------------------------------------------
  if (MODE == TM_COOP) {
    // every 16-byte group of the zero-padded tile is produced by one thread
    const int iy0 = oy0 * STRIDE - PAD;
    const int gpr = c.WS / S;
    const int n_groups = pv * c.TR * gpr;
    for (int g = tid; g < n_groups; g += nthr) {
      const int pl = g / (c.TR * gpr);
      const int rem = g - pl * (c.TR * gpr);
      const int tr = rem / gpr;
      const int gc = rem - tr * gpr;
      const int iy = iy0 + tr;
      const int ix0 = gc * S - S;
      float v[S];
#pragma unroll
      for (int j = 0; j < S; ++j) v[j] = 0.0f;
      if (iy >= 0 && iy < a.H && ix0 + S > 0 && ix0 < a.W) {
        const T *src = x + ((long long)(plane0 + pl) * a.H + iy) * a.W + ix0;
        if (c.vec_fill && ix0 >= 0 && ix0 + S <= a.W) {
          Vec16<T>::load_stream(src, v);
        } else {
#pragma unroll
          for (int j = 0; j < S; ++j)
            if (ix0 + j >= 0 && ix0 + j < a.W) v[j] = Elem<T>::to_f32(src[j]);
        }
      }
      Vec16<T>::store(tiles + (size_t)pl * c.tile_elems + (size_t)tr * c.WS + gc * S, v);
    }
  } else if (MODE == TM_RAW && !async_tile) {
    const int n = pv * plane_elems;
    T *dst = tiles + c.raw_lead;
    const T *src = x + (long long)plane0 * plane_elems;
    for (int i = tid; i < n; i += nthr) dst[i] = src[i];
  }
  __syncthreads();  // records, thread-copied data and the barrier initialisation are visible

  // Every lane waits itself with the hardware parking it (a one-lane poll would leave its
  // warp split in two for the rest of the kernel).
  if (ASYNC && async_tile && !mbar_wait_bounded_cta(bar, 0)) {  // async_tile is CTA-uniform
    if (a.flag) atomicExch(a.flag, 1);
    return;
  }

  // ---- consumer ---------------------------------------------------------------------------
  // R x S output patches from a rolling K-row register window, fully unrolled. Arithmetic
  // runs on packed pairs of horizontally adjacent outputs (f32x2). With stride 1 the window
  // of a row is kept as its NV-1 consecutive pairs (v[i], v[i+1]) so every tap of an output
  // pair is one packed multiply and one packed add; with stride 2 (and for the
  // register-heavy 5x5 half case) the taps stay scalar and only BN is packed.
  constexpr bool PACKED_CONV = (STRIDE == 1) && !(K == 5 && sizeof(T) == 2);
  constexpr int NPR = S / 2;   // output pairs per patch row
  constexpr int NWP = NV - 1;  // consecutive pairs of a window row
  const f32x2 nz = negzero2();
  // One patch per thread: the block is (strips, planes, row blocks), so the patch
  // coordinates are the thread indices (no division).
  for (int once = 0; once < 1; ++once) {
    const int sx = threadIdx.x;
    const int pl = threadIdx.y;
    const int rb = threadIdx.z;
    if (pl >= pv) break;
    const int ox0 = sx * S;
    const int oyb = oy0 + rb * R;
    const int plane = plane0 + pl;
    T *yp = y + ((long long)plane * a.Ho + oyb) * a.Wo + ox0;
    const float *pp = prm + pl * PL::COUNT;

    if (pp[PL::SCAL + 5] != 0.0f) {
      // exact evaluation of this patch, tap by tap from global memory
      const int oc = plane % a.OC;
      float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
      for (int r = 0; r < R; ++r) {
        for (int j = 0; j < S; ++j) {
          if (oyb + r >= a.Ho || ox0 + j >= a.Wo) continue;
          const float v = prequant_point<T>(a, plane / a.OC, oc, oyb + r, ox0 + j);
          if (QM == QM_MM_REDUCE) {
            lo = fminf(lo, v);
            hi = fmaxf(hi, v);
          } else {
            yp[(size_t)r * a.Wo + j] = Elem<T>::from_f32(quant_apply<QM>(v, a.q, load_mm<QM>(a, oc)));
          }
        }
      }
      if (QM == QM_MM_REDUCE) {
        atomicMin(red + 2 * pl, enc_ordered(lo));
        atomicMax(red + 2 * pl + 1, enc_ordered(hi));
      }
      continue;
    }

    // packed operands straight from the record
    const f32x2 *pq = reinterpret_cast<const f32x2 *>(pp);
    f32x2 w2[PACKED_CONV ? PL::KK : 1];
    float wr[PACKED_CONV ? 1 : PL::KK];
#pragma unroll
    for (int i = 0; i < PL::KK; ++i) {
      if (PACKED_CONV) {
        w2[i] = pq[i];
        pin(w2[i]);
      } else {
        wr[i] = pp[2 * i];
        pin(wr[i]);
      }
    }
    f32x2 bias2 = pq[PL::PAIRS / 2];
    pin(bias2);
    BnPacked bnp;
    bnp.nmean = pq[PL::PAIRS / 2 + 1];
    bnp.scale = pq[PL::PAIRS / 2 + 2];
    bnp.rcp = pq[PL::PAIRS / 2 + 3];
    bnp.nstd = pq[PL::PAIRS / 2 + 4];
    bnp.beta = pq[PL::PAIRS / 2 + 5];
    bnp.nz = nz;
    bnp.stdvar = pp[PL::SCAL];
    bnp.glo = pp[PL::SCAL + 1];
    const MmCoef mm{pp[PL::SCAL + 2], pp[PL::SCAL + 3], pp[PL::SCAL + 4]};
    const bool full_vec = c.vec_store && (ox0 + S <= a.Wo);

    // Window source. Padded modes: 16-byte aligned position of the first output's centre tap
    // column in tile row 0 of this row block. Raw mode: element (row 0, column of window
    // position 0) of the plane, any alignment, plus the per-position halo masks.
    const T *tp;
    unsigned int cmask[MODE == TM_RAW ? NV : 1];
    int iy_first = 0;
    int row_pitch;
    if (MODE == TM_RAW) {
      const int c0 = ox0 * STRIDE - PAD;
      iy_first = rb * R * STRIDE - PAD;
      row_pitch = a.W;
      tp = tiles + c.raw_lead + pl * c.tile_elems + iy_first * a.W + c0;
#pragma unroll
      for (int i = 0; i < NV; ++i) cmask[i] = (c0 + i >= 0 && c0 + i < a.W) ? 0xffffffffu : 0u;
    } else {
      row_pitch = c.WS;
      tp = tiles + pl * c.tile_elems + (rb * R * STRIDE) * c.WS + S + sx * (S * STRIDE);
    }

    float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
    // window storage: packed pairs or scalars, whichever the conv uses
    f32x2 wp[PACKED_CONV ? K : 1][PACKED_CONV ? NWP : 1];
    float win[PACKED_CONV ? 1 : K][PACKED_CONV ? 1 : NV];
    // loads tile row `row` of this item into window slot row % K (row is a compile-time
    // constant at every call site once the loops below are unrolled)
    auto load_row = [&](int row) {
      float v[NV];
      if (MODE == TM_RAW) {
        const int iy = iy_first + row;
        if (iy >= 0 && iy < a.H) {
          load_window_raw<T, NV>(tp + row * row_pitch, cmask, v);
        } else {
#pragma unroll
          for (int i = 0; i < NV; ++i) v[i] = 0.0f;
        }
      } else {
        load_window<T, PAD, NV>(tp + row * row_pitch, v);
      }
      if (PACKED_CONV) {
#pragma unroll
        for (int i = 0; i < NWP; ++i) wp[row % K][i] = pack2(v[i], v[i + 1]);
      } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) win[row % K][i] = v[i];
      }
    };
#pragma unroll
    for (int i = 0; i < K - STRIDE; ++i) load_row(i);

    // The rows of the patch. QM_FPQ_LEAN is the common case, selected by the host for the
    // whole launch - BN present, power-of-two unsigned FixedPointQuantize, Ho a multiple of R
    // and Wo of the vector width with y aligned - and compiled without any per-row test.
    {
      constexpr bool LEAN = QM == QM_FPQ_LEAN;
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int i = 0; i < STRIDE; ++i) load_row(r * STRIDE + (K - STRIDE) + i);
        f32x2 acc[NPR];
        if (PACKED_CONV) {
#pragma unroll
          for (int ky = 0; ky < K; ++ky) {
#pragma unroll
            for (int kx = 0; kx < K; ++kx) {
#pragma unroll
              for (int p = 0; p < NPR; ++p)
                acc[p] = add2((ky == 0 && kx == 0) ? bias2 : acc[p],
                              mul2(w2[ky * K + kx], wp[(r * STRIDE + ky) % K][2 * p + kx], nz));
            }
          }
        } else {
          float b0, b1;
          unpack2(bias2, b0, b1);
          float sa[S];
#pragma unroll
          for (int j = 0; j < S; ++j) sa[j] = b0;
#pragma unroll
          for (int ky = 0; ky < K; ++ky) {
#pragma unroll
            for (int kx = 0; kx < K; ++kx) {
#pragma unroll
              for (int j = 0; j < S; ++j)
                sa[j] = __fadd_rn(sa[j], __fmul_rn(wr[ky * K + kx], win[(r * STRIDE + ky) % K][j * STRIDE + kx]));
            }
          }
#pragma unroll
          for (int p = 0; p < NPR; ++p) acc[p] = pack2(sa[2 * p], sa[2 * p + 1]);
        }
        if (LEAN || a.has_bn) bn_apply_packed<NPR>(acc, bnp);
        float out[S];
#pragma unroll
        for (int p = 0; p < NPR; ++p) unpack2(acc[p], out[2 * p], out[2 * p + 1]);
        if (LEAN) {
#pragma unroll
          for (int j = 0; j < S; ++j) out[j] = fpq_apply_fast<false>(out[j], a.q);
          Vec16<T>::store_stream(yp + (size_t)r * a.Wo, out);
          continue;
        }
        const bool row_ok = oyb + r < a.Ho;
        if (QM == QM_MM_REDUCE) {
#pragma unroll
          for (int j = 0; j < S; ++j) {
            if (row_ok && ox0 + j < a.Wo) {
              lo = fminf(lo, out[j]);
              hi = fmaxf(hi, out[j]);
            }
          }
        } else {
          if (QM == QM_FPQ && a.q.fpq_fast) {
            if (a.q.fpq_min < 0.0f) {
#pragma unroll
              for (int j = 0; j < S; ++j) out[j] = fpq_apply_fast<true>(out[j], a.q);
            } else {
#pragma unroll
              for (int j = 0; j < S; ++j) out[j] = fpq_apply_fast<false>(out[j], a.q);
            }
          } else {
#pragma unroll
            for (int j = 0; j < S; ++j) out[j] = quant_apply<QM>(out[j], a.q, mm);
          }
          if (row_ok) {
            T *yr = yp + (size_t)r * a.Wo;
            if (full_vec) {
              Vec16<T>::store_stream(yr, out);
            } else {
#pragma unroll
              for (int j = 0; j < S; ++j)
                if (ox0 + j < a.Wo) yr[j] = Elem<T>::from_f32(out[j]);
            }
          }
        }
      }
    }
    if (QM == QM_MM_REDUCE) {
      atomicMin(red + 2 * pl, enc_ordered(lo));
      atomicMax(red + 2 * pl + 1, enc_ordered(hi));
    }
  }

  if (QM == QM_MM_REDUCE) {
    __syncthreads();
    for (int i = tid; i < pv; i += nthr) {
      const int ch = (plane0 + i) % a.OC;
      atomicMin(a.q.mm_enc_min + ch, red[2 * i]);
      atomicMax(a.q.mm_enc_max + ch, red[2 * i + 1]);
    }
  }
}

constexpr int kRowsPerPatch = 7;

// ---- host-side entry of each instantiation family (defined in fused_tiled_*.cu) --------
// Launches fused_tiled_kernel<T, K, STRIDE, kRowsPerPatch, QM, MODE>, one CTA per tile.
template <typename T, int K>
cudaError_t launch_tiled(int stride, int qm, int mode, const CUtensorMap &tmap, const FusedArgs &a,
                         const TileCfg &c, int ctas, int threads, size_t smem, cudaStream_t stream);

}  // namespace dwbnq
