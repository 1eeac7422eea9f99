// Fused DepthwiseConvolution -> BatchNormalization(inference) -> quantizer kernels.
//
// Two kernel families share one arithmetic core:
//  * fused_generic_kernel: one thread per output element, taps read straight from global
//    memory, out-of-bounds taps skipped. Handles every geometry the reference accepts
//    (any kernel size, stride, pad, dilation, multiplier, 1-D) and is also the in-kernel
//    fall-back of the tiled family for the parameter values where "skip the tap" and
//    "add w * 0" differ (bias == -0.0, non-finite weights).
//  * fused_tiled_kernel: a CTA owns `P` (n, c) planes x one tile of output rows. The
//    halo'd, zero-padded input tile is staged in shared memory - by one TMA tiled load
//    per plane (out-of-bounds rows / columns arrive as zeros) or, where the row pitch
//    is not a multiple of 16 bytes, by cooperative loads - and each thread computes
//    R x VEC output patches from a rolling register window, then applies BN and the
//    quantizer in registers and stores 16-byte vectors.
//
// Arithmetic contract (identical in both families): accumulator starts at the bias,
// taps in ky-major / kx-minor order, product and sum rounded separately (no FMA),
// then the BN and quantizer steps of dwbnq_device.cuh.
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
};

// Geometry of the tiled family, fixed by the host planner.
struct TileCfg {
  int P;            // planes per CTA
  int TH;           // output rows per tile (multiple of R)
  int n_row_tiles;  // ceil(Ho / TH)
  int n_strips;     // ceil(Wo / VEC)
  int n_rb;         // TH / R
  int WS;           // shared-memory row pitch in elements (multiple of VEC)
  int TR;           // input rows a tile needs: (TH - 1) * stride + K
  int box_rows;     // rows per TMA box (<= 256)
  int n_boxes;      // boxes per plane; the tile holds n_boxes * box_rows rows
  int tile_elems;   // elements per plane tile (multiple of 128 bytes)
  int vec_store;    // Wo % VEC == 0 and y 16-byte aligned
  int vec_fill;     // cooperative fill may use 16-byte global loads
};

// ---- exact single-output evaluation (generic family and fall-back) -------------------

template <typename T>
__device__ __forceinline__ float conv_point(const FusedArgs &a, long long n, int oc, int oy,
                                            int ox) {
  const T *x = static_cast<const T *>(a.x);
  const T *w = static_cast<const T *>(a.w);
  const T *b = static_cast<const T *>(a.b);
  const int ic = oc / a.mult;
  const T *xp = x + (n * a.C + ic) * (long long)a.H * a.W;
  const T *wp = w + (long long)oc * a.kh * a.kw;
  float acc = b ? Elem<T>::to_f32(b[oc]) : 0.0f;
  for (int ky = 0; ky < a.kh; ++ky) {
    const int iy = oy * a.sh + ky * a.dh - a.ph;
    for (int kx = 0; kx < a.kw; ++kx) {
      const int ix = ox * a.sw + kx * a.dw - a.pw;
      if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W) {
        const float xv = Elem<T>::to_f32(xp[(long long)iy * a.W + ix]);
        const float wv = Elem<T>::to_f32(wp[ky * a.kw + kx]);
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
    } else if (valid) {
      y[o] = Elem<T>::from_f32(quant_apply<QM>(v, a.q, load_mm<QM>(a, oc)));
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
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned int parity) {
  unsigned int ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after ~2^20 polls (each poll itself blocks for a hardware time
// slice), so a transfer that never lands cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long *bar, unsigned int parity) {
  for (unsigned int i = 0; i < (1u << 20); ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
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

// ---- the tiled kernel ----------------------------------------------------------------

// Per-plane parameter record in shared memory: K*K weights, bias, BN (mean, scale,
// stdvar, beta), MinMax (scale, lo, hi).
constexpr int kParamExtra = 8;
template <int K> struct ParamLayout {
  static constexpr int KK = K * K;
  static constexpr int BIAS = KK;
  static constexpr int BN = KK + 1;
  static constexpr int MM = KK + 5;
  static constexpr int COUNT = KK + kParamExtra;
};

// Shared-memory carve-up, also used by the host planner to size the launch.
__host__ __device__ inline size_t tiled_smem_bytes(int P, int tile_elems, int elem_size, int K) {
  size_t s = (size_t)P * tile_elems * elem_size;         // tiles (each a multiple of 128 B)
  s += (size_t)P * (K * K + kParamExtra) * sizeof(float);  // parameter records
  s += (size_t)P * 2 * sizeof(unsigned int);              // per-plane encoded min / max
  s = (s + 15) / 16 * 16;
  s += 16;                                                // mbarrier + fall-back flag
  return s;
}

template <typename T, int K, int STRIDE, int R, int QM, bool USE_TMA>
__global__ void __launch_bounds__(256)
    fused_tiled_kernel(const __grid_constant__ CUtensorMap tmap, const FusedArgs a,
                       const TileCfg c) {
  constexpr int S = Elem<T>::VEC;
  constexpr int PAD = K / 2;
  constexpr int NV = (S - 1) * STRIDE + K;
  using PL = ParamLayout<K>;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *tiles = reinterpret_cast<T *>(smem_raw);
  float *prm = reinterpret_cast<float *>(smem_raw + (size_t)c.P * c.tile_elems * sizeof(T));
  unsigned int *red = reinterpret_cast<unsigned int *>(prm + c.P * PL::COUNT);
  unsigned long long *bar = reinterpret_cast<unsigned long long *>(
      (reinterpret_cast<uintptr_t>(red + 2 * c.P) + 15) / 16 * 16);
  int *s_exact = reinterpret_cast<int *>(bar + 1);

  const int tid = threadIdx.x;
  const int nthr = blockDim.x;
  const long long n_planes = a.n * a.OC;  // multiplier == 1 in this family
  const long long grp = blockIdx.x / c.n_row_tiles;
  const int rt = (int)(blockIdx.x - grp * c.n_row_tiles);
  const long long plane0 = grp * c.P;
  const int pv = (int)min((long long)c.P, n_planes - plane0);
  const int oy0 = rt * c.TH;
  const int iy0 = oy0 * STRIDE - PAD;
  const int rows_alloc = c.box_rows * c.n_boxes;

  if (tid == 0) {
    *s_exact = 0;
    if (USE_TMA) {
      mbar_init(bar, 1);
      mbar_fence_init();
    }
  }
  __syncthreads();

  // ---- producer ------------------------------------------------------------------------
  if (USE_TMA) {
    if (tid == 0) {
      const unsigned int bytes =
          (unsigned int)((size_t)pv * rows_alloc * c.WS * sizeof(T));
      mbar_expect_tx(bar, bytes);
      for (int pl = 0; pl < pv; ++pl) {
        for (int bx = 0; bx < c.n_boxes; ++bx) {
          tma_load_3d(tiles + (size_t)pl * c.tile_elems + (size_t)bx * c.box_rows * c.WS, &tmap,
                      -S, iy0 + bx * c.box_rows, (int)(plane0 + pl), bar);
        }
      }
    }
  } else {
    // Cooperative fill: every 16-byte group of the zero-padded tile is produced by one
    // thread (zeros outside the image).
    const T *x = static_cast<const T *>(a.x);
    const int gpr = c.WS / S;  // groups per row
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
        const T *src = x + ((plane0 + pl) * (long long)a.H + iy) * a.W + ix0;
        if (c.vec_fill && ix0 >= 0 && ix0 + S <= a.W) {
          Vec16<T>::load_stream(src, v);
        } else {
#pragma unroll
          for (int j = 0; j < S; ++j) {
            if (ix0 + j >= 0 && ix0 + j < a.W) v[j] = Elem<T>::to_f32(src[j]);
          }
        }
      }
      Vec16<T>::store(tiles + (size_t)pl * c.tile_elems + (size_t)tr * c.WS + gc * S, v);
    }
  }

  // ---- per-plane parameters (overlaps the TMA transfer) ---------------------------------
  {
    const T *w = static_cast<const T *>(a.w);
    const T *b = static_cast<const T *>(a.b);
    for (int i = tid; i < pv * PL::COUNT; i += nthr) {
      const int pl = i / PL::COUNT;
      const int j = i - pl * PL::COUNT;
      const int ch = (int)((plane0 + pl) % a.OC);
      float val = 0.0f;
      if (j < PL::KK) {
        val = Elem<T>::to_f32(w[(long long)ch * PL::KK + j]);
        // w * 0 must be +-0 for the zero padding to act as "skip the tap".
        if (!(fabsf(val) <= 3.402823466e38f)) atomicExch(s_exact, 1);
      } else if (j == PL::BIAS) {
        val = b ? Elem<T>::to_f32(b[ch]) : 0.0f;
        // -0.0 + (+0.0) = +0.0 would change the sign of an all-zero accumulation.
        if (__float_as_uint(val) == 0x80000000u) atomicExch(s_exact, 1);
      } else if (j < PL::MM) {
        if (a.has_bn) {
          const BnCoef bc = load_bn<T>(a, ch);
          val = (j == PL::BN) ? bc.mean : (j == PL::BN + 1) ? bc.scale
                : (j == PL::BN + 2) ? bc.stdvar : bc.beta;
        }
      } else if (QM == QM_MM_APPLY) {
        val = (j == PL::MM) ? a.q.mm_scale[ch] : (j == PL::MM + 1) ? a.q.mm_lo[ch]
              : (j == PL::MM + 2) ? a.q.mm_hi[ch] : 0.0f;
      }
      prm[i] = val;
    }
    if (QM == QM_MM_REDUCE) {
      for (int i = tid; i < pv; i += nthr) {
        red[2 * i] = DWBNQ_ENC_POS_INF;
        red[2 * i + 1] = DWBNQ_ENC_NEG_INF;
      }
    }
  }
  __syncthreads();

  if (USE_TMA) {
    if (!mbar_wait_bounded(bar, 0)) {
      if (tid == 0 && a.flag) atomicExch(a.flag, 1);
      return;
    }
  }

  T *y = static_cast<T *>(a.y);

  // ---- exact fall-back for the rare parameter values named above ------------------------
  if (*s_exact) {
    const int per_plane = c.TH * a.Wo;
    for (int i = tid; i < pv * per_plane; i += nthr) {
      const int pl = i / per_plane;
      const int rem = i - pl * per_plane;
      const int oy = oy0 + rem / a.Wo;
      const int ox = rem % a.Wo;
      if (oy >= a.Ho) continue;
      const long long plane = plane0 + pl;
      const int oc = (int)(plane % a.OC);
      const float v = prequant_point<T>(a, plane / a.OC, oc, oy, ox);
      if (QM == QM_MM_REDUCE) {
        if (v == v) {
          atomicMin(a.q.mm_enc_min + oc, enc_ordered(v));
          atomicMax(a.q.mm_enc_max + oc, enc_ordered(v));
        }
      } else {
        y[(plane * a.Ho + oy) * (long long)a.Wo + ox] =
            Elem<T>::from_f32(quant_apply<QM>(v, a.q, load_mm<QM>(a, oc)));
      }
    }
    return;
  }

  // ---- consumer: R x S output patches from a rolling K-row register window ---------------
  // Arithmetic runs on packed pairs of horizontally adjacent outputs (f32x2). With stride 1
  // the window of a row is kept as its NV-1 consecutive pairs (v[i], v[i+1]) so every tap of
  // an output pair is one packed multiply and one packed add; with stride 2 (and for the
  // register-heavy 5x5 half case) the taps stay scalar and only BN / quantizer are packed.
  constexpr bool PACKED_CONV = (STRIDE == 1) && !(K == 5 && S == 8);
  constexpr int NPR = S / 2;   // output pairs per patch row
  constexpr int NWP = NV - 1;  // consecutive pairs of a window row
  const int ipp = c.n_strips * c.n_rb;  // items per plane
  const int n_items = pv * ipp;
  for (int it = tid; it < n_items; it += nthr) {
    const int pl = it / ipp;
    const int rem = it - pl * ipp;
    const int rb = rem / c.n_strips;
    const int st = rem - rb * c.n_strips;

    const float *pp = prm + pl * PL::COUNT;
    const float bias = pp[PL::BIAS];
    const BnCoef bn{pp[PL::BN], pp[PL::BN + 1], pp[PL::BN + 2], pp[PL::BN + 3]};
    const BnPacked bnp = make_bn_packed(bn);
    const MmCoef mm{pp[PL::MM], pp[PL::MM + 1], pp[PL::MM + 2]};

    // 16-byte aligned position of the first output's centre tap column in tile row 0 of
    // this row block.
    const T *tp = tiles + (size_t)pl * c.tile_elems + (size_t)(rb * R * STRIDE) * c.WS + S +
                  st * (S * STRIDE);
    const int ox0 = st * S;
    const int oyb = oy0 + rb * R;
    T *yp = y + ((plane0 + pl) * a.Ho + oyb) * (long long)a.Wo + ox0;
    const bool full_vec = c.vec_store && (ox0 + S <= a.Wo);

    float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
    // window storage: packed pairs or scalars, whichever the conv uses
    f32x2 wp[PACKED_CONV ? K : 1][PACKED_CONV ? NWP : 1];
    float win[PACKED_CONV ? 1 : K][PACKED_CONV ? 1 : NV];
    f32x2 w2[PACKED_CONV ? PL::KK : 1];
    float wr[PACKED_CONV ? 1 : PL::KK];
#pragma unroll
    for (int i = 0; i < PL::KK; ++i) {
      if (PACKED_CONV) w2[i] = splat2(pp[i]);
      else wr[i] = pp[i];
    }
    auto load_row = [&](int row) {
      if (PACKED_CONV) {
        float v[NV];
        load_window<T, PAD, NV>(tp + (size_t)row * c.WS, v);
#pragma unroll
        for (int i = 0; i < NWP; ++i) wp[row % K][i] = pack2(v[i], v[i + 1]);
      } else {
        load_window<T, PAD, NV>(tp + (size_t)row * c.WS, win[row % K]);
      }
    };
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r == 0) {
#pragma unroll
        for (int i = 0; i < K; ++i) load_row(i);
      } else {
#pragma unroll
        for (int i = 0; i < STRIDE; ++i) load_row((r - 1) * STRIDE + K + i);
      }
      f32x2 acc[NPR];
      if (PACKED_CONV) {
        const f32x2 bias2 = splat2(bias);
#pragma unroll
        for (int p = 0; p < NPR; ++p) acc[p] = bias2;
#pragma unroll
        for (int ky = 0; ky < K; ++ky) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) {
#pragma unroll
            for (int p = 0; p < NPR; ++p)
              acc[p] = add2(acc[p], mul2(w2[ky * K + kx], wp[(r * STRIDE + ky) % K][2 * p + kx]));
          }
        }
      } else {
        float sa[S];
#pragma unroll
        for (int j = 0; j < S; ++j) sa[j] = bias;
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
      if (a.has_bn) bn_apply_packed<NPR>(acc, bnp);
      if (QM == QM_FPQ && a.q.fpq_fast) fpq_apply_packed_fast<NPR>(acc, a.q, a.q.fpq_min < 0.0f);
      float out[S];
#pragma unroll
      for (int p = 0; p < NPR; ++p) unpack2(acc[p], out[2 * p], out[2 * p + 1]);
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
        if (!(QM == QM_FPQ && a.q.fpq_fast)) {
#pragma unroll
          for (int j = 0; j < S; ++j) out[j] = quant_apply<QM>(out[j], a.q, mm);
        }
        if (row_ok) {
          if (full_vec) {
            Vec16<T>::store_stream(yp + (size_t)r * a.Wo, out);
          } else {
#pragma unroll
            for (int j = 0; j < S; ++j) {
              if (ox0 + j < a.Wo) yp[(size_t)r * a.Wo + j] = Elem<T>::from_f32(out[j]);
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
      const int ch = (int)((plane0 + i) % a.OC);
      atomicMin(a.q.mm_enc_min + ch, red[2 * i]);
      atomicMax(a.q.mm_enc_max + ch, red[2 * i + 1]);
    }
  }
}

// ---- host-side entry of each instantiation family (defined in fused_tiled_*.cu) --------
// Launches fused_tiled_kernel<T, K, STRIDE, 7, QM, USE_TMA>.
template <typename T, int K>
cudaError_t launch_tiled(int stride, int qm, bool use_tma, const CUtensorMap &tmap,
                         const FusedArgs &a, const TileCfg &c, long long ctas, int threads,
                         size_t smem, cudaStream_t stream);

constexpr int kRowsPerPatch = 7;

}  // namespace dwbnq
