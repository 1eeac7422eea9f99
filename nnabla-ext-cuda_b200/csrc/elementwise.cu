// Streaming kernels of the standalone operators: BatchNormalization inference,
// FixedPointQuantize, Pow2Quantize and the pieces of MinMaxQuantize (per-channel min/max
// reduction, range derivation, quantize step). All are HBM-bound: 16-byte loads and
// stores, grids sized in multiples of the SM count, one pass over the data each.
#include "dwbnq_internal.h"

namespace dwbnq {

namespace {

constexpr int kThreads = 256;

// Grid of at most `per_sm` CTAs per SM of the current device (the entry points have made
// the call's device current before they come here).
inline unsigned int grid_for(long long work_items, int per_sm) {
  long long blocks = (work_items + kThreads - 1) / kThreads;
  const long long cap = (long long)sm_count(-1) * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned int)blocks;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) % 16) == 0; }

// ---- flat element-wise quantizers -------------------------------------------------------

template <typename T, int QM>
__global__ void __launch_bounds__(kThreads) quant_flat_kernel(const T *x, T *y,
                                                              const long long size, const int vec_ok,
                                                              const QuantArgs q) {
  constexpr int S = Elem<T>::VEC;
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const MmCoef none{1.0f, 0.0f, 0.0f};
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  const long long n_vec = vec_ok ? size / S : 0;
  constexpr int U = 4;  // vectors per thread whose loads are in flight together
  long long v = tid;
  for (; v + (U - 1) * step < n_vec; v += U * step) {
    float e[U][S];
#pragma unroll
    for (int u = 0; u < U; ++u) Vec16<T>::load_stream(x + (v + u * step) * S, e[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (QM == QM_POW2) {
        pow2_apply_n<S>(e[u], q);
      } else {
#pragma unroll
        for (int j = 0; j < S; ++j) e[u][j] = quant_apply<QM>(e[u][j], q, none);
      }
      Vec16<T>::store_stream(y + (v + u * step) * S, e[u]);
    }
  }
  for (; v < n_vec; v += step) {
    float e[S];
    Vec16<T>::load_stream(x + v * S, e);
#pragma unroll
    for (int j = 0; j < S; ++j) e[j] = quant_apply<QM>(e[j], q, none);
    Vec16<T>::store_stream(y + v * S, e);
  }
  for (long long i = n_vec * S + tid; i < size; i += step) {
    y[i] = Elem<T>::from_f32(quant_apply<QM>(Elem<T>::to_f32(x[i]), q, none));
  }
}

template <int QM>
int launch_quant_flat(int dtype, long long size, const QuantArgs &q, const void *x, void *y,
                      cudaStream_t stream) {
  if (size == 0) return DWBNQ_OK;
  const int vec_ok = aligned16(x) && aligned16(y);
  cudaError_t e;
  if (dtype == DWBNQ_F32) {
    e = launch_pdl(quant_flat_kernel<float, QM>, dim3(grid_for((size + 3) / 4, 16)), dim3(kThreads), 0, stream,
                   static_cast<const float *>(x), static_cast<float *>(y), size, vec_ok, q);
  } else {
    e = launch_pdl(quant_flat_kernel<__half, QM>, dim3(grid_for((size + 7) / 8, 16)), dim3(kThreads), 0, stream,
                   static_cast<const __half *>(x), static_cast<__half *>(y), size, vec_ok, q);
  }
  if (e != cudaSuccess) return fail_cuda(e, "quant_flat_kernel launch");
  return DWBNQ_OK;
}

// ---- per-channel element-wise ops on x viewed as [size0, C, size2] ------------------------
// 16-byte vectors of the flat array; (channel, offset inside the plane) is tracked
// incrementally per warp, so no division runs per vector in the common case.

enum ChanOp : int { OP_BN = 0, OP_MM_APPLY = 1 };

struct ChanArgs {
  // BN: vectors of the tensor dtype.
  const void *beta, *gamma, *mean, *var;
  float eps;
  // MinMax apply: fp32 workspace vectors.
  const float *mm_scale, *mm_lo, *mm_hi;
};

template <typename T, int OP> struct ChanCoef;
template <typename T> struct ChanCoef<T, OP_BN> {
  BnCoef c;
  __device__ __forceinline__ void load(const ChanArgs &a, int ch) {
    c.mean = Elem<T>::to_f32(static_cast<const T *>(a.mean)[ch]);
    c.scale = a.gamma ? Elem<T>::to_f32(static_cast<const T *>(a.gamma)[ch]) : 1.0f;
    c.stdvar = bn_stdvar(Elem<T>::to_f32(static_cast<const T *>(a.var)[ch]), a.eps);
    c.beta = a.beta ? Elem<T>::to_f32(static_cast<const T *>(a.beta)[ch]) : 0.0f;
  }
  __device__ __forceinline__ float apply(float v) const { return bn_apply(v, c); }
  __device__ __forceinline__ BnCoef coef() const { return c; }
};
template <typename T> struct ChanCoef<T, OP_MM_APPLY> {
  MmCoef c;
  __device__ __forceinline__ void load(const ChanArgs &a, int ch) {
    c.scale = a.mm_scale[ch];
    c.lo = a.mm_lo[ch];
    c.hi = a.mm_hi[ch];
  }
  __device__ __forceinline__ float apply(float v) const { return mm_apply(v, c); }
  __device__ __forceinline__ BnCoef coef() const { return BnCoef{0.0f, 1.0f, 1.0f, 0.0f}; }
};

// Vector path. A CTA owns a contiguous chunk of kChanChunkVecs vectors and each warp a
// contiguous run of it, 32 vectors per iteration: while the warp's span lies inside one plane
// (the common case) the per-channel operands are derived once per plane - for BN the packed
// form with the reciprocal of sqrt(var + eps) - and the arithmetic runs on f32x2 pairs.
// Spans that straddle a plane boundary fall back to per-element operands.
// x and y may be the same buffer (every vector is read before it is written, by one thread).
constexpr int kChanChunkVecs = kThreads * 8;

template <typename T, int OP>
__device__ __forceinline__ void chan_apply_whole(float *e, const ChanCoef<T, OP> &c, const BnPacked &bp) {
  constexpr int S = Elem<T>::VEC;
  if (OP == OP_BN) {
    f32x2 v[S / 2];
#pragma unroll
    for (int j = 0; j < S / 2; ++j) v[j] = pack2(e[2 * j], e[2 * j + 1]);
    bn_apply_packed<S / 2>(v, bp);
#pragma unroll
    for (int j = 0; j < S / 2; ++j) unpack2(v[j], e[2 * j], e[2 * j + 1]);
  } else {
#pragma unroll
    for (int j = 0; j < S; ++j) e[j] = c.apply(e[j]);
  }
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
    chan_vec_kernel(const T *x, T *y, const long long total, const int C,
                    const long long size2, const ChanArgs a) {
  constexpr int S = Elem<T>::VEC;
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const long long n_vec = total / S;
  const long long v_begin = (long long)blockIdx.x * kChanChunkVecs;
  const long long v_end = min(n_vec, v_begin + kChanChunkVecs);
  const long long e_begin = v_begin * S, e_end = v_end * S;
  const int lane = threadIdx.x & 31;
  const int iters = kChanChunkVecs / kThreads;
  const long long warp_first = e_begin + (long long)(threadIdx.x >> 5) * iters * 32 * S;
  if (warp_first < e_end) {
    long long plane = warp_first / size2;
    long long off = warp_first - plane * size2;  // offset of the warp's span inside its plane
    int ch = (int)(plane % C);
    bool have = false;
    ChanCoef<T, OP> c;
    BnPacked bp;
    const f32x2 nz = negzero2();
    auto advance = [&](int elems) {
      off += elems;
      while (off >= size2) {
        off -= size2;
        ch = ch + 1 == C ? 0 : ch + 1;
        have = false;
      }
    };
    auto ensure = [&]() {
      if (!have) {
        c.load(a, ch);
        if (OP == OP_BN) bp = make_bn_packed(c.coef(), nz);
        have = true;
      }
    };
    constexpr int U = 4;  // vectors per lane whose loads are in flight together
    static_assert((kChanChunkVecs / kThreads) % U == 0, "iterations come in groups of U");
    for (int it = 0; it < iters; it += U) {
      const long long span0 = warp_first + (long long)it * 32 * S;
      if (span0 >= e_end) break;  // uniform
      if (span0 + U * 32 * S <= e_end && off + U * 32 * S <= size2) {  // uniform: U spans, one plane
        ensure();
        const long long e0 = span0 + (long long)lane * S;
        float e[U][S];
#pragma unroll
        for (int u = 0; u < U; ++u) Vec16<T>::load_stream(x + e0 + u * 32 * S, e[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          chan_apply_whole<T, OP>(e[u], c, bp);
          Vec16<T>::store_stream(y + e0 + u * 32 * S, e[u]);
        }
        advance(U * 32 * S);
        continue;
      }
#pragma unroll 1
      for (int u = 0; u < U; ++u) {
        const long long sp = span0 + (long long)u * 32 * S;
        if (sp >= e_end) break;  // uniform
        const long long e0 = sp + (long long)lane * S;
        if (sp + 32 * S <= e_end && off + 32 * S <= size2) {  // uniform: the span lies in one plane
          ensure();
          float e[S];
          Vec16<T>::load_stream(x + e0, e);
          chan_apply_whole<T, OP>(e, c, bp);
          Vec16<T>::store_stream(y + e0, e);
        } else if (e0 + S <= e_end) {
          float e[S];
          Vec16<T>::load_stream(x + e0, e);
          const long long p0 = e0 / size2;
          const long long loff = e0 - p0 * size2;
          if (loff + S <= size2) {
            ChanCoef<T, OP> c0;
            c0.load(a, (int)(p0 % C));
#pragma unroll
            for (int j = 0; j < S; ++j) e[j] = c0.apply(e[j]);
          } else {
#pragma unroll
            for (int j = 0; j < S; ++j) {
              ChanCoef<T, OP> cj;
              cj.load(a, (int)(((e0 + j) / size2) % C));
              e[j] = cj.apply(e[j]);
            }
          }
          Vec16<T>::store_stream(y + e0, e);
        }
        advance(32 * S);
      }
    }
  }
  // scalar tail (total % VEC elements), by the last CTA
  if (blockIdx.x == gridDim.x - 1) {
    for (long long i = n_vec * S + threadIdx.x; i < total; i += blockDim.x) {
      ChanCoef<T, OP> ct;
      ct.load(a, (int)((i / size2) % C));
      y[i] = Elem<T>::from_f32(ct.apply(Elem<T>::to_f32(x[i])));
    }
  }
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
    chan_scalar_kernel(const T *x, T *y, const long long total, const int C,
                       const long long size2, const ChanArgs a) {
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int ch = (int)((i / size2) % C);
    ChanCoef<T, OP> c;
    c.load(a, ch);
    y[i] = Elem<T>::from_f32(c.apply(Elem<T>::to_f32(x[i])));
  }
}

template <typename T, int OP>
int launch_chan_t(long long size0, long long C, long long size2, const T *x, T *y, const ChanArgs &a,
                  cudaStream_t stream) {
  constexpr int S = Elem<T>::VEC;
  const long long total = size0 * C * size2;
  if (total == 0) return DWBNQ_OK;
  const bool vec = aligned16(x) && aligned16(y) && size2 >= S && size2 <= 0x7fffffffLL && C <= 0x7fffffffLL;
  const long long chunks = (total / S + kChanChunkVecs - 1) / kChanChunkVecs;
  if (vec && chunks >= 1 && chunks <= 0x7fffffffLL) {
    const cudaError_t le = launch_pdl(chan_vec_kernel<T, OP>, dim3((unsigned int)chunks), dim3(kThreads), 0, stream, x, y,
                                      total, (int)C, size2, a);
    if (le != cudaSuccess) return fail_cuda(le, "per-channel element-wise kernel launch");
  } else {
    chan_scalar_kernel<T, OP><<<grid_for(total, 16), kThreads, 0, stream>>>(x, y, total, (int)C, size2, a);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "per-channel element-wise kernel launch");
  return DWBNQ_OK;
}

// ---- MinMaxQuantize pieces ---------------------------------------------------------------

__global__ void mm_init_kernel(unsigned int *enc_min, unsigned int *enc_max, int C) {
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x) {
    enc_min[c] = DWBNQ_ENC_POS_INF;
    enc_max[c] = DWBNQ_ENC_NEG_INF;
  }
}

// Per-channel min / max of x viewed as [size0, C, size2]. A CTA owns a contiguous chunk of
// kChunkVecs vectors; it spans at most chunk/size2 + 2 planes, each with a pair of
// shared-memory slots that collect the CTA's partial result before one global atomic pair.
constexpr int kChunkVecs = kThreads * 8;

template <typename T>
__global__ void __launch_bounds__(kThreads)
    mm_reduce_kernel(const T *__restrict__ x, const long long total, const int C, const long long size2,
                     const int vec_ok, const int slots, unsigned int *__restrict__ enc_min,
                     unsigned int *__restrict__ enc_max) {
  constexpr int S = Elem<T>::VEC;
  extern __shared__ unsigned int s_red[];  // [slots][2]
  for (int i = threadIdx.x; i < slots; i += blockDim.x) {
    s_red[2 * i] = DWBNQ_ENC_POS_INF;
    s_red[2 * i + 1] = DWBNQ_ENC_NEG_INF;
  }
  __syncthreads();
  const long long chunk_elems = (long long)kChunkVecs * S;
  const long long e_begin = (long long)blockIdx.x * chunk_elems;
  const long long e_end = min(total, e_begin + chunk_elems);
  const long long plane_first = e_begin / size2;
  const float pinf = __uint_as_float(0x7f800000u), ninf = __uint_as_float(0xff800000u);
  if (vec_ok) {
    // A warp walks a contiguous run of the chunk, 32 vectors per iteration. While the warp's
    // span lies inside one plane (the common case for planes of a few hundred elements or
    // more) every lane accumulates in registers; the partial result goes to the plane's
    // shared-memory slot through one shuffle reduction when the plane changes. Spans that
    // straddle a plane boundary take the per-lane path.
    const int lane = threadIdx.x & 31;
    const int n_warps = blockDim.x >> 5;
    const int iters = kChunkVecs / kThreads;  // iterations per warp
    const long long warp_first = e_begin + (long long)(threadIdx.x >> 5) * iters * 32 * S;
    const long long rel0 = warp_first - plane_first * size2;  // < chunk + size2
    int slot = (int)(rel0 / size2);
    long long off = rel0 - (long long)slot * size2;  // offset of the warp's span inside its plane
    (void)n_warps;
    int cur = -1;
    float lo = pinf, hi = ninf;
    auto flush = [&]() {
      if (cur < 0) return;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
      }
      if (lane == 0) {
        if (lo != pinf) atomicMin(&s_red[2 * cur], enc_ordered(lo));
        if (hi != ninf) atomicMax(&s_red[2 * cur + 1], enc_ordered(hi));
      }
      lo = pinf;
      hi = ninf;
    };
    auto advance = [&](int elems) {
      off += elems;
      while (off >= size2) {
        off -= size2;
        ++slot;
      }
    };
    constexpr int U = 4;  // vectors per lane whose loads are in flight together
    static_assert((kChunkVecs / kThreads) % U == 0, "iterations come in groups of U");
    for (int it = 0; it < iters; it += U) {
      const long long span0 = warp_first + (long long)it * 32 * S;
      if (span0 >= e_end) break;  // uniform
      if (span0 + U * 32 * S <= e_end && off + U * 32 * S <= size2) {  // uniform: U spans, one plane
        if (slot != cur) {
          flush();
          cur = slot;
        }
        const long long e0 = span0 + (long long)lane * S;
        float e[U][S];
#pragma unroll
        for (int u = 0; u < U; ++u) Vec16<T>::load_stream(x + e0 + u * 32 * S, e[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int j = 0; j < S; ++j) {
            lo = fminf(lo, e[u][j]);
            hi = fmaxf(hi, e[u][j]);
          }
        }
        advance(U * 32 * S);
        continue;
      }
#pragma unroll 1
      for (int u = 0; u < U; ++u) {
        const long long sp = span0 + (long long)u * 32 * S;
        if (sp >= e_end) break;  // uniform
        const long long e0 = sp + (long long)lane * S;
        if (sp + 32 * S <= e_end && off + 32 * S <= size2) {  // uniform: the span lies in one plane
          if (slot != cur) {
            flush();
            cur = slot;
          }
          float e[S];
          Vec16<T>::load_stream(x + e0, e);
#pragma unroll
          for (int j = 0; j < S; ++j) {
            lo = fminf(lo, e[j]);
            hi = fmaxf(hi, e[j]);
          }
        } else if (e0 + S <= e_end) {
          float e[S];
          Vec16<T>::load_stream(x + e0, e);
          const long long plane = e0 / size2;
          const long long loff = e0 - plane * size2;
          const int sl = (int)(plane - plane_first);
          if (loff + S <= size2) {
            float l2 = pinf, h2 = ninf;
#pragma unroll
            for (int j = 0; j < S; ++j) {
              l2 = fminf(l2, e[j]);
              h2 = fmaxf(h2, e[j]);
            }
            if (l2 != pinf) atomicMin(&s_red[2 * sl], enc_ordered(l2));
            if (h2 != ninf) atomicMax(&s_red[2 * sl + 1], enc_ordered(h2));
          } else {
            // the vector straddles plane boundaries (possibly several when size2 < VEC)
#pragma unroll
            for (int j = 0; j < S; ++j) {
              const int s2 = (int)((e0 + j) / size2 - plane_first);
              if (e[j] == e[j]) {
                atomicMin(&s_red[2 * s2], enc_ordered(e[j]));
                atomicMax(&s_red[2 * s2 + 1], enc_ordered(e[j]));
              }
            }
          }
        } else {
          for (long long i = e0; i < e_end; ++i) {
            const float v = Elem<T>::to_f32(x[i]);
            const int s2 = (int)(i / size2 - plane_first);
            if (v == v) {
              atomicMin(&s_red[2 * s2], enc_ordered(v));
              atomicMax(&s_red[2 * s2 + 1], enc_ordered(v));
            }
          }
        }
        advance(32 * S);
      }
    }
    flush();
  } else {
    for (long long i = e_begin + threadIdx.x; i < e_end; i += blockDim.x) {
      const float v = Elem<T>::to_f32(x[i]);
      const int sl = (int)(i / size2 - plane_first);
      if (v == v) {
        atomicMin(&s_red[2 * sl], enc_ordered(v));
        atomicMax(&s_red[2 * sl + 1], enc_ordered(v));
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < slots; i += blockDim.x) {
    const long long plane = plane_first + i;
    if (plane * size2 >= e_end) break;
    const int ch = (int)(plane % C);
    if (s_red[2 * i] != DWBNQ_ENC_POS_INF) atomicMin(enc_min + ch, s_red[2 * i]);
    if (s_red[2 * i + 1] != DWBNQ_ENC_NEG_INF) atomicMax(enc_max + ch, s_red[2 * i + 1]);
  }
}

__global__ void mm_pack_kernel(const unsigned int *enc_min, const unsigned int *enc_max,
                               float *packed, int C) {
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x) {
    packed[c] = dec_ordered(enc_max[c]);
    packed[C + c] = -dec_ordered(enc_min[c]);
  }
}

// Range derivation: the two hooks of MinMaxQuantizeCuda
// (src/nbla/cuda/function/generic/min_max_quantize.cu:29-61) around the scale division.
template <typename T>
__global__ void mm_ranges_kernel(int C, int x_min_max, int ema, float decay, float eps, T *qr_min,
                                 T *qr_max, const T *ql_min, const T *ql_max,
                                 const unsigned int *enc_min, const unsigned int *enc_max,
                                 const float *packed, float *scale_out, float *lo_out,
                                 float *hi_out) {
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x) {
    float mn = Elem<T>::to_f32(qr_min[c]);
    float mx = Elem<T>::to_f32(qr_max[c]);
    if (x_min_max) {
      const float bmn = packed ? -packed[C + c] : dec_ordered(enc_min[c]);
      const float bmx = packed ? packed[c] : dec_ordered(enc_max[c]);
      if (ema) {
        const float om = __fsub_rn(1.0f, decay);
        mn = __fadd_rn(__fmul_rn(decay, mn), __fmul_rn(om, bmn));
        mx = __fadd_rn(__fmul_rn(decay, mx), __fmul_rn(om, bmx));
      } else {
        mn = bmn;
        mx = bmx;
      }
    }
    if (__fsub_rn(mx, mn) < eps) mx = __fadd_rn(mn, eps);
    if (x_min_max) qr_min[c] = Elem<T>::from_f32(mn);
    qr_max[c] = Elem<T>::from_f32(mx);
    const float qlo = Elem<T>::to_f32(ql_min[c]);
    const float qhi = Elem<T>::to_f32(ql_max[c]);
    const float scale = __fdiv_rn(__fsub_rn(mx, mn), __fsub_rn(qhi, qlo));
    const float zp_from_min = __fsub_rn(qlo, __fdiv_rn(mn, scale));
    float zp;
    if (zp_from_min <= qlo) zp = qlo;
    else if (zp_from_min >= qhi) zp = qhi;
    else zp = roundf(zp_from_min);
    scale_out[c] = scale;
    lo_out[c] = __fmul_rn(__fsub_rn(qlo, zp), scale);
    hi_out[c] = __fmul_rn(__fsub_rn(qhi, zp), scale);
  }
}

}  // namespace

int launch_fpq(int dtype, long long size, const QuantArgs &q, const void *x, void *y,
               cudaStream_t stream) {
  return launch_quant_flat<QM_FPQ>(dtype, size, q, x, y, stream);
}
int launch_pow2q(int dtype, long long size, const QuantArgs &q, const void *x, void *y,
                 cudaStream_t stream) {
  return launch_quant_flat<QM_POW2>(dtype, size, q, x, y, stream);
}

int launch_bn_infer(int dtype, long long size0, long long size1, long long size2, float eps,
                    const void *x, const void *beta, const void *gamma, const void *mean,
                    const void *var, void *y, cudaStream_t stream) {
  ChanArgs a{};
  a.beta = beta;
  a.gamma = gamma;
  a.mean = mean;
  a.var = var;
  a.eps = eps;
  if (dtype == DWBNQ_F32)
    return launch_chan_t<float, OP_BN>(size0, size1, size2, static_cast<const float *>(x),
                                       static_cast<float *>(y), a, stream);
  return launch_chan_t<__half, OP_BN>(size0, size1, size2, static_cast<const __half *>(x),
                                      static_cast<__half *>(y), a, stream);
}

MmWorkspace mm_workspace(void *ws, int C) {
  MmWorkspace w;
  unsigned int *u = static_cast<unsigned int *>(ws);
  w.enc_min = u;
  w.enc_max = u + C;
  float *f = reinterpret_cast<float *>(u + 2 * (size_t)C);
  w.scale = f;
  w.lo = f + C;
  w.hi = f + 2 * (size_t)C;
  w.packed = f + 3 * (size_t)C;
  return w;
}

int launch_mm_init(const MmWorkspace &w, int C, cudaStream_t stream) {
  mm_init_kernel<<<(C + 255) / 256, 256, 0, stream>>>(w.enc_min, w.enc_max, C);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "mm_init_kernel launch");
  return DWBNQ_OK;
}

int launch_mm_reduce(int dtype, long long size0, int C, long long size2, const void *x,
                     const MmWorkspace &w, cudaStream_t stream) {
  const long long total = size0 * C * size2;
  if (total == 0) return DWBNQ_OK;
  const int S = dtype == DWBNQ_F32 ? 4 : 8;
  const long long chunk_elems = (long long)kChunkVecs * S;
  const long long blocks = (total + chunk_elems - 1) / chunk_elems;
  if (blocks > 0x7fffffffLL) return fail(DWBNQ_ERR_UNSUPPORTED, "tensor too large for the min/max reduction grid");
  const int slots = (int)(chunk_elems / size2) + 2;
  const size_t smem = (size_t)slots * 2 * sizeof(unsigned int);
  const int vec_ok = aligned16(x) ? 1 : 0;
  cudaError_t e;
  if (dtype == DWBNQ_F32) {
    auto k = mm_reduce_kernel<float>;
    if (smem > 48 * 1024) {
      e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(mm_reduce_kernel)");
    }
    k<<<(unsigned)blocks, kThreads, smem, stream>>>(static_cast<const float *>(x), total, C, size2, vec_ok, slots, w.enc_min, w.enc_max);
  } else {
    auto k = mm_reduce_kernel<__half>;
    if (smem > 48 * 1024) {
      e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail_cuda(e, "cudaFuncSetAttribute(mm_reduce_kernel)");
    }
    k<<<(unsigned)blocks, kThreads, smem, stream>>>(static_cast<const __half *>(x), total, C, size2, vec_ok, slots, w.enc_min, w.enc_max);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "mm_reduce_kernel launch");
  return DWBNQ_OK;
}

int launch_mm_pack(const MmWorkspace &w, int C, cudaStream_t stream) {
  mm_pack_kernel<<<(C + 255) / 256, 256, 0, stream>>>(w.enc_min, w.enc_max, w.packed, C);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "mm_pack_kernel launch");
  return DWBNQ_OK;
}

int launch_mm_ranges(int dtype, int C, const dwbnq_quant_desc &q, const dwbnq_minmax_ptrs &mm,
                     const MmWorkspace &w, int from_packed, cudaStream_t stream) {
  const int grid = (C + 255) / 256;
  if (dtype == DWBNQ_F32) {
    mm_ranges_kernel<float><<<grid, 256, 0, stream>>>(
        C, q.x_min_max, q.ema, q.decay, q.eps, static_cast<float *>(mm.qr_min),
        static_cast<float *>(mm.qr_max), static_cast<const float *>(mm.ql_min),
        static_cast<const float *>(mm.ql_max), w.enc_min, w.enc_max,
        from_packed ? w.packed : nullptr, w.scale, w.lo, w.hi);
  } else {
    mm_ranges_kernel<__half><<<grid, 256, 0, stream>>>(
        C, q.x_min_max, q.ema, q.decay, q.eps, static_cast<__half *>(mm.qr_min),
        static_cast<__half *>(mm.qr_max), static_cast<const __half *>(mm.ql_min),
        static_cast<const __half *>(mm.ql_max), w.enc_min, w.enc_max,
        from_packed ? w.packed : nullptr, w.scale, w.lo, w.hi);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "mm_ranges_kernel launch");
  return DWBNQ_OK;
}

int launch_mm_apply(int dtype, long long size0, int C, long long size2, const void *x, void *y,
                    const MmWorkspace &w, cudaStream_t stream) {
  ChanArgs a{};
  a.mm_scale = w.scale;
  a.mm_lo = w.lo;
  a.mm_hi = w.hi;
  if (dtype == DWBNQ_F32)
    return launch_chan_t<float, OP_MM_APPLY>(size0, C, size2, static_cast<const float *>(x),
                                             static_cast<float *>(y), a, stream);
  return launch_chan_t<__half, OP_MM_APPLY>(size0, C, size2, static_cast<const __half *>(x),
                                            static_cast<__half *>(y), a, stream);
}

}  // namespace dwbnq
