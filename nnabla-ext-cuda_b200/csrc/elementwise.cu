// Streaming kernels of the standalone operators: BatchNormalization inference,
// FixedPointQuantize, Pow2Quantize and the pieces of MinMaxQuantize (per-channel min/max
// reduction, range derivation, quantize step). All are HBM-bound: 16-byte loads and
// stores, grids sized in multiples of the SM count, one pass over the data each.
#include "dwbnq_internal.h"

namespace dwbnq {

namespace {

constexpr int kThreads = 256;
constexpr int kSMs = 148;

inline unsigned int grid_for(long long work_items, int per_sm) {
  long long blocks = (work_items + kThreads - 1) / kThreads;
  const long long cap = (long long)kSMs * per_sm;
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
  const MmCoef none{1.0f, 0.0f, 0.0f};
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  const long long n_vec = vec_ok ? size / S : 0;
  for (long long v = tid; v < n_vec; v += step) {
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
  if (dtype == DWBNQ_F32) {
    quant_flat_kernel<float, QM><<<grid_for((size + 3) / 4, 16), kThreads, 0, stream>>>(
        static_cast<const float *>(x), static_cast<float *>(y), size, vec_ok, q);
  } else {
    quant_flat_kernel<__half, QM><<<grid_for((size + 7) / 8, 16), kThreads, 0, stream>>>(
        static_cast<const __half *>(x), static_cast<__half *>(y), size, vec_ok, q);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "quant_flat_kernel launch");
  return DWBNQ_OK;
}

// ---- per-channel element-wise ops on x viewed as [size0, C, size2] ------------------------
// A thread walks 16-byte vectors of the flat array with a fixed stride and tracks
// (channel, offset inside the plane) incrementally, so no division runs per vector. A
// vector may straddle one plane boundary (size2 >= VEC is required by the vector path).

struct ChanWalk {
  long long step_planes;  // (step * VEC) / size2
  int step_off;           // (step * VEC) % size2
  int step_ch;            // step_planes % C
};

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
};
template <typename T> struct ChanCoef<T, OP_MM_APPLY> {
  MmCoef c;
  __device__ __forceinline__ void load(const ChanArgs &a, int ch) {
    c.scale = a.mm_scale[ch];
    c.lo = a.mm_lo[ch];
    c.hi = a.mm_hi[ch];
  }
  __device__ __forceinline__ float apply(float v) const { return mm_apply(v, c); }
};

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
    chan_vec_kernel(const T *x, T *y, const long long total, const int C,
                    const int size2, const ChanWalk w, const ChanArgs a) {
  constexpr int S = Elem<T>::VEC;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  const long long n_vec = total / S;
  if (tid < n_vec) {
    const long long e0 = tid * S;
    const long long plane = e0 / size2;
    int off = (int)(e0 - plane * size2);
    int ch = (int)(plane % C);
    for (long long v = tid; v < n_vec; v += step) {
      float e[S];
      Vec16<T>::load_stream(x + v * S, e);
      ChanCoef<T, OP> c0;
      c0.load(a, ch);
      if (off + S <= size2) {
#pragma unroll
        for (int j = 0; j < S; ++j) e[j] = c0.apply(e[j]);
      } else {
        ChanCoef<T, OP> c1;
        c1.load(a, ch + 1 == C ? 0 : ch + 1);
#pragma unroll
        for (int j = 0; j < S; ++j) e[j] = (off + j < size2) ? c0.apply(e[j]) : c1.apply(e[j]);
      }
      Vec16<T>::store_stream(y + v * S, e);
      off += w.step_off;
      int carry = 0;
      if (off >= size2) {
        off -= size2;
        carry = 1;
      }
      ch += w.step_ch + carry;
      if (ch >= C) ch -= C;
    }
  }
  // scalar tail (total % VEC elements)
  for (long long i = n_vec * S + tid; i < total; i += step) {
    const int ch = (int)((i / size2) % C);
    ChanCoef<T, OP> c;
    c.load(a, ch);
    y[i] = Elem<T>::from_f32(c.apply(Elem<T>::to_f32(x[i])));
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
  if (vec) {
    const unsigned int grid = grid_for((total + S - 1) / S, 16);
    const long long step_elems = (long long)grid * kThreads * S;
    ChanWalk w;
    w.step_planes = step_elems / size2;
    w.step_off = (int)(step_elems % size2);
    w.step_ch = (int)(w.step_planes % C);
    chan_vec_kernel<T, OP><<<grid, kThreads, 0, stream>>>(x, y, total, (int)C, (int)size2, w, a);
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
    for (long long e0 = e_begin + (long long)threadIdx.x * S; e0 < e_end; e0 += (long long)blockDim.x * S) {
      if (e0 + S <= e_end) {
        float e[S];
        Vec16<T>::load_stream(x + e0, e);
        const long long plane = e0 / size2;
        const long long off = e0 - plane * size2;
        const int slot = (int)(plane - plane_first);
        if (off + S <= size2) {
          float lo = pinf, hi = ninf;
#pragma unroll
          for (int j = 0; j < S; ++j) {
            lo = fminf(lo, e[j]);
            hi = fmaxf(hi, e[j]);
          }
          atomicMin(&s_red[2 * slot], enc_ordered(lo));
          atomicMax(&s_red[2 * slot + 1], enc_ordered(hi));
        } else {
          // the vector straddles plane boundaries (possibly several when size2 < VEC)
#pragma unroll
          for (int j = 0; j < S; ++j) {
            const int sl = (int)((e0 + j) / size2 - plane_first);
            if (e[j] == e[j]) {
              atomicMin(&s_red[2 * sl], enc_ordered(e[j]));
              atomicMax(&s_red[2 * sl + 1], enc_ordered(e[j]));
            }
          }
        }
      } else {
        for (long long i = e0; i < e_end; ++i) {
          const float v = Elem<T>::to_f32(x[i]);
          const int sl = (int)(i / size2 - plane_first);
          if (v == v) {
            atomicMin(&s_red[2 * sl], enc_ordered(v));
            atomicMax(&s_red[2 * sl + 1], enc_ordered(v));
          }
        }
      }
    }
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
