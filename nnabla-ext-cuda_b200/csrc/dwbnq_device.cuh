// Device-side building blocks shared by every kernel of the path: element traits,
// vector memory access, and the exact (individually rounded, never contracted)
// arithmetic of BatchNormalization inference and the three quantizers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dwbnq {

// Quantizer epilogue selected at compile time.
enum QMode : int {
  QM_NONE = 0,      // store the (BN'd) convolution result
  QM_FPQ = 1,       // FixedPointQuantize
  QM_POW2 = 2,      // Pow2Quantize
  QM_MM_APPLY = 3,  // MinMaxQuantize, second pass: quantize with per-channel ranges
  QM_MM_REDUCE = 4  // MinMaxQuantize, first pass: per-channel min/max only, no store
};

// Kernel-argument block of the quantizers (passed by value; uniform -> constant bank).
struct QuantArgs {
  // FixedPointQuantize: range and step. `fpq_fast` is set by the host when delta is a
  // power of two in the normal range and max/delta < 2^22: then |x|/delta is the exact
  // product |x| * inv_delta and floor(t + 0.5) can be taken with two directed adds.
  float fpq_max, fpq_min, fpq_delta, fpq_inv_delta;
  int fpq_fast;
  // Pow2Quantize.
  float p_max, p_min, prune_thr;
  int p_sign, p_with_zero;
  int p_window;               // |mantissa - sqrt2 mantissa| beyond which no table look-up is needed
  const uint32_t *p_table;    // 277 thresholds, device memory
  // MinMaxQuantize second pass: per-channel fp32 arrays in the workspace.
  const float *mm_scale, *mm_lo, *mm_hi;
  // MinMaxQuantize first pass: per-channel order-encoded min / max in the workspace.
  unsigned int *mm_enc_min, *mm_enc_max;
};

// ---- element traits -----------------------------------------------------------------

template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int VEC = 4;  // elements per 16 bytes
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__half> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};

// 16-byte vector of VEC elements <-> VEC floats.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static __device__ __forceinline__ void load(const float *p, float *v) {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float *p, const float *v) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  // streaming variants for global memory touched exactly once
  static __device__ __forceinline__ void load_stream(const float *p, float *v) {
    const float4 t = __ldcs(reinterpret_cast<const float4 *>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store_stream(float *p, const float *v) {
    __stcs(reinterpret_cast<float4 *>(p), make_float4(v[0], v[1], v[2], v[3]));
  }
};
template <> struct Vec16<__half> {
  static __device__ __forceinline__ void unpack(const uint4 &t, float *v) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float *v) {
    uint4 t;
    __half2 *h = reinterpret_cast<__half2 *>(&t);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    return t;
  }
  static __device__ __forceinline__ void load(const __half *p, float *v) {
    unpack(*reinterpret_cast<const uint4 *>(p), v);
  }
  static __device__ __forceinline__ void store(__half *p, const float *v) {
    *reinterpret_cast<uint4 *>(p) = pack(v);
  }
  static __device__ __forceinline__ void load_stream(const __half *p, float *v) {
    unpack(__ldcs(reinterpret_cast<const uint4 *>(p)), v);
  }
  static __device__ __forceinline__ void store_stream(__half *p, const float *v) {
    __stcs(reinterpret_cast<uint4 *>(p), pack(v));
  }
};

// ---- order-preserving float <-> uint encoding for atomic min / max ------------------

__device__ __forceinline__ unsigned int enc_ordered(float f) {
  const unsigned int b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ __forceinline__ unsigned int enc_ordered_bits(unsigned int b) {
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float dec_ordered(unsigned int u) {
  const unsigned int b = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
  return __uint_as_float(b);
}
// Identity elements: +inf for the running minimum, -inf for the running maximum.
#define DWBNQ_ENC_POS_INF 0xff800000u /* enc_ordered(+inf) */
#define DWBNQ_ENC_NEG_INF 0x007fffffu /* enc_ordered(-inf) */

// ---- BatchNormalization inference ----------------------------------------------------
// y = (x - mean) * scale / stdvar + beta, left to right, each op rounded once; the
// division is IEEE (include/nbla/cuda/function/kernel/batch_normalization.cuh:343-347).
struct BnCoef {
  float mean, scale, stdvar, beta;
};
__device__ __forceinline__ float bn_apply(float x, const BnCoef &c) {
  const float a = __fsub_rn(x, c.mean);
  const float m = __fmul_rn(a, c.scale);
  const float q = __fdiv_rn(m, c.stdvar);
  return __fadd_rn(q, c.beta);
}
// stdvar = sqrt(var + eps): one rounded add, one IEEE square root.
__device__ __forceinline__ float bn_stdvar(float var, float eps) {
  return __fsqrt_rn(__fadd_rn(var, eps));
}

// ---- FixedPointQuantize --------------------------------------------------------------
// x > max -> max; x < min -> min; else sign(x) * floor(|x|/delta + 0.5) * delta with the
// "+ 0.5", the floor and the product exact in double and one rounding to float
// (src/nbla/cuda/function/generic/fixed_point_quantize.cu:37-47).
// In float: s = RD(t + 0.5) has floor(s) == floor(t + 0.5) exactly (s <= t + 0.5, and
// any integer <= t + 0.5 is representable, hence <= s); r = floor(s) is an exactly
// representable integer, so RN(r * delta) in float equals the double product rounded
// to float.
__device__ __forceinline__ float fpq_apply(float x, const QuantArgs &q) {
  float r;
  if (x > q.fpq_max) {
    r = q.fpq_max;
  } else if (x < q.fpq_min) {
    r = q.fpq_min;
  } else {
    const float ax = fabsf(x);
    float k;
    if (q.fpq_fast) {
      const float t = __fmul_rn(ax, q.fpq_inv_delta);
      const float s = __fadd_rd(t, 0.5f);
      // 0 <= s < 2^22: RD(s + 2^23) - 2^23 == floor(s); NaN propagates.
      k = __fsub_rn(__fadd_rd(s, 8388608.0f), 8388608.0f);
    } else {
      const float t = __fdiv_rn(ax, q.fpq_delta);
      k = floorf(__fadd_rd(t, 0.5f));
    }
    const float v = __fmul_rn(k, q.fpq_delta);
    r = (x < 0.0f) ? -v : v;
  }
  return r;
}

// ---- Pow2Quantize --------------------------------------------------------------------
// q = 2^round(log2f(|x|)) with the HOST libm's rounding of log2f, reproduced through
// per-binade thresholds on the bit pattern (table index e + 149, e = floor(log2|x|)):
// round(log2f) is e below the threshold and e + 1 from it on. Then the clamp / prune /
// sign rules of src/nbla/cuda/function/generic/pow2_quantize.cu:41-62.
__device__ __forceinline__ float pow2_of_int(int k) {
  // 2^k as powf(2, k) returns it in float: inf above 127, denormals down to 2^-149.
  if (k > 127) return __uint_as_float(0x7f800000u);
  if (k >= -126) return __uint_as_float((unsigned int)(k + 127) << 23);
  if (k >= -149) return __uint_as_float(1u << (k + 149));
  return 0.0f;
}
__device__ __forceinline__ float pow2_apply(float x, const QuantArgs &p) {
  const unsigned int a = __float_as_uint(x) & 0x7fffffffu;
  const float ax = __uint_as_float(a);
  const bool neg = x < 0.0f;
  float q;
  if (a >= 0x7f800000u) {
    q = ax;  // +inf stays +inf (clamped below); NaN fails every compare and passes through
  } else if (a == 0u) {
    q = 0.0f;  // log2f(0) = -inf -> 2^-inf = 0
  } else {
    int e;
    bool up;
    if (a >= 0x00800000u) {
      e = (int)(a >> 23) - 127;
      const int d = (int)(a & 0x007fffffu) - 0x3504f3;  // distance to the sqrt(2) mantissa
      if (d > p.p_window) up = true;
      else if (d < -p.p_window) up = false;
      else up = a >= __ldg(p.p_table + (e + 149));
    } else {
      e = 31 - __clz(a) - 149;
      up = a >= __ldg(p.p_table + (e + 149));
    }
    q = pow2_of_int(e + (up ? 1 : 0));
  }
  if (q > p.p_max) {
    q = p.p_max;
  } else if (q < p.p_min && p.p_with_zero) {
    q = ax < p.prune_thr ? 0.0f : p.p_min;
  } else if (q < p.p_min) {
    q = p.p_min;
  }
  if (p.p_sign) {
    q = neg ? -q : q;
  } else if (p.p_with_zero) {
    q = neg ? 0.0f : q;
  } else {
    q = neg ? p.p_min : q;
  }
  return q;
}

// ---- MinMaxQuantize, quantize step ---------------------------------------------------
// y = round((min(max(x, m'), M') - m') / scale) * scale + m', five rounded fp32 ops with
// round() = half away from zero (src/nbla/cuda/function/generic/round.cu:20).
struct MmCoef {
  float scale, lo, hi;
};
__device__ __forceinline__ float mm_apply(float x, const MmCoef &c) {
  float v = x > c.lo ? x : c.lo;
  v = v < c.hi ? v : c.hi;
  const float a = __fsub_rn(v, c.lo);
  const float q = __fdiv_rn(a, c.scale);
  const float r = roundf(q);
  const float t = __fmul_rn(r, c.scale);
  return __fadd_rn(t, c.lo);
}

// One epilogue for all modes (QM_MM_REDUCE does not come here).
template <int QM>
__device__ __forceinline__ float quant_apply(float v, const QuantArgs &q, const MmCoef &mm) {
  if (QM == QM_FPQ) return fpq_apply(v, q);
  if (QM == QM_POW2) return pow2_apply(v, q);
  if (QM == QM_MM_APPLY) return mm_apply(v, mm);
  return v;
}

}  // namespace dwbnq
