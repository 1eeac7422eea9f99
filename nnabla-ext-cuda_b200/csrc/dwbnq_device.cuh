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
  QM_MM_REDUCE = 4, // MinMaxQuantize, first pass: per-channel min/max only, no store
  QM_FPQ_LEAN = 5,  // FixedPointQuantize, the common case compiled without per-row tests (tiled family)
  QM_MM_REDUCE_STORE = 6  // MinMaxQuantize, first pass that also stores the fp32 activation (plane family)
};
// Whether a mode reduces to per-channel min / max, and whether it writes y.
__host__ __device__ constexpr bool qm_reduces(int qm) { return qm == QM_MM_REDUCE || qm == QM_MM_REDUCE_STORE; }
__host__ __device__ constexpr bool qm_stores(int qm) { return qm != QM_MM_REDUCE; }

// Kernel-argument block of the quantizers (passed by value; uniform -> constant bank).
struct QuantArgs {
  // FixedPointQuantize: range and step. `fpq_fast` is set by the host when delta is a
  // power of two in the normal range and max/delta < 2^22: then |x|/delta is the exact
  // product |x| * inv_delta and floor(t + 0.5) can be taken with two directed adds.
  float fpq_max, fpq_min, fpq_delta, fpq_inv_delta;
  float fpq_nmagic_delta;  // -2^23 * delta (fast form only)
  int fpq_fast;
  // Pow2Quantize.
  float p_max, p_min, prune_thr;
  int p_sign, p_with_zero;
  int p_window;               // |mantissa - sqrt2 mantissa| beyond which no table look-up is needed
  int p_fast;                 // p_min >= 2^-125: zeros and subnormals need no exact exponent
  const uint32_t *p_table;    // 277 thresholds, device memory
  // Pow2Quantize as a function of the magnitude bit pattern a = bits(|x|) alone (host-derived
  // from the same libm thresholds): a is clamped to [p_lo_bits, p_hi_bits] = bits(p_min),
  // bits(p_max) before the rounding (every pattern outside rounds to the same result as the
  // bound), a < p_prune_bits gives zero (with_zero: min(bits(pruning_threshold), first
  // pattern that rounds to p_min); otherwise 0 = never), and a negative input turns the
  // result q into (q & p_neg_keep) ^ p_neg_xor: -q (sign), +0.0 (unsigned, with_zero) or
  // p_min (unsigned, without zero).
  unsigned int p_lo_bits, p_hi_bits, p_prune_bits, p_neg_keep, p_neg_xor;
  // MinMaxQuantize second pass: per-channel fp32 arrays in the workspace.
  const float *mm_scale, *mm_lo, *mm_hi;
  // MinMaxQuantize first pass: per-channel order-encoded min / max in the workspace.
  unsigned int *mm_enc_min, *mm_enc_max;
};

// Bounds-checked debug build (make debug: -DDWBNQ_BOUNDS_CHECK, libdwbnq_debug.so): every global
// access whose index is computed by the kernel itself - not by the TMA / bulk-copy hardware,
// which clips by construction - is tested against its tensor's extent first. An index outside
// records 2 in the device flag and the access is skipped; nothing traps. In the normal build the
// macro is `true` and costs nothing.
#ifdef DWBNQ_BOUNDS_CHECK
__device__ __forceinline__ bool bounds_ok(long long i, long long n, int *flag) {
  if (i >= 0 && i < n) return true;
  if (flag) atomicExch(flag, 2);
  return false;
}
#define DWBNQ_IN_BOUNDS(index, extent, flag) ::dwbnq::bounds_ok((long long)(index), (long long)(extent), (flag))
#else
#define DWBNQ_IN_BOUNDS(index, extent, flag) true
#endif

// Programmatic dependent launch (no-ops when the launch does not carry the attribute): a grid
// lets its successor in the stream become resident early, and itself touches global memory
// only after its predecessor has completed and flushed.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

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
      // 0 <= t < 2^22: RD(RD(t + 0.5) + 2^23) - 2^23 == floor(t + 0.5); NaN propagates.
      const float u = __fmaf_rd(ax, q.fpq_inv_delta, 0.5f);
      k = __fsub_rn(__fadd_rd(u, 8388608.0f), 8388608.0f);
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
// 2^round(log2f(a)) for a bit pattern that needs the exact treatment: zero, subnormal,
// infinity / NaN, or a mantissa within `window` of the rounding threshold. Out of line: rare.
static __device__ __noinline__ float pow2_round_exact(unsigned int a, const uint32_t *table, int window) {
  if (a >= 0x7f800000u) return __uint_as_float(a);  // +inf stays +inf (clamped later); NaN passes through
  if (a == 0u) return 0.0f;                          // log2f(0) = -inf -> 2^-inf = 0
  int e;
  bool up;
  if (a >= 0x00800000u) {
    e = (int)(a >> 23) - 127;
    const int d = (int)(a & 0x007fffffu) - 0x3504f3;  // distance to the sqrt(2) mantissa
    if (d > window) up = true;
    else if (d < -window) up = false;
    else up = a >= __ldg(table + (e + 149));
  } else {
    e = 31 - __clz(a) - 149;
    up = a >= __ldg(table + (e + 149));
  }
  return pow2_of_int(e + (up ? 1 : 0));
}

// Clamp / prune / sign rules of the quantizer on q = 2^round(log2f(|x|)).
__device__ __forceinline__ float pow2_finish(float q, float x, float ax, const QuantArgs &p) {
  const bool neg = x < 0.0f;
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
// Common case, branch-free: away from the threshold the rounded exponent is e + 1 exactly
// when the mantissa is above sqrt(2)'s, i.e. adding (2^23 - 0x3504f3) carries into the
// exponent field. With p_min a normal number (p_fast) zeros and subnormals need no care
// either: whatever tiny power of two comes out is below p_min and the rules above decide on
// |x| alone. Infinity carries to infinity. Only NaN and the threshold window are `rare`.
__device__ __forceinline__ float pow2_round_fast(unsigned int a, const QuantArgs &p, bool *rare) {
  const int d = (int)(a & 0x007fffffu) - 0x3504f3;
  *rare = (unsigned int)(d + p.p_window) <= 2u * (unsigned int)p.p_window || a > 0x7f800000u || !p.p_fast;
  return __uint_as_float((a + 0x004afb0du) & 0x7f800000u);
}
__device__ __forceinline__ float pow2_apply(float x, const QuantArgs &p) {
  const unsigned int a = __float_as_uint(x) & 0x7fffffffu;
  bool rare;
  float q = pow2_round_fast(a, p, &rare);
  if (rare) q = pow2_round_exact(a, p.p_table, p.p_window);
  return pow2_finish(q, x, __uint_as_float(a), p);
}
// N values at once, branch-free in the common case. With the magnitude pattern clamped to
// [bits(p_min), bits(p_max)] first, the clamp rules of the quantizer need no test of their own
// (a pattern below bits(p_min) gives p_min unless it is pruned, one above bits(p_max) gives
// p_max, and the clamped bounds have a zero mantissa: never near a rounding threshold), the
// pruning rule is one compare on the pattern, and the sign rule one select. What does not fit
// this scheme - a NaN, a mantissa within the window around the rounding threshold, a p_min
// that is not a normal number - is detected for the whole group with a running minimum /
// maximum and re-evaluated value by value through pow2_apply (ONE branch per group).
template <int N>
__device__ __forceinline__ void pow2_apply_n(float *v, const QuantArgs &p) {
  unsigned int q[N];
  unsigned int near = 0xffffffffu, amax = 0u;
  const unsigned int w = (unsigned int)p.p_window;
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const unsigned int a = __float_as_uint(v[j]) & 0x7fffffffu;
    const unsigned int ac = min(max(a, p.p_lo_bits), p.p_hi_bits);
    const unsigned int t = ac + 0x004afb0du;  // carries into the exponent above sqrt(2)'s mantissa
    near = min(near, (t + w) & 0x007fffffu);  // <= 2w: within the window of the threshold
    amax = max(amax, a);
    q[j] = a < p.p_prune_bits ? 0u : (t & 0x7f800000u);
  }
  const bool any_rare = near <= 2u * w || amax > 0x7f800000u || !p.p_fast;
  if (any_rare) {
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = pow2_apply(v[j], p);
    return;
  }
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const unsigned int alt = (q[j] & p.p_neg_keep) ^ p.p_neg_xor;
    v[j] = __uint_as_float(v[j] < 0.0f ? alt : q[j]);
  }
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

// ---- packed fp32 pairs (sm_100 f32x2) ---------------------------------------------------
// mul / add / fma on two floats per instruction, each lane rounded to nearest exactly like
// the scalar instruction: twice the arithmetic per issue slot. A pair lives in an aligned
// 64-bit register pair; pack / unpack are register moves (free when the allocator can
// place the halves).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 splat2(float v) { return pack2(v, v); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
// Rounded product. Written as fma(a, b, -0.0): RN(a * b + (-0.0)) is RN(a * b) bit for
// bit (signed zeros included), and unlike mul.rn.f32x2 followed by add.rn.f32x2 - which
// ptxas 12.9 contracts into one fused multiply-add even under --fmad=false, measured on
// B200 - an fma feeding an add cannot be contracted.
// The -0.0 addend must be opaque to the compiler (with an immediate it folds the fma back
// into a multiply and then contracts again): negzero2() reads it from constant memory
// once and pins it in a register pair; callers hand that register to mul2.
static __constant__ unsigned long long k_negzero2 = 0x8000000080000000ull;
// Keeps a value in its registers: the compiler can neither rematerialise it (re-load it
// from shared / constant memory at each use) nor see through it.
__device__ __forceinline__ void pin(f32x2 &v) { asm volatile("" : "+l"(v)); }
__device__ __forceinline__ void pin(float &v) { asm volatile("" : "+f"(v)); }
__device__ __forceinline__ f32x2 negzero2() {
  f32x2 z = k_negzero2;
  pin(z);
  return z;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b, f32x2 nz) { return fma2(a, b, nz); }
// min / max that propagate NaN (x > hi ? hi : x keeps a NaN x, unlike fminf).
__device__ __forceinline__ float min_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float min3f(float a, float b, float c) {
  float r;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// ---- BatchNormalization on packed pairs ---------------------------------------------------
// Same four rounded steps as bn_apply. The IEEE division by the per-channel constant
// stdvar is evaluated as q0 = RN(a * r), then two residual corrections
// q <- RN(q + RN_exact(a - q * stdvar) * r) with r = RN(1 / stdvar): after the first
// correction q is within a fraction of an ulp of a / stdvar, and the second one then
// yields the correctly rounded quotient (Markstein's theorem) provided no intermediate
// leaves the normal range. That holds for 2^-100 < |a| < 2^100 and 2^-30 <= stdvar <=
// 2^30; everything else (zeros, infinities, NaN, extreme magnitudes) takes __fdiv_rn.
struct BnPacked {
  f32x2 nmean, scale, rcp, nstd, beta, nz;
  float stdvar, stdvar_hi;  // for the out-of-range path (low / high lane of a pair)
  float glo;     // lower guard on |a|: 2^-100, or +inf when stdvar itself is out of range
};
#define DWBNQ_DIV_GUARD_LO 7.888609052e-31f /* 2^-100 */
#define DWBNQ_DIV_GUARD_HI 1.267650600e30f  /* 2^100  */

__device__ __forceinline__ BnPacked make_bn_packed(const BnCoef &c, f32x2 nz) {
  BnPacked b;
  b.nmean = splat2(-c.mean);
  b.scale = splat2(c.scale);
  b.rcp = splat2(__frcp_rn(c.stdvar));
  b.nstd = splat2(-c.stdvar);
  b.beta = splat2(c.beta);
  b.nz = nz;
  b.stdvar = b.stdvar_hi = c.stdvar;
  const bool safe = c.stdvar >= 9.31322574615478515625e-10f && c.stdvar <= 1073741824.0f;
  b.glo = safe ? DWBNQ_DIV_GUARD_LO : __uint_as_float(0x7f800000u);
  return b;
}
// Two channels side by side: the low lane of every pair belongs to channel lo, the high lane
// to channel hi.
__device__ __forceinline__ BnPacked make_bn_packed2(const BnCoef &lo, const BnCoef &hi, f32x2 nz) {
  BnPacked b;
  b.nmean = pack2(-lo.mean, -hi.mean);
  b.scale = pack2(lo.scale, hi.scale);
  b.rcp = pack2(__frcp_rn(lo.stdvar), __frcp_rn(hi.stdvar));
  b.nstd = pack2(-lo.stdvar, -hi.stdvar);
  b.beta = pack2(lo.beta, hi.beta);
  b.nz = nz;
  b.stdvar = lo.stdvar;
  b.stdvar_hi = hi.stdvar;
  const bool safe = fminf(lo.stdvar, hi.stdvar) >= 9.31322574615478515625e-10f &&
                    fmaxf(lo.stdvar, hi.stdvar) <= 1073741824.0f;  // (a NaN fails both)
  b.glo = (safe && lo.stdvar == lo.stdvar && hi.stdvar == hi.stdvar) ? DWBNQ_DIV_GUARD_LO
                                                                     : __uint_as_float(0x7f800000u);
  return b;
}

// The IEEE quotients of the out-of-range path, out of line: the path is cold and the inline
// expansion of a correctly rounded division is several times the size of the whole BN step.
static __device__ __noinline__ f32x2 bn_div_cold(f32x2 a, float stdvar_lo, float stdvar_hi) {
  float lo, hi;
  unpack2(a, lo, hi);
  return pack2(__fdiv_rn(lo, stdvar_lo), __fdiv_rn(hi, stdvar_hi));
}

// In-place BN of NP pairs.
template <int NP>
__device__ __forceinline__ void bn_apply_packed(f32x2 *v, const BnPacked &b) {
  f32x2 a[NP];
  float mx = 0.0f, mn = __uint_as_float(0x7f800000u);
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    a[p] = mul2(add2(v[p], b.nmean), b.scale, b.nz);
    float lo, hi;
    unpack2(a[p], lo, hi);
    mx = max3f(mx, fabsf(lo), fabsf(hi));
    mn = min3f(mn, fabsf(lo), fabsf(hi));
    f32x2 q = mul2(a[p], b.rcp, b.nz);
    f32x2 e = fma2(q, b.nstd, a[p]);
    q = fma2(e, b.rcp, q);
    e = fma2(q, b.nstd, a[p]);
    v[p] = fma2(e, b.rcp, q);
  }
  if (!(mn > b.glo && mx < DWBNQ_DIV_GUARD_HI)) {
#pragma unroll
    for (int p = 0; p < NP; ++p) v[p] = bn_div_cold(a[p], b.stdvar, b.stdvar_hi);
  }
#pragma unroll
  for (int p = 0; p < NP; ++p) v[p] = add2(v[p], b.beta);
}

// FixedPointQuantize, power-of-two delta, one value, five instructions when unsigned:
//  - clamp first: max and min lie on the grid, so clamping commutes with the rounding, and
//    min.NaN / max.NaN keep a NaN;
//  - u = RD(|xc| * inv_delta + 0.5) in one round-down fma (the product is exact);
//  - kp = RD(u + 2^23) = floor(u) + 2^23;
//  - v = kp * delta - 2^23 * delta in one fma: both terms and the result k * delta are
//    exactly representable, so nothing is rounded.
template <bool SIGNED>
__device__ __forceinline__ float fpq_apply_fast(float x, const QuantArgs &q) {
  const float xc = max_nan(min_nan(x, q.fpq_max), q.fpq_min);
  // unsigned: xc >= 0 (or -0.0, which the arithmetic below maps to +0.0 as well)
  const float u = __fmaf_rd(SIGNED ? fabsf(xc) : xc, q.fpq_inv_delta, 0.5f);
  const float kp = __fadd_rd(u, 8388608.0f);
  const float v = __fmaf_rn(kp, q.fpq_delta, q.fpq_nmagic_delta);
  return (SIGNED && xc < 0.0f) ? -v : v;
}

// The same on a pair: the two directed-rounding steps and the final fma run packed (the
// packed instructions take every rounding mode), the NaN-keeping clamp stays scalar.
__device__ __forceinline__ f32x2 fma2_rm(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rm.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 add2_rm(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
struct FpqPacked {
  f32x2 inv, half, magic, delta, nmagic;
};
__device__ __forceinline__ FpqPacked make_fpq_packed(const QuantArgs &q) {
  FpqPacked f;
  f.inv = splat2(q.fpq_inv_delta);
  f.half = splat2(0.5f);
  f.magic = splat2(8388608.0f);
  f.delta = splat2(q.fpq_delta);
  f.nmagic = splat2(q.fpq_nmagic_delta);
  return f;
}
// Unsigned fast form on two values (x0, x1) -> pair.
__device__ __forceinline__ f32x2 fpq_apply_fast_unsigned2(float x0, float x1, const QuantArgs &q,
                                                          const FpqPacked &f) {
  const float c0 = max_nan(min_nan(x0, q.fpq_max), q.fpq_min);
  const float c1 = max_nan(min_nan(x1, q.fpq_max), q.fpq_min);
  const f32x2 u = fma2_rm(pack2(c0, c1), f.inv, f.half);
  const f32x2 kp = add2_rm(u, f.magic);
  return fma2(kp, f.delta, f.nmagic);
}

// One epilogue for all modes (QM_MM_REDUCE does not come here).
template <int QM>
__device__ __forceinline__ float quant_apply(float v, const QuantArgs &q, const MmCoef &mm) {
  if (QM == QM_FPQ || QM == QM_FPQ_LEAN) return fpq_apply(v, q);
  if (QM == QM_POW2) return pow2_apply(v, q);
  if (QM == QM_MM_APPLY) return mm_apply(v, mm);
  return v;
}

}  // namespace dwbnq
