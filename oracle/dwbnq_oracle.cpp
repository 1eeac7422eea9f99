// CPU oracle for the quantized depthwise-CNN inference path.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA path is compared
// against (tests, the smoke check and the bench's cpu_baseline / reference arm).
// No product code links, imports or calls it.
//
// PARITY UNPINNED: the CPU classes the results must equal
// (nbla::DepthwiseConvolution<float>, BatchNormalization, FixedPointQuantize,
// Pow2Quantize, MinMaxQuantize) live in sony/nnabla ("nnabla core", pinned by
// nnabla-ext-cuda as nnabla==<same version>, python/setup.py:57-60), which is not
// vendored in nnabla-ext-cuda and is not installed here. This file restates the
// arithmetic from the closest statement of it that IS available, the CUDA kernels of
// nnabla-ext-cuda that core's own tests hold equal to the CPU classes, and from
// nnabla's published function documentation for the parameters derived in core.
// Every function cites the lines it follows. The known-answer vectors derived by hand
// from those sources are in tests/golden/known_answers.json.
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
// (no -march=native: no FMA contraction, every binary op individually rounded).
//
// All entry points take `nthreads`: 1 = the plain single-threaded loops (how the
// reference CPU functions run), >1 = OpenMP over independent (n, c) planes or flat
// chunks; results do not depend on it.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <limits>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline int out_size(int in, int k, int s, int p, int d) {
  // Standard convolution output size (nnabla function docs, Convolution /
  // DepthwiseConvolution: L' = (L + 2p - d(k-1) - 1)/s + 1).
  return (in + 2 * p - d * (k - 1) - 1) / s + 1;
}

} // namespace

extern "C" {

int oracle_abi_version() { return 1; }

int oracle_max_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// ---------------------------------------------------------------------------------
// DepthwiseConvolution 2-D forward.
// Follows src/nbla/cuda/function/generic/depthwise_convolution.cu:84-111
// (forward_kernel_2d): the accumulator starts at bias[oc] (or 0), taps run ky outer /
// kx inner, out-of-bounds taps are SKIPPED (not added as zero), value += w * x with
// the product and the sum rounded separately. ic = oc / multiplier (:89).
// x [N, C, H, W], w [C*mult, kh, kw], b [C*mult] or null, y [N, C*mult, Ho, Wo].
// A 1-D convolution (forward_kernel_1d, :24-62) is the H = kh = 1 case.
// ---------------------------------------------------------------------------------
void oracle_dwconv_f32(const float *x, const float *w, const float *b, float *y,
                       int64_t N, int C, int H, int W, int kh, int kw, int sh, int sw,
                       int ph, int pw, int dh, int dw, int mult, int nthreads) {
  const int Ho = out_size(H, kh, sh, ph, dh);
  const int Wo = out_size(W, kw, sw, pw, dw);
  const int OC = C * mult;
  const int64_t planes = N * (int64_t)OC;
#pragma omp parallel for num_threads(nthreads) schedule(static) if (nthreads > 1)
  for (int64_t p = 0; p < planes; ++p) {
    const int oc = (int)(p % OC);
    const int64_t n = p / OC;
    const int ic = oc / mult;
    const float *xp = x + (n * C + ic) * (int64_t)H * W;
    const float *wp = w + (int64_t)oc * kh * kw;
    float *yp = y + p * (int64_t)Ho * Wo;
    for (int oy = 0; oy < Ho; ++oy) {
      for (int ox = 0; ox < Wo; ++ox) {
        float v = b ? b[oc] : 0.0f;
        for (int ky = 0; ky < kh; ++ky) {
          for (int kx = 0; kx < kw; ++kx) {
            const int iy = oy * sh + ky * dh - ph;
            const int ix = ox * sw + kx * dw - pw;
            if (iy >= 0 && iy < H && ix >= 0 && ix < W) {
              const float prod = wp[ky * kw + kx] * xp[(int64_t)iy * W + ix];
              v = v + prod;
            }
          }
        }
        yp[(int64_t)oy * Wo + ox] = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// BatchNormalization, inference mode (batch_stat = false).
// Follows include/nbla/cuda/function/kernel/batch_normalization.cuh:331-349
// (forward_global_kernel): per element, left to right,
//   stdvar = sqrt(rv[c] + eps);  y = (x - rm[c]) * gamma[c] / stdvar + beta[c]
// with gamma absent -> 1 and beta absent -> 0 (batch_normalization.cu:178-188).
// x is viewed as [size0, size1, size2] with the channel axis = size1
// (index i = i0*size1*size2 + i1*size2 + i2, .cuh:339-342).
// ---------------------------------------------------------------------------------
void oracle_bn_infer_f32(const float *x, const float *beta, const float *gamma,
                         const float *rm, const float *rv, float *y, int64_t size0,
                         int64_t size1, int64_t size2, float eps, int nthreads) {
  const int64_t planes = size0 * size1;
#pragma omp parallel for num_threads(nthreads) schedule(static) if (nthreads > 1)
  for (int64_t p = 0; p < planes; ++p) {
    const int64_t c = p % size1;
    const float mean = rm[c];
    const float stdvar = std::sqrt(rv[c] + eps);
    const float scale = gamma ? gamma[c] : 1.0f;
    const float bias = beta ? beta[c] : 0.0f;
    const float *xp = x + p * size2;
    float *yp = y + p * size2;
    for (int64_t i = 0; i < size2; ++i) {
      const float a = xp[i] - mean;
      const float m = a * scale;
      const float q = m / stdvar;
      yp[i] = q + bias;
    }
  }
}

// ---------------------------------------------------------------------------------
// FixedPointQuantize forward.
// Range (nnabla core, per the function documentation of F.fixed_point_quantize):
//   n_eff = sign ? n - 1 : n;  max = (2^n_eff - 1) * delta;  min = sign ? -max : 0.
// Element rule follows src/nbla/cuda/function/generic/fixed_point_quantize.cu:37-47:
//   x > max -> max; x < min -> min; else sign(x) * floor(|x| / delta + 0.5) * delta,
// where |x| / delta is a float division, "+ 0.5" and the product with delta are
// evaluated in double (0.5 is a double literal, :44) and the result is rounded to
// float once. sign(x) is (x < 0), so x = -0.0 gives +0.0 and a small negative x that
// rounds to zero gives -0.0.
// ---------------------------------------------------------------------------------
void oracle_fpq_params(int sign, int n, float delta, float *max_out, float *min_out) {
  const int n_eff = sign ? n - 1 : n;
  const float mx = (float)((1 << n_eff) - 1) * delta;
  *max_out = mx;
  *min_out = sign ? -mx : 0.0f;
}

void oracle_fpq_f32(const float *x, float *y, int64_t size, int sign, int n, float delta,
                    int nthreads) {
  float mx, mn;
  oracle_fpq_params(sign, n, delta, &mx, &mn);
#pragma omp parallel for num_threads(nthreads) schedule(static) if (nthreads > 1)
  for (int64_t i = 0; i < size; ++i) {
    const float xi = x[i];
    float r;
    if (xi > mx) {
      r = mx;
    } else if (xi < mn) {
      r = mn;
    } else {
      const bool neg = xi < 0.0f;
      const float ax = std::fabs(xi);
      const float t = ax / delta;
      const double q = std::floor((double)t + 0.5) * (double)delta;
      const float qf = (float)q;
      r = neg ? -qf : qf;
    }
    y[i] = r;
  }
}

// ---------------------------------------------------------------------------------
// Pow2Quantize forward.
// Parameters (nnabla core, per the function documentation of F.pow2_quantize):
//   n_eff = n - (sign ? 1 : 0) - (with_zero ? 1 : 0);
//   p_max = 2^m;  p_min = 2^(m - (2^n_eff - 1));  pruning_threshold = p_min * 2^-0.5.
// Element rule follows src/nbla/cuda/function/generic/pow2_quantize.cu:36-62:
//   q = powf(2, round(log2f(|x|)));  q > p_max -> p_max;
//   q < p_min -> with_zero ? (|x| < pruning_threshold ? 0 : p_min) : p_min;
//   sign: (sign ? (x<0 ? -q : q) : (x<0 ? (with_zero ? 0 : p_min) : q)).
// log2f / roundf / powf are the host libm's: their rounding at the binade mid-points
// IS the behaviour to match.
// ---------------------------------------------------------------------------------
void oracle_pow2q_params(int sign, int with_zero, int n, int m, float *p_max, float *p_min,
                         float *pruning_threshold) {
  int n_eff = n - (sign ? 1 : 0) - (with_zero ? 1 : 0);
  if (n_eff < 0) n_eff = 0;
  const double pmax = std::pow(2.0, (double)m);
  const double e = (n_eff >= 31) ? 2147483647.0 : (double)((1LL << n_eff) - 1);
  const double pmin = std::pow(2.0, (double)m - e);
  *p_max = (float)pmax;
  *p_min = (float)pmin;
  *pruning_threshold = (float)((double)(*p_min) * std::pow(2.0, -0.5));
}

void oracle_pow2q_f32(const float *x, float *y, int64_t size, int sign, int with_zero,
                      int n, int m, int nthreads) {
  float p_max, p_min, thr;
  oracle_pow2q_params(sign, with_zero, n, m, &p_max, &p_min, &thr);
#pragma omp parallel for num_threads(nthreads) schedule(static) if (nthreads > 1)
  for (int64_t i = 0; i < size; ++i) {
    const float xi = x[i];
    const bool neg = xi < 0.0f;
    const float ax = std::fabs(xi);
    float q = powf(2.0f, roundf(log2f(ax)));
    if (q > p_max) {
      q = p_max;
    } else if (q < p_min && with_zero) {
      q = ax < thr ? 0.0f : p_min;
    } else if (q < p_min) {
      q = p_min;
    }
    if (sign) {
      q = neg ? -q : q;
    } else if (with_zero) {
      q = neg ? 0.0f : q;
    } else {
      q = neg ? p_min : q;
    }
    y[i] = q;
  }
}

// round(log2f(|x|)) alone, for the exhaustive check of the product's threshold table.
void oracle_round_log2(const float *x, float *k, int64_t size, int nthreads) {
#pragma omp parallel for num_threads(nthreads) schedule(static) if (nthreads > 1)
  for (int64_t i = 0; i < size; ++i) k[i] = roundf(log2f(std::fabs(x[i])));
}

// ---------------------------------------------------------------------------------
// MinMaxQuantize forward on x viewed as [size0, C, size2] with per-channel ranges
// qr_min / qr_max / ql_min / ql_max of C elements (shape [1, C, 1, 1]).
// The two hooks follow src/nbla/cuda/function/generic/min_max_quantize.cu:
//   nudge_range (:29-37):  if qr_max - qr_min < eps: qr_max = qr_min + eps
//   nudge_qr_min_max (:39-61): zp_from_min = ql_min - qr_min / scale;
//     zp = zp_from_min <= ql_min ? ql_min : zp_from_min >= ql_max ? ql_max
//          : round(zp_from_min);  m' = (ql_min - zp) * scale; M' = (ql_max - zp) * scale
// The composite they plug into is nnabla core's; its order is restated from the
// function documentation of F.min_max_quantize:
//   x_min_max && !ema: qr_min = min over the reduced axes of x, qr_max = max (written
//     back into the qr_min / qr_max inputs);
//   x_min_max && ema : qr = decay * qr + (1 - decay) * batch statistic;
//   scale = (qr_max - qr_min) / (ql_max - ql_min);
//   y = round((min(max(x, m'), M') - m') / scale) * scale + m'
// with every binary op rounded to fp32 and round() = half away from zero
// (src/nbla/cuda/function/generic/round.cu:20).
// qr_min / qr_max are in/out. m_nudged / M_nudged / scale_out (C each, may be null)
// receive the per-channel intermediates for diagnosis.
// ---------------------------------------------------------------------------------
void oracle_minmax_reduce_f32(const float *x, float *mn, float *mx, int64_t size0, int C,
                              int64_t size2, int nthreads) {
#pragma omp parallel for num_threads(nthreads) schedule(static) if (nthreads > 1)
  for (int c = 0; c < C; ++c) {
    float lo = std::numeric_limits<float>::infinity();
    float hi = -std::numeric_limits<float>::infinity();
    for (int64_t i0 = 0; i0 < size0; ++i0) {
      const float *xp = x + (i0 * C + c) * size2;
      for (int64_t i = 0; i < size2; ++i) {
        const float v = xp[i];
        if (v < lo) lo = v;
        if (v > hi) hi = v;
      }
    }
    mn[c] = lo;
    mx[c] = hi;
  }
}

void oracle_minmaxq_ranges_f32(float *qr_min, float *qr_max, const float *ql_min,
                               const float *ql_max, float *scale_out, float *m_nudged,
                               float *M_nudged, int C, float eps) {
  for (int c = 0; c < C; ++c) {
    if (qr_max[c] - qr_min[c] < eps) qr_max[c] = qr_min[c] + eps;
    const float num = qr_max[c] - qr_min[c];
    const float den = ql_max[c] - ql_min[c];
    const float scale = num / den;
    const float zp_from_min = ql_min[c] - qr_min[c] / scale;
    float zp;
    if (zp_from_min <= ql_min[c]) {
      zp = ql_min[c];
    } else if (zp_from_min >= ql_max[c]) {
      zp = ql_max[c];
    } else {
      zp = roundf(zp_from_min);
    }
    scale_out[c] = scale;
    m_nudged[c] = (ql_min[c] - zp) * scale;
    M_nudged[c] = (ql_max[c] - zp) * scale;
  }
}

void oracle_minmaxq_apply_f32(const float *x, float *y, const float *scale,
                              const float *m_nudged, const float *M_nudged, int64_t size0,
                              int C, int64_t size2, int nthreads) {
  const int64_t planes = size0 * C;
#pragma omp parallel for num_threads(nthreads) schedule(static) if (nthreads > 1)
  for (int64_t p = 0; p < planes; ++p) {
    const int c = (int)(p % C);
    const float s = scale[c], lo = m_nudged[c], hi = M_nudged[c];
    const float *xp = x + p * size2;
    float *yp = y + p * size2;
    for (int64_t i = 0; i < size2; ++i) {
      float v = xp[i];
      v = v > lo ? v : lo; // max(x, m')
      v = v < hi ? v : hi; // min(., M')
      const float a = v - lo;
      const float q = a / s;
      const float r = roundf(q);
      const float t = r * s;
      yp[i] = t + lo;
    }
  }
}

void oracle_minmaxq_f32(const float *x, float *qr_min, float *qr_max, const float *ql_min,
                        const float *ql_max, float *y, int64_t size0, int C, int64_t size2,
                        float decay, int x_min_max, int ema, float eps, float *scale_out,
                        float *m_nudged_out, float *M_nudged_out, int nthreads) {
  float *scale = new float[C], *lo = new float[C], *hi = new float[C];
  if (x_min_max) {
    float *bmn = new float[C], *bmx = new float[C];
    oracle_minmax_reduce_f32(x, bmn, bmx, size0, C, size2, nthreads);
    for (int c = 0; c < C; ++c) {
      if (ema) {
        const float one_minus = 1.0f - decay;
        qr_min[c] = decay * qr_min[c] + one_minus * bmn[c];
        qr_max[c] = decay * qr_max[c] + one_minus * bmx[c];
      } else {
        qr_min[c] = bmn[c];
        qr_max[c] = bmx[c];
      }
    }
    delete[] bmn;
    delete[] bmx;
  }
  oracle_minmaxq_ranges_f32(qr_min, qr_max, ql_min, ql_max, scale, lo, hi, C, eps);
  oracle_minmaxq_apply_f32(x, y, scale, lo, hi, size0, C, size2, nthreads);
  if (scale_out) std::memcpy(scale_out, scale, sizeof(float) * C);
  if (m_nudged_out) std::memcpy(m_nudged_out, lo, sizeof(float) * C);
  if (M_nudged_out) std::memcpy(M_nudged_out, hi, sizeof(float) * C);
  delete[] scale;
  delete[] lo;
  delete[] hi;
}

} // extern "C"
