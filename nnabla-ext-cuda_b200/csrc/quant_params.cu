// Host-side quantizer parameters: the members nnabla core's FixedPointQuantize /
// Pow2Quantize base classes derive in setup_impl, and the threshold table that lets the
// device reproduce round(log2f(|x|)) of the host libm with integer compares.
#include <cmath>
#include <cstring>
#include <mutex>

#include "dwbnq_internal.h"

namespace dwbnq {

void fpq_range(int sign, int n, float delta, float *mx, float *mn) {
  // max = (2^(n - sign) - 1) * delta, min = sign ? -max : 0.
  const int n_eff = sign ? n - 1 : n;
  const float m = (float)((1LL << n_eff) - 1) * delta;
  *mx = m;
  *mn = sign ? -m : 0.0f;
}

void pow2q_range(int sign, int with_zero, int n, int m, float *p_max, float *p_min, float *thr) {
  // n_eff = n - sign - with_zero; p_max = 2^m; p_min = 2^(m - (2^n_eff - 1));
  // pruning_threshold = p_min * 2^-0.5.
  int n_eff = n - (sign ? 1 : 0) - (with_zero ? 1 : 0);
  if (n_eff < 0) n_eff = 0;
  const double e = (n_eff >= 31) ? 2147483647.0 : (double)((1LL << n_eff) - 1);
  *p_max = (float)std::pow(2.0, (double)m);
  *p_min = (float)std::pow(2.0, (double)m - e);
  *thr = (float)((double)(*p_min) * std::pow(2.0, -0.5));
}

int fill_fpq(QuantArgs *q, int sign, int n, float delta) {
  if (n < 1 || n > 31 || (sign && n < 2))
    return fail(DWBNQ_ERR_INVALID_ARG, "FixedPointQuantize: bit width n=%d (sign=%d) out of range", n, sign);
  if (!(delta > 0.0f) || std::isinf(delta))
    return fail(DWBNQ_ERR_INVALID_ARG, "FixedPointQuantize: delta must be positive and finite");
  fpq_range(sign, n, delta, &q->fpq_max, &q->fpq_min);
  q->fpq_delta = delta;
  int ex = 0;
  const float mant = std::frexp(delta, &ex);
  const int n_eff = sign ? n - 1 : n;
  // delta = 2^(ex-1) exactly, far from the range ends, and max/delta = 2^n_eff - 1 < 2^22.
  q->fpq_fast = (mant == 0.5f && ex > -100 && ex < 100 && n_eff <= 22) ? 1 : 0;
  q->fpq_inv_delta = q->fpq_fast ? 1.0f / delta : 0.0f;
  q->fpq_nmagic_delta = q->fpq_fast ? -8388608.0f * delta : 0.0f;
  return DWBNQ_OK;
}

namespace {

uint32_t g_table[277];
int g_window = 0;
std::once_flag g_table_once;

inline float bits_to_float(uint32_t b) {
  float f;
  std::memcpy(&f, &b, 4);
  return f;
}

void build_table() {
  int window = 0;
  for (int e = -149; e <= 127; ++e) {
    uint32_t lo, hi;
    if (e >= -126) {
      lo = (uint32_t)(e + 127) << 23;
      hi = lo + (1u << 23);
    } else {
      lo = 1u << (e + 149);
      hi = 1u << (e + 150);
    }
    // smallest pattern in [lo, hi) whose rounded log2 reaches e + 1 (hi when none does)
    uint32_t a = lo, b = hi;
    while (a < b) {
      const uint32_t mid = a + (b - a) / 2;
      if (roundf(log2f(bits_to_float(mid))) >= (float)(e + 1)) b = mid;
      else a = mid + 1;
    }
    g_table[e + 149] = a;
    if (e >= -126) {
      const int d = (int)(a - lo) - 0x3504f3;
      const int ad = d < 0 ? -d : d;
      if (ad > window) window = ad;
    }
  }
  g_window = window + 2;
}

}  // namespace

const uint32_t *pow2_table_host() {
  std::call_once(g_table_once, build_table);
  return g_table;
}
int pow2_table_window() {
  std::call_once(g_table_once, build_table);
  return g_window;
}

uint32_t pow2_first_pattern_reaching(float v) {
  uint32_t lo = 1u, hi = 0x7f800000u;  // q(hi) = inf >= v
  while (lo < hi) {
    const uint32_t mid = lo + (hi - lo) / 2;
    if (powf(2.0f, roundf(log2f(bits_to_float(mid)))) >= v) hi = mid;
    else lo = mid + 1;
  }
  return lo;
}

int fill_pow2(QuantArgs *q, int sign, int with_zero, int n, int m, int device) {
  if (n < 1 || n > 31) return fail(DWBNQ_ERR_INVALID_ARG, "Pow2Quantize: bit width n=%d out of range", n);
  pow2q_range(sign, with_zero, n, m, &q->p_max, &q->p_min, &q->prune_thr);
  q->p_sign = sign ? 1 : 0;
  q->p_with_zero = with_zero ? 1 : 0;
  q->p_window = pow2_table_window();
  q->p_fast = q->p_min >= 2.350988701644575e-38f ? 1 : 0;  // 2^-125
  // The quantizer as a function of the magnitude pattern (see QuantArgs). first_reaching(v):
  // the smallest pattern a with 2^round(log2f(a)) >= v, by bisection with the host libm (the
  // rounded exponent is monotone in a).
  auto float_bits = [](float f) {
    uint32_t b;
    std::memcpy(&b, &f, 4);
    return b;
  };
  auto first_reaching = [&](float v) { return pow2_first_pattern_reaching(v); };
  q->p_lo_bits = float_bits(q->p_min);
  q->p_hi_bits = float_bits(q->p_max);
  q->p_prune_bits = 0u;
  if (with_zero && q->p_min > 0.0f) {
    const uint32_t a_min = first_reaching(q->p_min);  // patterns below it round below p_min
    const uint32_t thr = float_bits(q->prune_thr);
    q->p_prune_bits = a_min < thr ? a_min : thr;
  }
  if (sign) {
    q->p_neg_keep = 0xffffffffu;
    q->p_neg_xor = 0x80000000u;
  } else {
    q->p_neg_keep = 0u;
    q->p_neg_xor = with_zero ? 0u : float_bits(q->p_min);
  }
  // the pattern form needs p_min and p_max to be normal numbers with p_min <= p_max
  if (!(q->p_max < INFINITY) || !(q->p_min <= q->p_max)) q->p_fast = 0;
  return pow2_table_device(device, &q->p_table);
}

}  // namespace dwbnq
