// Training side of the path: straight-through backward of FixedPointQuantize and
// Pow2Quantize, and the three gradients of DepthwiseConvolution.
//
// What each kernel computes is the reference's backward
// (src/nbla/cuda/function/generic/fixed_point_quantize.cu:63-128, pow2_quantize.cu:79-160,
// depthwise_convolution.cu:114-366 and 492-650):
//  * quantizers: dx (+)= c * dy with c = 1, except (fine-grained STE) c = 0 where the forward
//    clipped: FixedPointQuantize x > max or x < min (then dx is left alone when accumulating,
//    zeroed otherwise); Pow2Quantize 2^round(log2f|x|) > p_max, or x < 0 for the unsigned form.
//    Element-wise, one rounded operation per element: bit-identical to the CPU loop.
//  * dw-conv input gradient: dx[n,c,iy,ix] += sum over ky, kx (ascending), m of
//    w[c*mult+m][ky][kx] * dy[n, c*mult+m, oy, ox] with oy*s = iy + p - ky*d (taps that do not
//    land on an output are skipped); the sum starts at +0, runs in that order with product and
//    sum rounded separately, and is added to the gradient (to +0 when not accumulating): the
//    order of the reference loop, so the result is bit-identical to the CPU restatement.
//  * dw-conv weight and bias gradients: dw[oc][ky][kx] += sum over n, oy, ox of
//    x[n, oc/mult, oy*s + ky*d - p, ox*s + kx*d - p] * dy[n,oc,oy,ox]; db[oc] += sum of dy.
//    The reference reduces with a block tree (blockReduceSum), this kernel with per-thread
//    partial sums, a warp and block reduction and one atomic add per CTA: the association of
//    the fp32 sum differs (from the reference's as from the CPU loop's), so these two
//    gradients are compared within a tolerance, not bit for bit.
// All kernels are bandwidth-shaped: 16-byte accesses where the layout allows, grids sized from
// the SM count.
#include <cstdlib>
#include <cstring>

#include "dwbnq_internal.h"

namespace dwbnq {

namespace {

constexpr int kThreads = 256;

unsigned int grid_for(long long items, int per_sm) {
  long long blocks = (items + kThreads - 1) / kThreads;
  const long long cap = (long long)sm_count(-1) * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned int)blocks;
}
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) % 16) == 0; }

// DWBNQ_BWD_INPUT_DIRECT=1 keeps every input gradient on the direct kernel (the reference's
// summation order, bit-identical to the CPU loop); read once.
bool bwd_input_by_forward_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("DWBNQ_BWD_INPUT_DIRECT");
    return !(e && e[0] == '1');
  }();
  return on;
}

// ---- straight-through backward of the quantizers ------------------------------------------
// MODE 0: pass-through (ste_fine_grained = false); 1: FixedPointQuantize mask; 2: Pow2 mask.
struct SteArgs {
  float fpq_max, fpq_min;
  unsigned int pow2_first_above;  // smallest |x| pattern whose rounded power of two exceeds p_max
  int pow2_sign;
};

template <int MODE, bool ACCUM>
__device__ __forceinline__ float ste_one(float x, float dy, float dx_old, const SteArgs &s) {
  if (MODE == 0) return ACCUM ? __fadd_rn(dx_old, dy) : dy;
  if (MODE == 1) {
    if (x > s.fpq_max || x < s.fpq_min) return ACCUM ? dx_old : 0.0f;
    return ACCUM ? __fadd_rn(dx_old, dy) : dy;
  }
  // Pow2: c = 1; q > p_max -> 0 (a NaN x compares false); unsigned and x < 0 -> 0; dx (+)= c * dy
  const unsigned int a = __float_as_uint(x) & 0x7fffffffu;
  float c = (a >= s.pow2_first_above && a <= 0x7f800000u) ? 0.0f : 1.0f;
  if (!s.pow2_sign && x < 0.0f) c = 0.0f;
  const float g = __fmul_rn(c, dy);
  return ACCUM ? __fadd_rn(dx_old, g) : g;
}

template <typename T, int MODE, bool ACCUM>
__global__ void __launch_bounds__(kThreads)
    ste_backward_kernel(const T *__restrict__ x, const T *__restrict__ dy, T *dx, long long size, int vec_ok,
                        SteArgs s) {
  constexpr int S = Elem<T>::VEC;
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  const long long n_vec = vec_ok ? size / S : 0;
  for (long long v = tid; v < n_vec; v += step) {
    float ex[S], ey[S], eo[S];
    if (MODE != 0) Vec16<T>::load_stream(x + v * S, ex);
    Vec16<T>::load_stream(dy + v * S, ey);
    if (ACCUM) Vec16<T>::load(dx + v * S, eo);
#pragma unroll
    for (int j = 0; j < S; ++j) eo[j] = ste_one<MODE, ACCUM>(MODE != 0 ? ex[j] : 0.0f, ey[j], ACCUM ? eo[j] : 0.0f, s);
    Vec16<T>::store_stream(dx + v * S, eo);
  }
  for (long long i = n_vec * S + tid; i < size; i += step) {
    const float xo = MODE != 0 ? Elem<T>::to_f32(x[i]) : 0.0f;
    const float old = ACCUM ? Elem<T>::to_f32(dx[i]) : 0.0f;
    dx[i] = Elem<T>::from_f32(ste_one<MODE, ACCUM>(xo, Elem<T>::to_f32(dy[i]), old, s));
  }
}

template <typename T>
cudaError_t launch_ste_t(int mode, int accum, const T *x, const T *dy, T *dx, long long size, const SteArgs &s,
                         cudaStream_t stream) {
  const int S = Elem<T>::VEC;
  const int vec_ok = aligned16(dy) && aligned16(dx) && (mode == 0 || aligned16(x));
  const dim3 grid(grid_for((size + S - 1) / S, 16)), block(kThreads);
#define DWBNQ_STE(M, A) \
  return launch_pdl(ste_backward_kernel<T, M, A>, grid, block, 0, stream, x, dy, dx, size, vec_ok, s)
  if (mode == 0) {
    if (accum) DWBNQ_STE(0, true);
    DWBNQ_STE(0, false);
  }
  if (mode == 1) {
    if (accum) DWBNQ_STE(1, true);
    DWBNQ_STE(1, false);
  }
  if (accum) DWBNQ_STE(2, true);
  DWBNQ_STE(2, false);
#undef DWBNQ_STE
}

// ---- DepthwiseConvolution: input gradient ------------------------------------------------------
struct BwdArgs {
  const void *x, *w, *dy;
  void *dx, *dw, *db;
  long long n;
  int C, H, W, OC, Ho, Wo;
  int kh, kw, sh, sw, ph, pw, dh, dw_, mult;
};

// One thread per input-gradient element, in the reference's order (ky outer, kx inner,
// multiplier innermost). K > 0: square K x K kernel, multiplier 1, no dilation, stride S (1 or
// 2), everything about the taps known at compile time (no division: a tap lands on an output
// when iy + p - ky is a non-negative multiple of S inside the output). K == 0: any geometry.
// A CTA owns a run of consecutive elements; the plane and the position inside it come from one
// 64-bit division per CTA and two 32-bit ones per element.
template <typename T, int K, int S, bool ACCUM>
__global__ void __launch_bounds__(kThreads)
    dwconv_bwd_input_kernel(const BwdArgs a, const long long total, const int per_cta) {
  const T *w = static_cast<const T *>(a.w);
  const T *dy = static_cast<const T *>(a.dy);
  T *dx = static_cast<T *>(a.dx);
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const int HW = a.H * a.W;
  const int plane_out = a.Ho * a.Wo;
  for (long long base = (long long)blockIdx.x * per_cta; base < total; base += (long long)gridDim.x * per_cta) {
    const long long plane0 = base / HW;
    const int rem0 = (int)(base - plane0 * HW);
    const int n_here = (int)(total - base < per_cta ? total - base : per_cta);
    for (int t = threadIdx.x; t < n_here; t += kThreads) {
      const int idx = rem0 + t;
      const int dp = idx / HW;
      const int e = idx - dp * HW;
      const int iy = e / a.W, ix = e - iy * a.W;
      const long long plane = plane0 + dp;  // = n * C + c
      const int c = (int)(plane % a.C);
      float value = 0.0f;
      if (K > 0) {
        const T *dyp = dy + plane * plane_out;  // multiplier 1: output plane index = input plane index
        const T *wp = w + (long long)c * K * K;
#pragma unroll
        for (int ky = 0; ky < K; ++ky) {
          const int ty = iy + a.ph - ky;
          const int oy = S == 1 ? ty : ty >> 1;
          const bool row_ok = (S == 1 || (ty & 1) == 0) && (unsigned int)oy < (unsigned int)a.Ho;
#pragma unroll
          for (int kx = 0; kx < K; ++kx) {
            const int tx = ix + a.pw - kx;
            const int ox = S == 1 ? tx : tx >> 1;
            if (row_ok && (S == 1 || (tx & 1) == 0) && (unsigned int)ox < (unsigned int)a.Wo)
              value = __fadd_rn(value, __fmul_rn(Elem<T>::to_f32(wp[ky * K + kx]), Elem<T>::to_f32(dyp[oy * a.Wo + ox])));
          }
        }
      } else {
        const long long n = plane / a.C;
        const int oc0 = c * a.mult;
        const T *dyp = dy + (n * a.OC + oc0) * plane_out;
        const T *wp = w + (long long)oc0 * a.kh * a.kw;
        for (int ky = 0; ky < a.kh; ++ky) {
          const int ty = iy + a.ph - ky * a.dh;
          // C division truncates toward zero: the reference tests (t - (t / s) * s == 0) and then
          // the range, so a negative multiple of the stride passes the first test and fails the second
          const int oy = ty / a.sh;
          const bool row_ok = (ty - oy * a.sh == 0) && oy >= 0 && oy < a.Ho;
          for (int kx = 0; kx < a.kw; ++kx) {
            const int tx = ix + a.pw - kx * a.dw_;
            const int ox = tx / a.sw;
            if (row_ok && (tx - ox * a.sw == 0) && ox >= 0 && ox < a.Wo) {
              const int off = oy * a.Wo + ox;
              const int wi = ky * a.kw + kx;
              for (int m = 0; m < a.mult; ++m)
                value = __fadd_rn(value, __fmul_rn(Elem<T>::to_f32(wp[m * a.kh * a.kw + wi]),
                                                   Elem<T>::to_f32(dyp[(long long)m * plane_out + off])));
            }
          }
        }
      }
      const long long o = base + t;
      const float old = ACCUM ? Elem<T>::to_f32(dx[o]) : 0.0f;
      dx[o] = Elem<T>::from_f32(__fadd_rn(old, value));
    }
  }
}

// ---- DepthwiseConvolution: weight and bias gradients ---------------------------------------------
// CTA = one output channel x one slice of the batch; a warp takes one image of the slice at a
// time and its lanes walk over the output positions of that plane 32 at a time, so dy and the
// K x K input values under each position are read as coalesced rows (the nine or twenty-five
// shifted reads of a row hit L1). Each lane accumulates x * dy for every tap in registers, plus
// dy for the bias. Positions whose K x K window lies inside the image (all but a border) are
// enumerated on their own and load without tests; the border positions test every tap. Warp shuffles and shared memory reduce the CTA's partial sums, which are added to the
// gradients with one atomic per value: the gradients must be zero (or hold the value to
// accumulate onto) when the kernel starts.
template <typename T, int K, int S>
__global__ void __launch_bounds__(kThreads, K == 3 ? 4 : 2)
    dwconv_bwd_weights_kernel(const BwdArgs a, const int slices) {
  constexpr int KK = K * K;
  __shared__ float red[kThreads / 32][KK + 1];
  const T *x = static_cast<const T *>(a.x);
  const T *dy = static_cast<const T *>(a.dy);
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const int oc = blockIdx.x / slices;
  const int slice = blockIdx.x % slices;
  const int ic = oc / a.mult;
  const int plane_out = a.Ho * a.Wo;
  const int plane_in = a.H * a.W;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // images [n0, n1) of this slice
  const long long per = (a.n + slices - 1) / slices;
  const long long n0 = (long long)slice * per;
  const long long n1 = n0 + per < a.n ? n0 + per : a.n;
  float acc[KK];
#pragma unroll
  for (int i = 0; i < KK; ++i) acc[i] = 0.0f;
  float bsum = 0.0f;
  // output rows / columns whose window lies wholly inside the image
  const int oy_lo = min(a.Ho, (a.ph + S - 1) / S), ox_lo = min(a.Wo, (a.pw + S - 1) / S);
  const int oy_hi = max(oy_lo, min(a.Ho, a.H - K + a.ph >= 0 ? (a.H - K + a.ph) / S + 1 : 0));
  const int ox_hi = max(ox_lo, min(a.Wo, a.W - K + a.pw >= 0 ? (a.W - K + a.pw) / S + 1 : 0));
  const int w_int = ox_hi - ox_lo, n_int = (oy_hi - oy_lo) * w_int;
  const int n_top = oy_lo * a.Wo, n_bot = (a.Ho - oy_hi) * a.Wo;
  const int w_edge = a.Wo - w_int, n_edge = n_top + n_bot + (oy_hi - oy_lo) * w_edge;
  for (long long n = n0 + warp; n < n1; n += kThreads / 32) {
    const T *dyp = dy + (n * a.OC + oc) * plane_out;
    const T *xp = x + (n * a.C + ic) * plane_in;
    // Interior positions (the whole K x K window inside the image: rows [oy_lo, oy_hi), columns
    // [ox_lo, ox_hi)): loads without any test, two positions per trip so that their loads are in
    // flight together.
    for (int idx = lane; idx < n_int; idx += 64) {
      float g[2], xv[2][KK];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int iu = idx + 32 * u;
        const bool live = iu < n_int;
        const int ic2 = live ? iu : idx;
        const int r = ic2 / w_int;
        const int oy = oy_lo + r, ox = ox_lo + (ic2 - r * w_int);
        g[u] = live ? Elem<T>::to_f32(dyp[oy * a.Wo + ox]) : 0.0f;
        const T *xw = xp + (oy * S - a.ph) * a.W + (ox * S - a.pw);
#pragma unroll
        for (int ky = 0; ky < K; ++ky) {
#pragma unroll
          for (int kx = 0; kx < K; ++kx) xv[u][ky * K + kx] = Elem<T>::to_f32(xw[ky * a.W + kx]);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        bsum += g[u];
#pragma unroll
        for (int i = 0; i < KK; ++i) acc[i] = fmaf(xv[u][i], g[u], acc[i]);
      }
    }
    // Border positions: rows above / below the interior in full, and the columns left / right of
    // it on the interior rows; every tap tested.
    for (int e = lane; e < n_edge; e += 32) {
      int oy, ox;
      if (e < n_top) {
        oy = e / a.Wo;
        ox = e - oy * a.Wo;
      } else if (e < n_top + n_bot) {
        const int t = e - n_top;
        oy = oy_hi + t / a.Wo;
        ox = t - (t / a.Wo) * a.Wo;
      } else {
        const int t = e - n_top - n_bot;
        const int r = t / w_edge, j = t - r * w_edge;
        oy = oy_lo + r;
        ox = j < ox_lo ? j : ox_hi + (j - ox_lo);
      }
      const float g = Elem<T>::to_f32(dyp[oy * a.Wo + ox]);
      bsum += g;
      const int iy0 = oy * S - a.ph, ix0 = ox * S - a.pw;
#pragma unroll
      for (int ky = 0; ky < K; ++ky) {
#pragma unroll
        for (int kx = 0; kx < K; ++kx) {
          if ((unsigned int)(iy0 + ky) < (unsigned int)a.H && (unsigned int)(ix0 + kx) < (unsigned int)a.W)
            acc[ky * K + kx] = fmaf(Elem<T>::to_f32(xp[(iy0 + ky) * a.W + ix0 + kx]), g, acc[ky * K + kx]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i <= KK; ++i) {
    float v = i < KK ? acc[i < KK ? i : 0] : bsum;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp][i] = v;
  }
  __syncthreads();
  if (threadIdx.x <= KK) {
    float v = 0.0f;
#pragma unroll
    for (int wv = 0; wv < kThreads / 32; ++wv) v += red[wv][threadIdx.x];
    if (threadIdx.x < KK) {
      if (a.dw) atomicAdd(static_cast<float *>(a.dw) + (long long)oc * KK + threadIdx.x, v);
    } else if (a.db) {
      atomicAdd(static_cast<float *>(a.db) + oc, v);
    }
  }
}

// 3 x 3, stride 1, pad 1 (the output plane is the input plane's size; any multiplier): the common
// layer, with a register window in place of nine loads per output. A lane owns four output columns
// of a band of rows and slides three rows of the six input columns under them down the band: per
// row one 16-byte load of x (plus the two neighbours), one of dy, 36 fused multiply-adds onto the
// nine sums. Lanes = (band, column block): 14 blocks x 2 bands on a 56-wide plane, 7 x 4 on 28,
// 4 x 8 on 14. VEC: rows are 16-byte aligned (W a multiple of 4, aligned tensors); otherwise the
// same window from single loads, the last block's missing columns read as zero. A warp per image,
// CTAs = (channel, slice of the batch), reduction and atomics as in the kernel above.
template <bool VEC, int NC>
__global__ void __launch_bounds__(kThreads, 4) dwconv_bwd_weights_rows_kernel(const BwdArgs a, const int slices) {
  __shared__ float red[kThreads / 32][10];
  const float *x = static_cast<const float *>(a.x);
  const float *dy = static_cast<const float *>(a.dy);
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const int oc = blockIdx.x / slices;
  const int slice = blockIdx.x % slices;
  const int ic = oc / a.mult;
  const int H = a.H, W = a.W, plane = H * W;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long per = (a.n + slices - 1) / slices;
  const long long n0 = (long long)slice * per;
  const long long n1 = n0 + per < a.n ? n0 + per : a.n;
  const int ncb = (W + NC - 1) / NC;
  int bands = ncb >= 32 ? 1 : 32 / ncb;
  if (bands > H) bands = H;
  const int rows_per_band = (H + bands - 1) / bands;
  const int items = ncb * bands;
  float acc[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) acc[i] = 0.0f;
  float bsum = 0.0f;
  for (long long n = n0 + warp; n < n1; n += kThreads / 32) {
    const float *dyp = dy + (n * a.OC + oc) * plane;
    const float *xp = x + (n * a.C + ic) * plane;
    for (int item = lane; item < items; item += 32) {
      const int band = item / ncb, c0 = (item - band * ncb) * NC;
      const int r0 = band * rows_per_band;
      const int r1 = r0 + rows_per_band < H ? r0 + rows_per_band : H;
      const bool whole = VEC && c0 + NC <= W;  // the block's 16-byte vectors lie inside the row
      // input columns c0 - 1 .. c0 + NC of row iy; zero outside the plane
      auto load_row = [&](int iy, float(&r)[NC + 2]) {
        if ((unsigned int)iy >= (unsigned int)H) {
#pragma unroll
          for (int j = 0; j < NC + 2; ++j) r[j] = 0.0f;
          return;
        }
        const float *p = xp + iy * W + c0;
        if (whole) {
#pragma unroll
          for (int v4 = 0; v4 < NC / 4; ++v4) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(p) + v4);
            r[1 + 4 * v4] = v.x; r[2 + 4 * v4] = v.y; r[3 + 4 * v4] = v.z; r[4 + 4 * v4] = v.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < NC; ++j) r[1 + j] = c0 + j < W ? __ldg(p + j) : 0.0f;
        }
        r[0] = c0 > 0 ? __ldg(p - 1) : 0.0f;
        r[NC + 1] = c0 + NC < W ? __ldg(p + NC) : 0.0f;
      };
      float top[NC + 2], mid[NC + 2], bot[NC + 2];
      load_row(r0 - 1, top);
      load_row(r0, mid);
      for (int oy = r0; oy < r1; ++oy) {
        load_row(oy + 1, bot);
        float g[NC];
        const float *q = dyp + oy * W + c0;
        if (whole) {
#pragma unroll
          for (int v4 = 0; v4 < NC / 4; ++v4) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(q) + v4);
            g[4 * v4] = v.x; g[4 * v4 + 1] = v.y; g[4 * v4 + 2] = v.z; g[4 * v4 + 3] = v.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < NC; ++j) g[j] = c0 + j < W ? __ldg(q + j) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < NC; j += 4) bsum += (g[j] + g[j + 1]) + (g[j + 2] + g[j + 3]);
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
#pragma unroll
          for (int j = 0; j < NC; ++j) {
            acc[kx] = fmaf(top[j + kx], g[j], acc[kx]);
            acc[3 + kx] = fmaf(mid[j + kx], g[j], acc[3 + kx]);
            acc[6 + kx] = fmaf(bot[j + kx], g[j], acc[6 + kx]);
          }
        }
#pragma unroll
        for (int j = 0; j < NC + 2; ++j) {
          top[j] = mid[j];
          mid[j] = bot[j];
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i <= 9; ++i) {
    float v = i < 9 ? acc[i < 9 ? i : 0] : bsum;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp][i] = v;
  }
  __syncthreads();
  if (threadIdx.x <= 9) {
    float v = 0.0f;
#pragma unroll
    for (int wv = 0; wv < kThreads / 32; ++wv) v += red[wv][threadIdx.x];
    if (threadIdx.x < 9) {
      if (a.dw) atomicAdd(static_cast<float *>(a.dw) + (long long)oc * 9 + threadIdx.x, v);
    } else if (a.db) {
      atomicAdd(static_cast<float *>(a.db) + oc, v);
    }
  }
}

// The same register window for 3 x 3, stride 2, pad 1: a lane's four output columns read the nine
// input columns 8 cb - 1 .. 8 cb + 7, and an output row the input rows 2 oy - 1, 2 oy, 2 oy + 1, of
// which the first is the last one of the row above: two new rows of x (two 16-byte loads and the
// left neighbour each) and one row of dy per 36 multiply-adds. VECX / VECY: the rows of x / of dy
// are 16-byte aligned.
template <bool VECX, bool VECY>
__global__ void __launch_bounds__(kThreads, 4) dwconv_bwd_weights_rows_s2_kernel(const BwdArgs a, const int slices) {
  __shared__ float red[kThreads / 32][10];
  const float *x = static_cast<const float *>(a.x);
  const float *dy = static_cast<const float *>(a.dy);
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const int oc = blockIdx.x / slices;
  const int slice = blockIdx.x % slices;
  const int ic = oc / a.mult;
  const int H = a.H, W = a.W, Ho = a.Ho, Wo = a.Wo;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long per = (a.n + slices - 1) / slices;
  const long long n0 = (long long)slice * per;
  const long long n1 = n0 + per < a.n ? n0 + per : a.n;
  const int ncb = (Wo + 3) >> 2;
  int bands = ncb >= 32 ? 1 : 32 / ncb;
  if (bands > Ho) bands = Ho;
  const int rows_per_band = (Ho + bands - 1) / bands;
  const int items = ncb * bands;
  float acc[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) acc[i] = 0.0f;
  float bsum = 0.0f;
  for (long long n = n0 + warp; n < n1; n += kThreads / 32) {
    const float *dyp = dy + (n * a.OC + oc) * ((long long)Ho * Wo);
    const float *xp = x + (n * a.C + ic) * ((long long)H * W);
    for (int item = lane; item < items; item += 32) {
      const int band = item / ncb, cb = item - band * ncb;
      const int c0 = cb * 4, i0 = cb * 8;  // first output column, input column under its middle tap
      const int r0 = band * rows_per_band;
      const int r1 = r0 + rows_per_band < Ho ? r0 + rows_per_band : Ho;
      // input columns i0 - 1 .. i0 + 7 of row iy; zero outside the plane
      auto load_row = [&](int iy, float(&r)[9]) {
        if ((unsigned int)iy >= (unsigned int)H) {
#pragma unroll
          for (int j = 0; j < 9; ++j) r[j] = 0.0f;
          return;
        }
        const float *p = xp + iy * W + i0;
        if (VECX && i0 + 8 <= W) {
          const float4 u = __ldg(reinterpret_cast<const float4 *>(p)), v = __ldg(reinterpret_cast<const float4 *>(p + 4));
          r[1] = u.x; r[2] = u.y; r[3] = u.z; r[4] = u.w; r[5] = v.x; r[6] = v.y; r[7] = v.z; r[8] = v.w;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) r[1 + j] = i0 + j < W ? __ldg(p + j) : 0.0f;
        }
        r[0] = i0 > 0 ? __ldg(p - 1) : 0.0f;
      };
      float top[9], mid[9], bot[9];
      load_row(2 * r0 - 1, top);
      for (int oy = r0; oy < r1; ++oy) {
        load_row(2 * oy, mid);
        load_row(2 * oy + 1, bot);
        float g[4];
        const float *q = dyp + oy * Wo + c0;
        if (VECY) {
          const float4 v = __ldg(reinterpret_cast<const float4 *>(q));
          g[0] = v.x; g[1] = v.y; g[2] = v.z; g[3] = v.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) g[j] = c0 + j < Wo ? __ldg(q + j) : 0.0f;
        }
        bsum += (g[0] + g[1]) + (g[2] + g[3]);
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[kx] = fmaf(top[2 * j + kx], g[j], acc[kx]);
            acc[3 + kx] = fmaf(mid[2 * j + kx], g[j], acc[3 + kx]);
            acc[6 + kx] = fmaf(bot[2 * j + kx], g[j], acc[6 + kx]);
          }
        }
#pragma unroll
        for (int j = 0; j < 9; ++j) top[j] = bot[j];
      }
    }
  }
#pragma unroll
  for (int i = 0; i <= 9; ++i) {
    float v = i < 9 ? acc[i < 9 ? i : 0] : bsum;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp][i] = v;
  }
  __syncthreads();
  if (threadIdx.x <= 9) {
    float v = 0.0f;
#pragma unroll
    for (int wv = 0; wv < kThreads / 32; ++wv) v += red[wv][threadIdx.x];
    if (threadIdx.x < 9) {
      if (a.dw) atomicAdd(static_cast<float *>(a.dw) + (long long)oc * 9 + threadIdx.x, v);
    } else if (a.db) {
      atomicAdd(static_cast<float *>(a.db) + oc, v);
    }
  }
}

// Any kernel size: one CTA per weight value (and one more per channel for the bias), the
// reference's own decomposition. Slow path for kernels other than 3x3 and 5x5.
template <typename T>
__global__ void __launch_bounds__(kThreads) dwconv_bwd_weights_any_kernel(const BwdArgs a) {
  __shared__ float red[kThreads / 32];
  const T *x = static_cast<const T *>(a.x);
  const T *dy = static_cast<const T *>(a.dy);
  const int kk = a.kh * a.kw;
  const int oc = blockIdx.x / (kk + 1);
  const int tap = blockIdx.x % (kk + 1);  // kk = the bias
  if (tap == kk && !a.db) return;
  if (tap < kk && !a.dw) return;
  const int ic = oc / a.mult;
  const int ky = tap < kk ? tap / a.kw : 0, kx = tap < kk ? tap % a.kw : 0;
  const long long plane_out = (long long)a.Ho * a.Wo;
  float v = 0.0f;
  for (long long it = threadIdx.x; it < a.n * plane_out; it += kThreads) {
    const long long n = it / plane_out;
    const int pos = (int)(it % plane_out);
    const int oy = pos / a.Wo, ox = pos - oy * a.Wo;
    const float g = Elem<T>::to_f32(dy[(n * a.OC + oc) * plane_out + pos]);
    if (tap == kk) {
      v += g;
    } else {
      const int iy = oy * a.sh + ky * a.dh - a.ph;
      const int ix = ox * a.sw + kx * a.dw_ - a.pw;
      if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W)
        v += Elem<T>::to_f32(x[((n * a.C + ic) * a.H + iy) * (long long)a.W + ix]) * g;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.0f;
    for (int i = 0; i < kThreads / 32; ++i) s += red[i];
    if (tap == kk) atomicAdd(static_cast<float *>(a.db) + oc, s);
    else atomicAdd(static_cast<float *>(a.dw) + (long long)oc * kk + tap, s);
  }
}

__global__ void zero_f32_kernel(float *p, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    p[i] = 0.0f;
}

}  // namespace

int launch_ste_backward(int dtype, int mode, int accum, long long size, float fpq_max, float fpq_min,
                        unsigned int pow2_first_above, int pow2_sign, const void *x, const void *dy, void *dx,
                        cudaStream_t stream) {
  SteArgs s;
  s.fpq_max = fpq_max;
  s.fpq_min = fpq_min;
  s.pow2_first_above = pow2_first_above;
  s.pow2_sign = pow2_sign;
  const cudaError_t e =
      dtype == DWBNQ_F32
          ? launch_ste_t<float>(mode, accum, static_cast<const float *>(x), static_cast<const float *>(dy),
                                static_cast<float *>(dx), size, s, stream)
          : launch_ste_t<__half>(mode, accum, static_cast<const __half *>(x), static_cast<const __half *>(dy),
                                 static_cast<__half *>(dx), size, s, stream);
  if (e != cudaSuccess) return fail_cuda(e, "ste_backward_kernel launch");
  return DWBNQ_OK;
}

int launch_dwconv_backward(const dwbnq_conv_desc &d, int ho, int wo, const void *x, const void *w, const void *dy,
                           void *dx, void *dw, void *db, int accum_mask, cudaStream_t stream) {
  BwdArgs a;
  a.x = x;
  a.w = w;
  a.dy = dy;
  a.dx = dx;
  a.dw = dw;
  a.db = db;
  a.n = d.n;
  a.C = d.c;
  a.H = d.h;
  a.W = d.w;
  a.OC = d.c * d.multiplier;
  a.Ho = ho;
  a.Wo = wo;
  a.kh = d.kh;
  a.kw = d.kw;
  a.sh = d.stride_h;
  a.sw = d.stride_w;
  a.ph = d.pad_h;
  a.pw = d.pad_w;
  a.dh = d.dil_h;
  a.dw_ = d.dil_w;
  a.mult = d.multiplier;
  cudaError_t e = cudaSuccess;
  // Stride 1, no dilation, multiplier 1, pad = (k - 1) / 2 on an odd square kernel, overwrite:
  // the input gradient IS the forward convolution of dy with the kernel rotated by 180
  // degrees (same padding), so it runs on the fused family's kernels (no bias, no BN, no
  // quantizer) with the taps read back to front - at their speed. Its sum runs over the taps
  // in the forward kernels' order, the reverse of the reference loop's: equal within rounding,
  // not bit for bit. Every other case takes the direct kernel below, in the reference's order.
  if (dx && !(accum_mask & 1) && d.stride_h == 1 && d.stride_w == 1 && d.dil_h == 1 && d.dil_w == 1 &&
      d.multiplier == 1 && d.kh == d.kw && (d.kh % 2) == 1 && d.pad_h == d.kh / 2 && d.pad_w == d.kw / 2 && d.n > 0 &&
      bwd_input_by_forward_enabled()) {
    dwbnq_conv_desc g = d;  // dy has the shape of x here (same padding, stride 1)
    FusedArgs fa;
    std::memset(&fa, 0, sizeof(fa));
    fa.x = dy;
    fa.w = w;
    fa.y = dx;
    fa.n = d.n;
    fa.C = fa.OC = d.c;
    fa.H = fa.Ho = d.h;
    fa.W = fa.Wo = d.w;
    fa.kh = d.kh;
    fa.kw = d.kw;
    fa.sh = fa.sw = fa.dh = fa.dw = fa.mult = 1;
    fa.ph = d.pad_h;
    fa.pw = d.pad_w;
    fa.w_flip = 1;
    int dev = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
    const int st = launch_fused(g, fa, QM_NONE, dev, stream);
    if (st != DWBNQ_OK) return st;
    dx = nullptr;  // done
  }
  if (dx) {
    const long long total = d.n * (long long)d.c * d.h * d.w;
    const int per_cta = kThreads * 8;
    long long ctas = (total + per_cta - 1) / per_cta;
    const long long cap = (long long)sm_count(-1) * 32;
    if (ctas > cap) ctas = cap;
    const dim3 grid((unsigned int)(ctas < 1 ? 1 : ctas)), block(kThreads);
    const bool acc = (accum_mask & 1) != 0;
    const bool simple = d.kh == d.kw && d.dil_h == 1 && d.dil_w == 1 && d.multiplier == 1 && d.stride_h == d.stride_w &&
                        (long long)d.h * d.w < 0x40000000LL && (long long)ho * wo < 0x40000000LL;
    const int key = !simple ? 0 : (d.kh == 3 ? 30 : d.kh == 5 ? 50 : 0) + (d.stride_h == 1 ? 1 : d.stride_h == 2 ? 2 : -100);
#define DWBNQ_BIN(KV, SV)                                                                                       \
  e = acc ? launch_pdl(dwconv_bwd_input_kernel<float, KV, SV, true>, grid, block, 0, stream, a, total, per_cta) \
          : launch_pdl(dwconv_bwd_input_kernel<float, KV, SV, false>, grid, block, 0, stream, a, total, per_cta)
    if ((long long)d.h * d.w >= 0x40000000LL || (long long)ho * wo >= 0x40000000LL)
      return fail(DWBNQ_ERR_UNSUPPORTED, "DepthwiseConvolution backward: planes of 2^30 elements or more");
    switch (key) {
      case 31: DWBNQ_BIN(3, 1); break;
      case 32: DWBNQ_BIN(3, 2); break;
      case 51: DWBNQ_BIN(5, 1); break;
      case 52: DWBNQ_BIN(5, 2); break;
      default: DWBNQ_BIN(0, 1); break;
    }
#undef DWBNQ_BIN
    if (e != cudaSuccess) return fail_cuda(e, "dwconv_bwd_input_kernel launch");
  }
  if (dw || db) {
    const int kk = d.kh * d.kw;
    // gradients that are not accumulated onto start from zero (the kernels add atomically)
    if (dw && !(accum_mask & 2)) {
      zero_f32_kernel<<<grid_for((long long)a.OC * kk, 4), kThreads, 0, stream>>>(static_cast<float *>(dw),
                                                                                    (long long)a.OC * kk);
      if ((e = cudaGetLastError()) != cudaSuccess) return fail_cuda(e, "zero_f32_kernel launch");
    }
    if (db && !(accum_mask & 4)) {
      zero_f32_kernel<<<grid_for(a.OC, 4), kThreads, 0, stream>>>(static_cast<float *>(db), a.OC);
      if ((e = cudaGetLastError()) != cudaSuccess) return fail_cuda(e, "zero_f32_kernel launch");
    }
    const bool fast = d.kh == d.kw && (d.kh == 3 || d.kh == 5) && d.stride_h == d.stride_w &&
                      (d.stride_h == 1 || d.stride_h == 2) && d.dil_h == 1 && d.dil_w == 1 &&
                      (long long)d.h * d.w < 0x40000000LL && d.n > 0;
    if (fast) {
      // A CTA is (channel, slice of the batch), a warp per image. The slice count is the one whose
      // CTAs fill whole waves of the resident slots (four CTAs per SM) and whose images fill whole
      // rounds of a CTA's eight warps: the product of the two fill ratios, searched over the
      // counts that leave every warp about a thousand outputs or more - below that the CTA's
      // reduction and atomics outweigh its sums (fewest slices on ties).
      long long slices = 1;
      {
        const long long slots = (long long)sm_count(-1) * 4, warps = kThreads / 32;
        double best = -1.0;
        const long long most = d.n < 2048 ? d.n : 2048;
        const long long plane_out = (long long)ho * wo;
        const long long min_per = warps * (plane_out >= 1024 ? 1 : (1024 + plane_out - 1) / plane_out);
        for (long long s = 1; s <= most; ++s) {
          const long long per = (d.n + s - 1) / s;       // images of a full slice
          if (s > 1 && per < min_per) break;
          const long long busy = (d.n + per - 1) / per;  // slices that have images
          const long long ctas = busy * a.OC, waves = (ctas + slots - 1) / slots;
          const double fill = (double)ctas / (double)(waves * slots) * (double)per / (double)((per + warps - 1) / warps * warps);
          if (fill > best + 1e-9) { best = fill; slices = s; }
        }
      }
      const dim3 grid((unsigned int)(a.OC * slices)), block(kThreads);
      const int key = d.kh * 10 + d.stride_h;
      const bool same_size = key == 31 && d.pad_h == 1 && d.pad_w == 1;
      const bool rows16 = d.w % 4 == 0 && (((uintptr_t)x | (uintptr_t)dy) & 15) == 0;
      // eight output columns per lane on planes wide enough to keep a warp's lanes busy with them (twice the
      // loads in flight per lane), four on the narrow ones
      if (same_size && rows16 && d.w >= 32) e = launch_pdl(dwconv_bwd_weights_rows_kernel<true, 8>, grid, block, 0, stream, a, (int)slices);
      else if (same_size && rows16) e = launch_pdl(dwconv_bwd_weights_rows_kernel<true, 4>, grid, block, 0, stream, a, (int)slices);
      else if (same_size && d.w >= 32) e = launch_pdl(dwconv_bwd_weights_rows_kernel<false, 8>, grid, block, 0, stream, a, (int)slices);
      else if (same_size) e = launch_pdl(dwconv_bwd_weights_rows_kernel<false, 4>, grid, block, 0, stream, a, (int)slices);
      else if (key == 32 && d.pad_h == 1 && d.pad_w == 1) {
        const bool vx = rows16, vy = wo % 4 == 0 && rows16;
        e = vx ? (vy ? launch_pdl(dwconv_bwd_weights_rows_s2_kernel<true, true>, grid, block, 0, stream, a, (int)slices)
                     : launch_pdl(dwconv_bwd_weights_rows_s2_kernel<true, false>, grid, block, 0, stream, a, (int)slices))
               : launch_pdl(dwconv_bwd_weights_rows_s2_kernel<false, false>, grid, block, 0, stream, a, (int)slices);
      } else if (key == 31) e = launch_pdl(dwconv_bwd_weights_kernel<float, 3, 1>, grid, block, 0, stream, a, (int)slices);
      else if (key == 32) e = launch_pdl(dwconv_bwd_weights_kernel<float, 3, 2>, grid, block, 0, stream, a, (int)slices);
      else if (key == 51) e = launch_pdl(dwconv_bwd_weights_kernel<float, 5, 1>, grid, block, 0, stream, a, (int)slices);
      else e = launch_pdl(dwconv_bwd_weights_kernel<float, 5, 2>, grid, block, 0, stream, a, (int)slices);
    } else if (d.n == 0) {
      e = cudaSuccess;  // nothing to add to the (zeroed or kept) gradients
    } else {
      const dim3 grid((unsigned int)(a.OC * (kk + 1))), block(kThreads);
      dwconv_bwd_weights_any_kernel<float><<<grid, block, 0, stream>>>(a);
      e = cudaGetLastError();
    }
    if (e != cudaSuccess) return fail_cuda(e, "dwconv_bwd_weights_kernel launch");
  }
  return DWBNQ_OK;
}

}  // namespace dwbnq
