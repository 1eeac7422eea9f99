// Pointwise (1x1) convolution, optionally fused with BatchNormalization inference, an
// activation and FixedPointQuantize / Pow2Quantize: y[n][co][p] = epilogue(sum_ci w[co][ci] *
// x[n][ci][p] + b[co]) for NCHW tensors, p running over the h*w positions of an image.
//
// The tensor-core kernel is written for sm_100a directly (tcgen05.mma with the accumulator
// in tensor memory, TMA tiled loads, mbarrier pipelines):
//  * per image the product is D[position][co] = X^T[position][ci] * W^T[ci][co]: the A operand
//    is a tile of 128 positions (MN-major in shared memory, exactly how NCHW stores it), the B
//    operand the weights (K-major), so the 128 TMEM lanes are positions and the columns are
//    output channels. A warp that reads the accumulator back holds, per column, 32 consecutive
//    positions of one channel: BN / activation / quantizer run in registers with warp-uniform
//    per-channel coefficients and every store is one coalesced 128-byte line - no staging of
//    the output in shared memory;
//  * one CTA per SM walks over (channel tile, 128 positions) pairs; warp 0 issues the TMA
//    loads, warp 1 the MMAs, warps 2-9 bring the activations into operand form - they split the
//    TMA-loaded fp32 values into TF32 halves for the three-pass mode, or, in gather mode, load
//    them with plain loads (planes TMA cannot take or would tile badly), rows flattened over
//    (image, position) - and warps 10-25 are the epilogue (four groups of four warps, each
//    group a tile of its own, or all four sharing a tile's columns when a CTA has few tiles);
//    up to eight accumulator buffers in TMEM decouple the MMAs from the epilogue;
//  * binary16 tensors whose rows are multiples of 16 bytes stay binary16 all the way: TMA loads
//    of x and w, tcgen05.mma.kind::f16, 64 channels per stage and no worker pass; the others are
//    gathered and converted (exactly) for one TF32 pass;
//  * every wait on an mbarrier is bounded in time; a wait that runs out records it in the
//    device flag, the roles leave their loops, and the CTA frees its tensor memory and returns.
// c_in that is not a multiple of 4 (the weight rows must be 16-byte multiples for their TMA
// loads) runs on a plain FMA kernel with the same epilogue.
#include <cstdlib>
#include <cstring>

#include "dwbnq_internal.h"

namespace dwbnq {

namespace {

constexpr int kPwXWarps = 8, kPwFirstEpiWarp = 2 + kPwXWarps, kPwEpiGroups = 4, kPwEpiWarps = 4 * kPwEpiGroups;
constexpr int kPwThreads = 32 * (kPwFirstEpiWarp + kPwEpiWarps);
constexpr int kPwTmemCols = 512;           // the whole tensor memory of the SM (one CTA per SM)
constexpr int kPwMaxAcc = 8;               // accumulator buffers in flight
constexpr int kPwMaxCout = 4096;           // channel pairs of the coefficient table: 48 bytes each
constexpr int kPwPosTile = 128;            // accumulator rows = TMEM lanes
constexpr int kPwKChunk = 32;              // fp32 elements of c_in per pipeline stage
constexpr int kPwXBytes = kPwPosTile * kPwKChunk * 4;  // 4 boxes of [32 k][32 positions]
constexpr int kPwMaxStages = 8;
constexpr int kPwMaxCoTile = 256;          // two accumulators of 256 columns fill the 512 of TMEM
constexpr int kPwSmemMax = 227 * 1024 - 1024;  // dynamic shared memory the kernel may ask for
constexpr unsigned long long kPwWaitNs = 2000000000ull;

// Epilogue variants compiled separately (a run-time switch inside the unrolled loops costs more
// instructions than the arithmetic): bias only; BN + unsigned power-of-two FixedPointQuantize
// with or without ReLU6 in between (after ReLU6 the quantizer's clamps are redundant when its
// range reaches 6); BN + signed power-of-two FixedPointQuantize (the linear projection of an
// inverted residual); everything else with run-time switches.
// How the activations reach shared memory: TMA boxes per image (fp32, or binary16 as it is); plain loads with the rows
// flattened over (image, position), one element or - where the plane size is a multiple of 4
// and the base aligned - four consecutive positions per load.
enum PwXMode : int { PW_X_TMA = 0, PW_X_GATHER = 1, PW_X_GATHER4 = 2 };
enum PwEpi : int { PW_EPI_BIAS = 0, PW_EPI_BN_FPQ = 1, PW_EPI_BN_RELU6_FPQ = 2, PW_EPI_BN_FPQS = 3, PW_EPI_GENERIC = 4 };

// Per pair of output channels, everything the epilogue needs (three 16-byte shared-memory words).
struct __align__(16) PwPair {
  f32x2 bias, nmean, scale, rcp, nstd, beta;
};

struct PwArgs {
  int HW, Ci, Co;
  long long N;
  int npad;       // accumulator columns per channel tile (multiple of 32, <= 256)
  int co_tiles, pos_tiles, kchunks;
  int total_tiles, per_ct;  // per_ct = N * pos_tiles
  int stages, stage_bytes;
  int nacc;       // accumulator buffers of npad columns in TMEM, a multiple of ngroups
  int ngroups;    // epilogue groups in use (<= kPwEpiGroups): buffer b always belongs to group b % ngroups
  int col_split;  // 1: every group works on every tile, a quarter of its columns each (few tiles per CTA)
  const float *coef;  // [5][cstride]: bias, mean, scale, stdvar, beta
  int cstride;        // >= co_tiles * npad
  const void *x;      // gather mode: the activations (fp32 or fp16), read with plain loads
  long long total_pos;  // gather mode: N * HW, the flattened positions
  void *y;            // fp32 or fp16 like x
  int *flag;
  int has_bn, act, qkind;
  QuantArgs q;
};

// ---- sm_100a PTX wrappers ------------------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *tm, int x, int y, unsigned long long *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Bounded waits of this kernel. Most of the twenty-odd warps of a CTA wait most of the time;
// the poll carries a suspend-time hint so that a waiting warp is parked by the hardware and
// leaves the issue slots to the warps that compute (a bare spin took about a third of them).
__device__ __forceinline__ bool pw_try_wait(unsigned long long *bar, unsigned int parity) {
  unsigned int ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool pw_wait_lane(unsigned long long *bar, unsigned int parity) {
  if (pw_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
#pragma unroll 1
  for (unsigned int i = 0; i < (1u << 28); ++i) {
    if (pw_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > kPwWaitNs) break;
  }
  return false;
}
// Warp-uniform form: every lane has seen the phase, or every lane gives up.
__device__ __forceinline__ bool pw_wait(unsigned long long *bar, unsigned int parity) {
  bool ok = pw_wait_lane(bar, parity);
  if (!__all_sync(0xffffffffu, ok)) {
    if (__any_sync(0xffffffffu, ok) && !ok) ok = pw_try_wait(bar, parity);
    ok = __all_sync(0xffffffffu, ok);
  }
  return ok;
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// The barrier receives one arrival once every MMA this thread has issued so far is complete.
__device__ __forceinline__ void tc_commit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[128 x N] (+)= A[128 x 8] * B[N x 8]^T, TF32 operands from shared memory, fp32 accumulator in TMEM.
__device__ __forceinline__ void tc_mma_tf32(unsigned int tmem_d, unsigned long long da, unsigned long long db,
                                            unsigned int idesc, unsigned int accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Four consecutive elements as floats (16-byte load of fp32, 8-byte load of fp16).
__device__ __forceinline__ float4 pw_load4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float4 pw_load4(const __half *p) {
  const uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
// D[128 x N] (+)= A[128 x 16] * B[N x 16]^T, binary16 operands, fp32 accumulator.
__device__ __forceinline__ void tc_mma_f16(unsigned int tmem_d, unsigned long long da, unsigned long long db,
                                           unsigned int idesc, unsigned int accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 8 consecutive accumulator columns of this thread's lane (issue only; tc_ld_wait8 completes it).
__device__ __forceinline__ void tc_ld8(unsigned int taddr, unsigned int *r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
// Waits for this thread's outstanding TMEM loads. The loaded registers are operands, so the
// compiler cannot move a use of them above the wait.
__device__ __forceinline__ void tc_ld_wait8(unsigned int *r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
               :
               : "memory");
}

// Shared-memory matrix descriptor of tcgen05.mma (addresses and offsets in bytes; the fields
// hold them divided by 16). layout 2 = 128-byte swizzle, 1 = 128-byte swizzle of 32-byte
// units, the only form the hardware takes for an MN-major operand of 32-bit elements.
__device__ __forceinline__ unsigned long long pw_smem_desc(unsigned int addr, unsigned int lbo, unsigned int sbo,
                                                          unsigned int layout) {
  return (unsigned long long)((addr >> 4) & 0x3fffu) | ((unsigned long long)((lbo >> 4) & 0x3fffu) << 16) |
         ((unsigned long long)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46) | ((unsigned long long)layout << 61);
}
// A: 128 positions x 8 channels of a stage's activation buffer. The buffer is four TMA boxes
// of [32 channels][32 positions] fp32 (4 KiB each, 128-byte rows, 32-byte units swizzled by
// row mod 4): consecutive groups of 32 positions are 4096 bytes apart (leading offset), the
// two groups of 4 channels one MMA consumes 512 bytes (stride offset).
__device__ __forceinline__ unsigned long long pw_desc_a(unsigned int buf, int kstep) {
  return pw_smem_desc(buf + kstep * 1024, 4096, 512, 1);
}
// A for binary16 tensors (kind::f16, 16 channels per MMA): two TMA boxes of [64 channels][64
// positions] binary16 per stage (128-byte rows in the ordinary 128-byte swizzle, layout type 2):
// the two groups of 64 positions are 8192 bytes apart (leading offset), groups of 8 channels 1024
// bytes (stride offset); a step of 16 channels advances the start by 2048 bytes. (Found with a
// probe over descriptor fields against a CPU product; the weights' [N][64] box takes the same
// descriptor as the fp32 one, its 16-channel step being 32 bytes too.)
__device__ __forceinline__ unsigned long long pw_desc_a16(unsigned int buf, int kstep) {
  return pw_smem_desc(buf + kstep * 2048, 8192, 1024, 2);
}
// B: N channels-out x 8 channels-in of a stage's weight buffer, one TMA box of [N][32] fp32
// (128-byte rows, 16-byte units swizzled by row mod 8): groups of 8 rows are 1024 bytes apart,
// a step of 8 along c_in advances the start by 32 bytes inside the row.
__device__ __forceinline__ unsigned long long pw_desc_b(unsigned int buf, int kstep) {
  return pw_smem_desc(buf + kstep * 32, 16, 1024, 2);
}

// ---- epilogue --------------------------------------------------------------------------------

__device__ __forceinline__ float pw_act(float v, int act) {
  if (act == DWBNQ_ACT_RELU6) return fminf(fmaxf(v, 0.0f), 6.0f);
  if (act == DWBNQ_ACT_RELU) return fmaxf(0.0f, v);
  return v;
}

__device__ __forceinline__ PwPair pw_make_pair(const PwArgs &a, int cpad, int c, bool *safe) {
  // c is even and c + 1 < cpad; padded channels hold neutral coefficients
  const BnCoef lo{a.coef[cpad + c], a.coef[2 * cpad + c], a.coef[3 * cpad + c], a.coef[4 * cpad + c]};
  const BnCoef hi{a.coef[cpad + c + 1], a.coef[2 * cpad + c + 1], a.coef[3 * cpad + c + 1], a.coef[4 * cpad + c + 1]};
  const BnPacked b = make_bn_packed2(lo, hi, 0ull);
  PwPair p;
  p.bias = pack2(a.coef[c], a.coef[c + 1]);
  p.nmean = b.nmean; p.scale = b.scale; p.rcp = b.rcp; p.nstd = b.nstd; p.beta = b.beta;
  *safe = b.glo == DWBNQ_DIV_GUARD_LO;
  return p;
}

// Eight adjacent channels (four pairs) of one position: accumulators in, final values out.
// BN divides through the packed reciprocal sequence of bn_apply_packed; one range test covers
// the unit, and a unit that fails it (or a launch whose stdvar leaves the range the sequence
// is proven for) takes the IEEE division.
template <int EPI>
__device__ __forceinline__ void pw_finish_unit(const unsigned int *acc, const PwPair *tp, const PwArgs &a, f32x2 nz,
                                               const FpqPacked &fq, bool bn_safe, float *r) {
  f32x2 v[4];
  const bool bn = EPI == PW_EPI_BN_FPQ || EPI == PW_EPI_BN_RELU6_FPQ || EPI == PW_EPI_BN_FPQS || (EPI == PW_EPI_GENERIC && a.has_bn);
  if (bn) {
    f32x2 t[4], nstd[4];
    float mx = 0.0f, mn = __uint_as_float(0x7f800000u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const PwPair cp = tp[i];
      const f32x2 s = add2(pack2(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1])), cp.bias);
      t[i] = mul2(add2(s, cp.nmean), cp.scale, nz);
      float lo, hi;
      unpack2(t[i], lo, hi);
      mx = max3f(mx, fabsf(lo), fabsf(hi));
      mn = min3f(mn, fabsf(lo), fabsf(hi));
      f32x2 q = mul2(t[i], cp.rcp, nz);
      f32x2 e = fma2(q, cp.nstd, t[i]);
      q = fma2(e, cp.rcp, q);
      e = fma2(q, cp.nstd, t[i]);
      v[i] = fma2(e, cp.rcp, q);
      nstd[i] = cp.nstd;
    }
    if (!(bn_safe && mn > DWBNQ_DIV_GUARD_LO && mx < DWBNQ_DIV_GUARD_HI)) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float slo, shi;
        unpack2(nstd[i], slo, shi);
        v[i] = bn_div_cold(t[i], -slo, -shi);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = add2(v[i], tp[i].beta);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      v[i] = add2(pack2(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1])), tp[i].bias);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float r0, r1;
    unpack2(v[i], r0, r1);
    if (EPI == PW_EPI_BN_RELU6_FPQ) {
      r0 = fminf(fmaxf(r0, 0.0f), 6.0f);
      r1 = fminf(fmaxf(r1, 0.0f), 6.0f);
      const f32x2 kp = add2_rm(fma2_rm(pack2(r0, r1), fq.inv, fq.half), fq.magic);
      unpack2(fma2(kp, fq.delta, fq.nmagic), r0, r1);
    } else if (EPI == PW_EPI_BN_FPQ) {
      unpack2(fpq_apply_fast_unsigned2(r0, r1, a.q, fq), r0, r1);
    } else if (EPI == PW_EPI_BN_FPQS) {
      r0 = fpq_apply_fast<true>(r0, a.q);
      r1 = fpq_apply_fast<true>(r1, a.q);
    } else if (EPI == PW_EPI_GENERIC) {
      if (a.act) { r0 = pw_act(r0, a.act); r1 = pw_act(r1, a.act); }
      if (a.qkind == DWBNQ_Q_FPQ) { r0 = fpq_apply(r0, a.q); r1 = fpq_apply(r1, a.q); }
      else if (a.qkind == DWBNQ_Q_POW2) { r0 = pow2_apply(r0, a.q); r1 = pow2_apply(r1, a.q); }
    }
    r[2 * i] = r0;
    r[2 * i + 1] = r1;
  }
}

// ---- the tcgen05 kernel ------------------------------------------------------------------------

// T: the tensors' element type. fp16 tensors come in through the gather path only and run the single
// pass: a binary16 value has 11 significant bits, so it is exact in TF32 and so is every product.
template <typename T, int XMODE, bool MATH3, int EPI>
__global__ void __launch_bounds__(kPwThreads, 1)
pw_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
             const __grid_constant__ CUtensorMap tm_wlo, const PwArgs a) {
  constexpr bool GATHER = XMODE != PW_X_TMA;  // rows = positions flattened over (image, position)
  // binary16 tensors through TMA: operands stay binary16 (kind::f16), 64 channels per stage, no X workers
  constexpr bool F16MMA = XMODE == PW_X_TMA && sizeof(T) == 2;
  constexpr int KCHUNK = F16MMA ? 64 : kPwKChunk;
  extern __shared__ unsigned char pw_smem_raw[];
  // full / empty / split per stage, then accumulator full / empty per buffer
  __shared__ unsigned long long bars[3 * kPwMaxStages + 2 * kPwMaxAcc];
  __shared__ unsigned int tmem_base_s;
  __shared__ int abort_s, unsafe_s;
  unsigned long long *full = bars, *empty = bars + kPwMaxStages, *split = bars + 2 * kPwMaxStages;
  unsigned long long *acc_full = bars + 3 * kPwMaxStages, *acc_empty = acc_full + kPwMaxAcc;
  const unsigned int base = (smem_u32(pw_smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  unsigned char *sm = pw_smem_raw + (base - smem_u32(pw_smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wbytes = a.npad * 128;
  const int off_xlo = kPwXBytes, off_w = MATH3 ? 2 * kPwXBytes : kPwXBytes, off_wlo = off_w + wbytes;
  const int cpad = a.co_tiles * a.npad;
  // after the stages: the coefficient table of every channel pair
  PwPair *table = reinterpret_cast<PwPair *>(sm + (size_t)a.stages * a.stage_bytes);

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&split[s], kPwXWarps);  // one arrival per X-worker warp
    }
    for (int b = 0; b < a.nacc; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], a.col_split ? 4 * kPwEpiGroups : 4);  // the warps that read the buffer
    }
    abort_s = 0;
    unsafe_s = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(kPwTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Launched with programmatic stream serialization: up to here (no global access) the CTA may
  // run while its predecessor in the stream drains; everything below follows the predecessor's
  // completion. The successor may become resident as soon as this grid's CTAs leave their SMs.
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const unsigned int tmem_base = tmem_base_s;
  volatile int *abort_v = &abort_s;

  if (warp == 0) {
    // ---- producer: one lane issues the TMA loads of every (tile, c_in chunk) ----
    if (lane == 0) {
      // (stage, phase) advance with a counter: this one thread's instruction stream is the
      // latency of the whole load pipeline, so nothing in it divides or recomputes addresses
      int s = 0;
      unsigned int ph = 0;
      const unsigned int bytes = (GATHER ? 0 : kPwXBytes) + wbytes * (MATH3 ? 2 : 1);
      bool ok = true;
      for (int t = blockIdx.x; ok && t < a.total_tiles; t += gridDim.x) {
        const int ct = t / a.per_ct;
        const int r = t - ct * a.per_ct;
        const int n = GATHER ? 0 : r / a.pos_tiles, pt = GATHER ? r : r - n * a.pos_tiles;
        const int c0 = ct * a.npad, p0 = pt * kPwPosTile;
        for (int kc = 0; kc < a.kchunks; ++kc) {
          if (!pw_wait_lane(&empty[s], ph ^ 1u) || *abort_v) { ok = false; break; }
          unsigned char *st = sm + (size_t)s * a.stage_bytes;
          mbar_expect_tx(&full[s], bytes);
          if (F16MMA) {
#pragma unroll
            for (int q = 0; q < 2; ++q) tma_load_3d(st + q * 8192, &tm_x, p0 + q * 64, kc * KCHUNK, n, &full[s]);
          } else if (!GATHER) {
#pragma unroll
            for (int q = 0; q < 4; ++q) tma_load_3d(st + q * 4096, &tm_x, p0 + q * 32, kc * KCHUNK, n, &full[s]);
          }
          tma_load_2d(st + off_w, &tm_w, kc * KCHUNK, c0, &full[s]);
          if (MATH3) tma_load_2d(st + off_wlo, &tm_wlo, kc * KCHUNK, c0, &full[s]);
          if (++s == a.stages) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok && !*abort_v) { atomicExch(a.flag, 1); *abort_v = 1; }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one thread. Its instruction stream is serial, so the descriptors of a
    // stage are the stage-0 descriptors plus a multiple of the stage size (the address field
    // counts 16-byte units and cannot carry into the next field: shared memory ends below
    // 2^18), and stages / buffers advance with counters ----
    if (lane == 0) {
      // instruction descriptor: fp32 accumulator, TF32 A and B, A MN-major, B K-major, N, M = 128
      // (binary16 operands: formats 0, 16 channels per instruction)
      const unsigned int idesc = (1u << 4) | (F16MMA ? 0u : (2u << 7) | (2u << 10)) | (1u << 15) |
                                 ((unsigned)(a.npad >> 3) << 17) | (8u << 24);
      const unsigned long long da0 = F16MMA ? pw_desc_a16(base, 0) : pw_desc_a(base, 0), dal0 = pw_desc_a(base + off_xlo, 0);
      const unsigned long long db0 = pw_desc_b(base + off_w, 0), dbl0 = pw_desc_b(base + off_wlo, 0);
      const unsigned long long stage_step = (unsigned long long)(a.stage_bytes >> 4);
      constexpr int KSTEP = F16MMA ? 16 : 8;  // channels per MMA
      const int last_steps = ((a.Ci - (a.kchunks - 1) * KCHUNK) + KSTEP - 1) / KSTEP;  // rows past c_in are zero-filled
      int s = 0, b = 0;
      unsigned int ph = 0, aph = 0;
      unsigned long long so = 0;  // s * stage_step
      bool ok = true;
      for (int t = blockIdx.x; ok && t < a.total_tiles; t += gridDim.x) {
        const unsigned int d = tmem_base + b * a.npad;
        for (int kc = 0; ok && kc < a.kchunks; ++kc) {
          // the polls of a chunk's barriers are issued together (each is a shared-memory round trip
          // of ~150 cycles for this one thread); a poll that fails goes to the bounded wait
          const bool r0 = kc ? true : pw_try_wait(&acc_empty[b], aph ^ 1u);
          const bool r1 = pw_try_wait(&full[s], ph);
          const bool r2 = (MATH3 || GATHER) ? pw_try_wait(&split[s], ph) : true;
          if (!r0) ok = pw_wait_lane(&acc_empty[b], aph ^ 1u);
          if (ok && !r1) ok = pw_wait_lane(&full[s], ph);
          if (ok && !r2) ok = pw_wait_lane(&split[s], ph);
          if (!ok) break;
          tc_fence_after();
          const int ksteps = kc == a.kchunks - 1 ? last_steps : KCHUNK / KSTEP;
          unsigned long long da = da0 + so, db = db0 + so, dal = dal0 + so, dbl = dbl0 + so;
          unsigned int acc = kc ? 1u : 0u;
#pragma unroll 1
          for (int j = 0; j < ksteps; ++j) {
            if (F16MMA) tc_mma_f16(d, da, db, idesc, acc);
            else tc_mma_tf32(d, da, db, idesc, acc);
            if (MATH3) {
              tc_mma_tf32(d, dal, db, idesc, 1u);
              tc_mma_tf32(d, da, dbl, idesc, 1u);
            }
            acc = 1u;
            da += F16MMA ? 128 : 64; dal += 64;  // 8 rows of 128 bytes (binary16: 16 rows)
            db += 2; dbl += 2;                   // 32 bytes along the row
          }
          tc_commit(&empty[s]);
          if (kc == a.kchunks - 1) tc_commit(&acc_full[b]);
          so += stage_step;
          if (++s == a.stages) { s = 0; ph ^= 1u; so = 0; }
        }
        if (++b == a.nacc) { b = 0; aph ^= 1u; }
        if (*abort_v) ok = false;
      }
      if (!ok && !*abort_v) { atomicExch(a.flag, 1); *abort_v = 1; }
    }
  } else if (warp < kPwFirstEpiWarp) {
    // ---- X workers (eight warps) ----
    const int tid = threadIdx.x - 64;
    if (XMODE == PW_X_GATHER4) {
      // The gather below with four positions per load. A timeline of the one-element form showed
      // the eight worker warps, not the MMA thread, setting the pace of the gathered layers (about
      // 1850 cycles per chunk: 16 loads and 32 stores per thread, each a warp instruction for 128
      // bytes). Here thread (position group pg, channel lane cw) loads positions 4 pg .. 4 pg + 3 of
      // channels cw, cw + 8, cw + 16, cw + 24 of the chunk - a warp reads 512 consecutive bytes of one
      // channel row - and stores each as one 16-byte vector: four consecutive positions are 16
      // consecutive bytes of the swizzled layout too, and k mod 4 = cw mod 4 for all four channels.
      // A group of four never straddles two images (the plane size is a multiple of 4).
      const int pg = tid & 31, cw = tid >> 5;
      const unsigned int sw4 = (unsigned)((pg >> 3) * 4096 + cw * 128 + (pg & 1) * 16) +
                               (((((unsigned)pg >> 1) & 3u) ^ ((unsigned)cw & 3u)) << 5);
      int t_l = blockIdx.x, kc_l = 0;
      bool valid_l = false;
      const T *const xbase = static_cast<const T *>(a.x);
      const T *xp_l = xbase;
      auto locate = [&]() {
        const long long g = (long long)(t_l % a.per_ct) * kPwPosTile + 4 * pg;
        valid_l = g < a.total_pos;
        const long long n = valid_l ? g / a.HW : 0;
        xp_l = xbase + (size_t)n * a.Ci * a.HW + (valid_l ? (int)(g - n * a.HW) : 0);
      };
      const size_t plane = (size_t)a.HW;
      auto load = [&](float4(&v)[4]) {
        const int k0 = kc_l * kPwKChunk + cw;
        const T *q = xp_l + (size_t)k0 * plane;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const T *qi = q + (size_t)(8 * i) * plane;
          v[i] = (valid_l && k0 + 8 * i < a.Ci && DWBNQ_IN_BOUNDS((qi + 3) - xbase, a.total_pos * a.Ci, a.flag))
                     ? pw_load4(qi)
                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        if (++kc_l == a.kchunks) {
          kc_l = 0;
          t_l += gridDim.x;
          if (t_l < a.total_tiles) locate();
        }
      };
      int s = 0;
      unsigned int ph = 0;
      auto store = [&](const float4(&v)[4]) -> bool {
        if (!pw_wait(&empty[s], ph ^ 1u) || *abort_v) return false;
        unsigned char *xh = sm + (size_t)s * a.stage_bytes + sw4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float4 *dst = reinterpret_cast<float4 *>(xh + i * 1024);
          if (MATH3) {
            float4 h;
            h.x = __uint_as_float(__float_as_uint(v[i].x) & 0xffffe000u);
            h.y = __uint_as_float(__float_as_uint(v[i].y) & 0xffffe000u);
            h.z = __uint_as_float(__float_as_uint(v[i].z) & 0xffffe000u);
            h.w = __uint_as_float(__float_as_uint(v[i].w) & 0xffffe000u);
            *dst = h;
            *reinterpret_cast<float4 *>(reinterpret_cast<unsigned char *>(dst) + off_xlo) =
                make_float4(__fsub_rn(v[i].x, h.x), __fsub_rn(v[i].y, h.y), __fsub_rn(v[i].z, h.z), __fsub_rn(v[i].w, h.w));
          } else {
            *dst = v[i];
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&split[s]);
        if (++s == a.stages) { s = 0; ph ^= 1u; }
        return true;
      };
      float4 va[4], vb[4];
      bool ok = true, have_a = t_l < a.total_tiles, have_b = false;
      if (have_a) {
        locate();
        load(va);
      }
      while (have_a) {
        have_b = t_l < a.total_tiles;
        if (have_b) load(vb);
        ok = store(va);
        if (!ok || !have_b) break;
        have_a = t_l < a.total_tiles;
        if (have_a) load(va);
        ok = store(vb);
        if (!ok) break;
      }
      if (!ok && lane == 0 && !*abort_v) { atomicExch(a.flag, 1); *abort_v = 1; }
    } else if (GATHER) {
      // Plain loads in place of TMA: the 128 rows of a tile are consecutive positions of the
      // batch flattened over (image, position), so a tile may straddle images and no lane is
      // wasted on planes whose size is not a multiple of 128 (or of 4, which TMA needs). Thread
      // (m, half) loads 16 of the chunk's 32 channels of position m - a warp reads 32
      // consecutive floats per channel - and stores the TF32 halves straight into the swizzled
      // operand layout the TMA path produces (32-byte units of a 128-byte row, XOR row mod 4).
      const int m = tid & 127, kh = tid >> 7;
      const unsigned int sw_base = (unsigned)((m >> 5) * 4096 + (m & 7) * 4);
      const unsigned int unit = (unsigned)((m >> 3) & 3);
      // The loads of a chunk are issued one chunk ahead of its stores (two register sets), so the
      // memory latency of chunk i + 1 runs under the barrier wait, the stores and the MMAs of
      // chunk i; the load cursor runs through the (tile, chunk) sequence on its own.
      int t_l = blockIdx.x, kc_l = 0;
      bool valid_l = false;
      const T *const xbase = static_cast<const T *>(a.x);
      const T *xp_l = xbase;
      auto locate = [&]() {
        const long long g = (long long)(t_l % a.per_ct) * kPwPosTile + m;
        valid_l = g < a.total_pos;
        const long long n = valid_l ? g / a.HW : 0;
        xp_l = xbase + (size_t)n * a.Ci * a.HW + (valid_l ? (int)(g - n * a.HW) : 0);
      };
      const size_t plane = (size_t)a.HW;
      auto load = [&](float(&v)[16]) {
        const int k0 = kc_l * kPwKChunk + kh * 16;
        const T *q = xp_l + (size_t)k0 * plane;
        if (valid_l && k0 + 16 <= a.Ci) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            v[j] = DWBNQ_IN_BOUNDS((q + j * plane) - xbase, a.total_pos * a.Ci, a.flag) ? Elem<T>::to_f32(__ldg(q + j * plane)) : 0.0f;
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            v[j] = (valid_l && k0 + j < a.Ci && DWBNQ_IN_BOUNDS((q + j * plane) - xbase, a.total_pos * a.Ci, a.flag))
                       ? Elem<T>::to_f32(__ldg(q + j * plane))
                       : 0.0f;
        }
        if (++kc_l == a.kchunks) {
          kc_l = 0;
          t_l += gridDim.x;
          if (t_l < a.total_tiles) locate();
        }
      };
      int s = 0;
      unsigned int ph = 0;
      auto store = [&](const float(&v)[16]) -> bool {
        if (!pw_wait(&empty[s], ph ^ 1u) || *abort_v) return false;
        // row k = 16 kh + j of the chunk: k mod 4 = j mod 4, so four base addresses serve all rows
        unsigned char *xh = sm + (size_t)s * a.stage_bytes + sw_base + kh * 2048;
        unsigned char *const rb[4] = {xh + ((unit ^ 0u) << 5), xh + ((unit ^ 1u) << 5), xh + ((unit ^ 2u) << 5),
                                      xh + ((unit ^ 3u) << 5)};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float *dst = reinterpret_cast<float *>(rb[j & 3] + j * 128);
          if (MATH3) {
            const float h = __uint_as_float(__float_as_uint(v[j]) & 0xffffe000u);
            *dst = h;
            *reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(dst) + off_xlo) = __fsub_rn(v[j], h);
          } else {
            *dst = v[j];
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&split[s]);
        if (++s == a.stages) { s = 0; ph ^= 1u; }
        return true;
      };
      float va[16], vb[16];
      bool ok = true, have_a = t_l < a.total_tiles, have_b = false;
      if (have_a) {
        locate();
        load(va);
      }
      while (have_a) {
        have_b = t_l < a.total_tiles;
        if (have_b) load(vb);
        ok = store(va);
        if (!ok || !have_b) break;
        have_a = t_l < a.total_tiles;
        if (have_a) load(va);
        ok = store(vb);
        if (!ok) break;
      }
      if (!ok && lane == 0 && !*abort_v) { atomicExch(a.flag, 1); *abort_v = 1; }
    } else if (MATH3) {
      // three-pass mode: x -> (x with the low 13 mantissa bits cleared, the exact rest), in place
      int s = 0;
      unsigned int ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < a.total_tiles; t += gridDim.x) {
        for (int kc = 0; kc < a.kchunks; ++kc) {
          ok = pw_wait(&full[s], ph) && !*abort_v;
          if (!ok) break;
          uint4 *xh = reinterpret_cast<uint4 *>(sm + (size_t)s * a.stage_bytes);
          uint4 *xl = reinterpret_cast<uint4 *>(sm + (size_t)s * a.stage_bytes + off_xlo);
#pragma unroll
          for (int i = tid; i < kPwXBytes / 16; i += 32 * kPwXWarps) {
            const uint4 v = xh[i];
            uint4 h, l;
            h.x = v.x & 0xffffe000u; h.y = v.y & 0xffffe000u; h.z = v.z & 0xffffe000u; h.w = v.w & 0xffffe000u;
            l.x = __float_as_uint(__fsub_rn(__uint_as_float(v.x), __uint_as_float(h.x)));
            l.y = __float_as_uint(__fsub_rn(__uint_as_float(v.y), __uint_as_float(h.y)));
            l.z = __float_as_uint(__fsub_rn(__uint_as_float(v.z), __uint_as_float(h.z)));
            l.w = __float_as_uint(__fsub_rn(__uint_as_float(v.w), __uint_as_float(h.w)));
            xh[i] = h;
            xl[i] = l;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(&split[s]);
          if (++s == a.stages) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok && lane == 0 && !*abort_v) { atomicExch(a.flag, 1); *abort_v = 1; }
    }
  } else {
    // ---- epilogue: groups of four warps; group g takes the tiles g, g + ngroups, ... of this CTA,
    // warp (group, quarter) the 32 positions in TMEM lanes [32 quarter, +32) with every column.
    // The buffer count is a multiple of ngroups, so every use of a buffer is awaited by the same
    // group in order: a barrier is never waited on more than one phase ahead (a parity wait
    // cannot tell phase k from phase k + 2).
    // With few tiles per CTA (col_split) that would leave most groups idle and one group alone
    // with the last tile - 7 us for 160 columns, a seventh of such a launch - so there every group
    // takes every tile, in order, and a quarter of its column units; all sixteen warps release
    // the buffer ----
    const int ew = warp - kPwFirstEpiWarp, quarter = warp & 3, group = ew >> 2;
    {
      // the coefficient table is the epilogue's alone: its sixteen warps build it while the loads
      // and the first MMAs are already under way, and meet at a barrier of their own
      bool all_safe = true;
      for (int i = threadIdx.x - 32 * kPwFirstEpiWarp; i < (cpad >> 1); i += 32 * kPwEpiWarps) {
        bool safe;
        table[i] = pw_make_pair(a, a.cstride, 2 * i, &safe);
        all_safe = all_safe && safe;
      }
      if (!all_safe) atomicOr(&unsafe_s, 1);
      asm volatile("bar.sync 1, %0;" ::"n"(32 * kPwEpiWarps) : "memory");
    }
    const f32x2 nz = negzero2();
    const FpqPacked fq = make_fpq_packed(a.q);
    const bool bn_safe = unsafe_s == 0;
    const bool cs = a.col_split != 0;
    const int b_step = cs ? 1 : a.ngroups;
    int b = cs ? 0 : group;  // tile i of this CTA lives in buffer i mod nacc; the group's tiles are b_step apart
    unsigned int aph = 0;
    const long long t_step = (long long)gridDim.x * b_step;
    for (long long tl = (long long)blockIdx.x + (cs ? 0LL : (long long)group * gridDim.x);
         (cs || group < a.ngroups) && tl < a.total_tiles; tl += t_step) {
      const int t = (int)tl;
      const int ct = t / a.per_ct;
      const int r = t - ct * a.per_ct;
      long long n;
      int p;
      bool p_ok;
      if (GATHER) {
        const long long g = (long long)r * kPwPosTile + quarter * 32 + lane;
        p_ok = g < a.total_pos;
        n = p_ok ? g / a.HW : 0;
        p = p_ok ? (int)(g - n * a.HW) : 0;
      } else {
        n = r / a.pos_tiles;
        p = (r - (int)n * a.pos_tiles) * kPwPosTile + quarter * 32 + lane;
        p_ok = p < a.HW;
      }
      if (!pw_wait(&acc_full[b], aph) || *abort_v) {
        if (lane == 0 && !*abort_v) { atomicExch(a.flag, 1); *abort_v = 1; }
        break;
      }
      tc_fence_after();
      const int c_first = ct * a.npad;
      int c_valid = a.Co - c_first;  // channels of this tile that exist
      if (c_valid > a.npad) c_valid = a.npad;
      const int units = (c_valid + 7) >> 3;  // warp-uniform
      const unsigned int taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + b * a.npad;
      T *img = static_cast<T *>(a.y) + ((size_t)n * a.Co + c_first) * a.HW + (p_ok ? p : 0);
      const size_t unit_stride = (size_t)8 * a.HW;
      const PwPair *tp = table + (c_first >> 1);
      if (!DWBNQ_IN_BOUNDS((c_first >> 1) + units * 4 - 1, cpad >> 1, a.flag)) break;
      int u0 = 0, u1 = units;  // this group's column units
      if (cs) {
        const int per_group = (units + kPwEpiGroups - 1) / kPwEpiGroups;
        u0 = group * per_group < units ? group * per_group : units;
        u1 = u0 + per_group < units ? u0 + per_group : units;
      }
      unsigned int acc0[8], acc1[8];
      if (u0 < u1) tc_ld8(taddr + u0 * 8, acc0);
      for (int u = u0; u < u1; u += 2) {
        tc_ld_wait8(acc0);
        if (u + 1 < u1) tc_ld8(taddr + (u + 1) * 8, acc1);
        float res[8];
        pw_finish_unit<EPI>(acc0, tp + u * 4, a, nz, fq, bn_safe, res);
        if (p_ok) {
          const int c0 = u * 8;
          T *q = img + (size_t)u * unit_stride;
          if (c0 + 8 <= c_valid) {
#pragma unroll
            for (int i = 0; i < 8; ++i) if (DWBNQ_IN_BOUNDS((q + (unsigned)(i * a.HW)) - static_cast<T *>(a.y), a.total_pos * a.Co, a.flag))
                  q[(unsigned)(i * a.HW)] = Elem<T>::from_f32(res[i]);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (c0 + i < c_valid) if (DWBNQ_IN_BOUNDS((q + (unsigned)(i * a.HW)) - static_cast<T *>(a.y), a.total_pos * a.Co, a.flag))
                  q[(unsigned)(i * a.HW)] = Elem<T>::from_f32(res[i]);
          }
        }
        if (u + 1 < u1) {
          tc_ld_wait8(acc1);
          if (u + 2 < u1) tc_ld8(taddr + (u + 2) * 8, acc0);
          pw_finish_unit<EPI>(acc1, tp + (u + 1) * 4, a, nz, fq, bn_safe, res);
          if (p_ok) {
            const int c0 = (u + 1) * 8;
            T *q = img + (size_t)(u + 1) * unit_stride;
            if (c0 + 8 <= c_valid) {
#pragma unroll
              for (int i = 0; i < 8; ++i) if (DWBNQ_IN_BOUNDS((q + (unsigned)(i * a.HW)) - static_cast<T *>(a.y), a.total_pos * a.Co, a.flag))
                  q[(unsigned)(i * a.HW)] = Elem<T>::from_f32(res[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (c0 + i < c_valid) if (DWBNQ_IN_BOUNDS((q + (unsigned)(i * a.HW)) - static_cast<T *>(a.y), a.total_pos * a.Co, a.flag))
                  q[(unsigned)(i * a.HW)] = Elem<T>::from_f32(res[i]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
      b += b_step;
      if (b >= a.nacc) { b -= a.nacc; aph ^= 1u; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPwTmemCols) : "memory");
  }
}

// ---- preparation: per-channel coefficients and the TF32 halves of the weights --------------------

template <typename T>
__global__ void pw_prepare_kernel(const T *w, const T *b, const T *beta, const T *gamma, const T *mean, const T *var,
                                  float eps, int Co, int cpad, long long wsize, float *coef, float *w_hi, float *w_lo,
                                  T *w_same) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cpad) {
    const bool in = i < Co;
    coef[i] = (in && b) ? Elem<T>::to_f32(b[i]) : 0.0f;
    coef[cpad + i] = in ? (mean ? Elem<T>::to_f32(mean[i]) : 0.0f) : -1.0f;  // a padded column normalises 0 to 1

    coef[2 * cpad + i] = (in && gamma) ? Elem<T>::to_f32(gamma[i]) : 1.0f;
    coef[3 * cpad + i] = (in && var) ? bn_stdvar(Elem<T>::to_f32(var[i]), eps) : 1.0f;
    coef[4 * cpad + i] = (in && beta) ? Elem<T>::to_f32(beta[i]) : 0.0f;
  }
  if (i < wsize) {
    const float v = Elem<T>::to_f32(w[i]);
    if (w_same) w_same[i] = w[i];  // binary16 tensors: the weights as they are, for the kind::f16 path
    if (w_lo) {  // the two TF32 halves
      const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
      w_hi[i] = h;
      w_lo[i] = __fsub_rn(v, h);
    } else {  // the fp32 value itself
      w_hi[i] = v;
    }
  }
}

// ---- plain FMA kernel (any shape, fp32 / fp16 tensors) -------------------------------------------
// 64 output channels x 64 positions per CTA, 4 x 4 outputs per thread, c_in in chunks of 16.

struct PwSimtArgs {
  const void *x;
  const float *w;  // fp32 copy in the workspace
  void *y;
  const float *coef;
  int HW, Ci, Co, cpad, pos_tiles;
  int *flag;
  int has_bn, act, qkind;
  QuantArgs q;
};

template <typename T>
__global__ void __launch_bounds__(256) pw_simt_kernel(const PwSimtArgs a) {
  __shared__ float ws[16][64 + 4], xs[16][64 + 4];
  const T *x = static_cast<const T *>(a.x);
  const float *w = a.w;
  T *y = static_cast<T *>(a.y);
  const long long n = blockIdx.x / a.pos_tiles;
  const int p0 = (int)(blockIdx.x - n * a.pos_tiles) * 64, c0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  const T *xn = x + (size_t)n * a.Ci * a.HW;
  for (int k0 = 0; k0 < a.Ci; k0 += 16) {
    for (int e = threadIdx.x; e < 16 * 64; e += 256) {
      const int k = e >> 6, j = e & 63;  // xs: positions contiguous in memory
      xs[k][j] = (k0 + k < a.Ci && p0 + j < a.HW &&
                  DWBNQ_IN_BOUNDS((xn - x) + (long long)(k0 + k) * a.HW + p0 + j, (long long)gridDim.x / a.pos_tiles * a.Ci * a.HW, a.flag))
                     ? Elem<T>::to_f32(xn[(size_t)(k0 + k) * a.HW + p0 + j])
                     : 0.0f;
      const int kk = e & 15, c = e >> 4;  // ws: c_in contiguous in memory
      ws[kk][c] = (k0 + kk < a.Ci && c0 + c < a.Co) ? w[(size_t)(c0 + c) * a.Ci + k0 + kk] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float wv[4], xv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { wv[i] = ws[k][ty * 4 + i]; xv[i] = xs[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(wv[i], xv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty * 4 + i;
    if (c >= a.Co) continue;
    const BnCoef bc{a.coef[a.cpad + c], a.coef[2 * a.cpad + c], a.coef[3 * a.cpad + c], a.coef[4 * a.cpad + c]};
    const float bias = a.coef[c];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = p0 + tx * 4 + j;
      if (p >= a.HW) continue;
      float v = __fadd_rn(acc[i][j], bias);
      if (a.has_bn) v = bn_apply(v, bc);
      v = pw_act(v, a.act);
      if (a.qkind == DWBNQ_Q_FPQ) v = fpq_apply(v, a.q);
      else if (a.qkind == DWBNQ_Q_POW2) v = pow2_apply(v, a.q);
      if (DWBNQ_IN_BOUNDS(((long long)n * a.Co + c) * a.HW + p, (long long)gridDim.x / a.pos_tiles * a.Co * a.HW, a.flag))
        y[((size_t)n * a.Co + c) * a.HW + p] = Elem<T>::from_f32(v);
    }
  }
}

// ---- host side -------------------------------------------------------------------------------------

typedef CUresult (*PwEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
PwEncodeFn pw_encode_fn() {
  static PwEncodeFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<PwEncodeFn>(p);
  }();
  return fn;
}

constexpr int kPwPathUnset = -2;
thread_local int t_forced_pw = kPwPathUnset;
thread_local int t_pw_max_ctas = 0;  // 0 = one CTA per SM

int forced_pw_path() {
  static const int env_default = [] {
    const char *e = std::getenv("DWBNQ_PW_FORCE");
    if (e && !std::strcmp(e, "simt")) return 0;
    if (e && !std::strcmp(e, "tc")) return 1;
    return -1;
  }();
  return t_forced_pw == kPwPathUnset ? env_default : t_forced_pw;
}

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct PwGeom {
  int npad, co_tiles, cpad;
};
// Equal channel tiles of at most `widest` columns, rounded up to the 32 columns the epilogue's
// units and the MMA shape want.
PwGeom pw_tiles(int Co, int widest) {
  PwGeom g;
  const int tiles = (Co + widest - 1) / widest;
  g.npad = ((Co + tiles - 1) / tiles + 31) / 32 * 32;
  g.co_tiles = (Co + g.npad - 1) / g.npad;
  g.cpad = g.co_tiles * g.npad;
  return g;
}
// Stride of the coefficient vectors in the workspace: covers either tiling, depends on c_out alone
// (a workspace prepared once serves every batch size).
int pw_coef_stride(int Co) {
  const int a = pw_tiles(Co, 128).cpad, b = pw_tiles(Co, kPwMaxCoTile).cpad;
  return a > b ? a : b;
}
// Channel tiles of up to 128 or up to 256 columns, whichever the launch finishes sooner with.
// A tile costs the longer of its sum (every chunk of 32 input channels about 1850 cycles of loads,
// splits and MMAs - wider tiles do that work for fewer tiles) and its epilogue (about 500 cycles
// per unit of 8 valid columns with all sixteen warps busy); the launch takes as many rounds of
// tiles as the SMs need for all of them. Measured on the layers of MobileNetV2 at 256 images:
// 160 -> 960 on 7x7 1.26x and 96 -> 576 on 14x14 1.21x with 256 (240 used) / 192 columns, 64 -> 384 on
// 14x14 0.95x with 192 (six rounds of 24 units against eight of 16) - the estimate ranks all three.
// Ties go to the wide tile for long sums (c_in >= 256), else to the narrow one.
PwGeom pw_geom(int Co, int Ci, long long total_pos, int sms) {
  const PwGeom narrow = pw_tiles(Co, 128), wide = pw_tiles(Co, kPwMaxCoTile);
  if (narrow.npad == wide.npad) return narrow;
  const long long pos_tiles = (total_pos + kPwPosTile - 1) / kPwPosTile;
  const long long kloop = (long long)((Ci + kPwKChunk - 1) / kPwKChunk) * 1850;
  auto cost = [&](const PwGeom &g) {
    const long long rounds = (g.co_tiles * pos_tiles + sms - 1) / sms;
    const long long epi = (long long)((Co + g.co_tiles - 1) / g.co_tiles + 7) / 8 * 500;
    return rounds * (kloop > epi ? kloop : epi);
  };
  const long long cn = cost(narrow), cw = cost(wide);
  return (Ci >= 256 ? cw <= cn : cw * 100 < cn * 97) ? wide : narrow;
}

int validate_pw(const dwbnq_pwconv_desc *d) {
  if (!d) return fail(DWBNQ_ERR_INVALID_ARG, "pointwise conv desc is null");
  if (d->dtype != DWBNQ_F32 && d->dtype != DWBNQ_F16)
    return fail(DWBNQ_ERR_INVALID_ARG, "dtype %d is neither DWBNQ_F32 nor DWBNQ_F16", d->dtype);
  if (d->n < 0 || d->c_in <= 0 || d->c_out <= 0 || d->h <= 0 || d->w <= 0)
    return fail(DWBNQ_ERR_INVALID_ARG, "shape [%lld,%d->%d,%d,%d] is not positive", (long long)d->n, d->c_in, d->c_out, d->h, d->w);
  if (d->math != DWBNQ_PW_MATH_FP32 && d->math != DWBNQ_PW_MATH_TF32)
    return fail(DWBNQ_ERR_INVALID_ARG, "math %d is not a dwbnq_pw_math", d->math);
  if (d->act < DWBNQ_ACT_NONE || d->act > DWBNQ_ACT_RELU6) return fail(DWBNQ_ERR_INVALID_ARG, "act %d is not a dwbnq_act", d->act);
  if ((long long)d->h * d->w > 0x7fffffffLL || d->n > 0x7fffffffLL)
    return fail(DWBNQ_ERR_UNSUPPORTED, "plane or batch beyond 2^31 - 1 elements");
  return DWBNQ_OK;
}

// Whether the activations can come in through TMA (plane pitch and base 16-byte aligned), or
// have to be gathered with plain loads.
bool pw_tma_x(const dwbnq_pwconv_desc &d, const void *x) {
  return ((long long)d.h * d.w) % 4 == 0 && ((uintptr_t)x & 15) == 0;
}
bool pw_tc_eligible(const dwbnq_pwconv_desc &d, const void *x, const void *w) {
  const long long hw = (long long)d.h * d.w;
  return d.c_in % 4 == 0 && d.c_out <= kPwMaxCout && (long long)d.c_out * hw <= 0x7fffffffLL &&
         d.n * hw <= (1LL << 40);
}

template <typename T, int GATHER, bool MATH3>
cudaError_t launch_pw_tc(int epi, dim3 grid, size_t smem, cudaStream_t stream, const CUtensorMap &tx, const CUtensorMap &tw,
                         const CUtensorMap &twl, const PwArgs &a) {
  void (*k)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const PwArgs) =
      epi == PW_EPI_BIAS ? pw_tc_kernel<T, GATHER, MATH3, PW_EPI_BIAS>
      : epi == PW_EPI_BN_FPQ ? pw_tc_kernel<T, GATHER, MATH3, PW_EPI_BN_FPQ>
      : epi == PW_EPI_BN_RELU6_FPQ ? pw_tc_kernel<T, GATHER, MATH3, PW_EPI_BN_RELU6_FPQ>
      : epi == PW_EPI_BN_FPQS ? pw_tc_kernel<T, GATHER, MATH3, PW_EPI_BN_FPQS> : pw_tc_kernel<T, GATHER, MATH3, PW_EPI_GENERIC>;
  // the opt-in to large dynamic shared memory is per function and per device
  static thread_local const void *attr_done[5] = {nullptr};
  static thread_local int attr_dev[5] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (attr_done[epi] != (const void *)k || attr_dev[epi] != dev + 1) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kPwSmemMax);
    if (e != cudaSuccess) return e;
    attr_done[epi] = (const void *)k;
    attr_dev[epi] = dev + 1;
  }
  return launch_pdl(k, grid, dim3(kPwThreads), smem, stream, tx, tw, twl, a);
}

// Which kernel and which arithmetic a descriptor gets: the same answer at preparation and at
// every forward call (the forced choice of include/dwbnq_debug.h must not change in between).
struct PwMode {
  bool tc, math3;
};
PwMode pw_mode(const dwbnq_pwconv_desc &d, const void *x, int *status) {
  const int forced = forced_pw_path();
  const bool eligible = pw_tc_eligible(d, x, nullptr);
  *status = DWBNQ_OK;
  if (forced == 1 && !eligible) *status = fail(DWBNQ_ERR_UNSUPPORTED, "the tcgen05 kernel cannot take this shape / alignment");
  PwMode m;
  m.tc = forced == 0 ? false : eligible;
  // binary16 factors are exact in TF32: one pass gives exact products
  m.math3 = m.tc && d.dtype == DWBNQ_F32 && d.math == DWBNQ_PW_MATH_FP32;
  return m;
}

// Everything about a launch of the tcgen05 kernel that follows from the descriptor, the
// alignment of x, the arithmetic and the device's SM count (max_ctas > 0 caps the grid: a test hook).
struct PwShape {
  PwGeom g;
  int xmode;       // PwXMode
  int pos_tiles, kchunks, per_ct, total_tiles;
  int stage_bytes, table_bytes, stages;
  int ngroups, nacc, grid, col_split;
};
int pw_shape(const dwbnq_pwconv_desc &d, const void *x, bool math3, int sms, int max_ctas, PwShape *out) {
  PwShape s;
  std::memset(&s, 0, sizeof(s));
  const int HW = d.h * d.w;
  const long long total_pos = d.n * HW;
  s.g = pw_geom(d.c_out, d.c_in, total_pos, sms);
  s.pos_tiles = (HW + kPwPosTile - 1) / kPwPosTile;
  s.kchunks = (d.c_in + kPwKChunk - 1) / kPwKChunk;
  // Gathered when TMA cannot take the plane, or when the per-image tiling would leave more than
  // a tenth of the accumulator rows empty (196 positions fill 1.53 tiles of 128); four positions
  // per load where every group of four lies in one image and is aligned.
  const bool vec4 = HW % 4 == 0 && ((uintptr_t)x & (d.dtype == DWBNQ_F16 ? 7 : 15)) == 0;
  bool scalar_gather = !vec4;
  bool gather = !pw_tma_x(d, x) || (long long)s.pos_tiles * kPwPosTile * 10 > (long long)HW * 11;
  if (d.dtype == DWBNQ_F16) {
    // binary16 tensors go through TMA (and stay binary16 in the MMA) where the rows of x and w are
    // multiples of 16 bytes; no worker touches them there, which is worth up to a seventh of empty rows (28 x 28)
    gather = HW % 8 != 0 || d.c_in % 8 != 0 || ((uintptr_t)x & 15) != 0 ||
             (long long)s.pos_tiles * kPwPosTile * 6 > (long long)HW * 7;
  }
  {
    // DWBNQ_PW_GATHER: 0 = TMA wherever it can be used, 1 = always gather, 2 = the one-element gather
    static const int env = [] {
      const char *e = std::getenv("DWBNQ_PW_GATHER");
      return e && (e[0] == '0' || e[0] == '1' || e[0] == '2') ? e[0] - '0' : -1;
    }();
    if (env == 1 || env == 2) gather = true;
    if (env == 2) scalar_gather = true;
    if (env == 0 && pw_tma_x(d, x) && d.dtype == DWBNQ_F32) gather = false;
  }
  if (!gather && d.dtype == DWBNQ_F16) s.kchunks = (d.c_in + 63) / 64;  // 64 binary16 channels per stage
  s.xmode = !gather ? PW_X_TMA : scalar_gather ? PW_X_GATHER : PW_X_GATHER4;
  {
    const long long per_ct = gather ? (total_pos + kPwPosTile - 1) / kPwPosTile : d.n * s.pos_tiles;
    const long long total = (long long)s.g.co_tiles * per_ct;
    if (total > 0x7fffffffLL) return fail(DWBNQ_ERR_UNSUPPORTED, "more than 2^31 - 1 tiles");
    s.total_tiles = (int)total;
    s.per_ct = (int)per_ct;
  }
  s.stage_bytes = (kPwXBytes + s.g.npad * 128) * (math3 ? 2 : 1);
  s.table_bytes = (s.g.cpad / 2) * (int)sizeof(PwPair);
  {
    const int fit = kPwTmemCols / s.g.npad < kPwMaxAcc ? kPwTmemCols / s.g.npad : kPwMaxAcc;
    s.ngroups = fit < kPwEpiGroups ? fit : kPwEpiGroups;
    s.nacc = fit / s.ngroups * s.ngroups;
  }
  s.stages = (kPwSmemMax - 1024 - s.table_bytes) / s.stage_bytes;
  if (s.stages > kPwMaxStages) s.stages = kPwMaxStages;
  if (s.stages < 2) return fail(DWBNQ_ERR_UNSUPPORTED, "pipeline stage of %d bytes does not fit twice", s.stage_bytes);
  s.grid = s.total_tiles < sms ? s.total_tiles : sms;
  if (max_ctas > 0 && s.grid > max_ctas) s.grid = max_ctas;
  // tiles of at least 64 columns, up to six per CTA or too wide for four accumulator buffers (a group
  // per buffer would leave groups idle): the groups share each tile's columns
  s.col_split = s.g.npad >= 64 && ((long long)s.total_tiles <= 6LL * s.grid || s.ngroups < kPwEpiGroups);
  *out = s;
  return DWBNQ_OK;
}

struct PwWorkspace {
  float *coef, *w_a, *w_b;  // coefficients; fp32 weights (or their TF32 high halves); the low halves
};
PwWorkspace pw_workspace(const dwbnq_pwconv_desc &d, void *workspace) {
  PwWorkspace w;
  w.coef = static_cast<float *>(workspace);
  w.w_a = reinterpret_cast<float *>(static_cast<char *>(workspace) + align256((size_t)5 * pw_coef_stride(d.c_out) * 4));
  w.w_b = reinterpret_cast<float *>(reinterpret_cast<char *>(w.w_a) + align256((size_t)d.c_in * d.c_out * 4));
  return w;
}

}  // namespace

int pwconv_prepare(const dwbnq_pwconv_desc &d, float bn_eps, const void *w, const void *b, const void *beta,
                   const void *gamma, const void *mean, const void *var, void *workspace, cudaStream_t stream) {
  if (mean && !var) return fail(DWBNQ_ERR_INVALID_ARG, "bn_var is null although bn_mean is given");
  if (!w || !workspace) return fail(DWBNQ_ERR_INVALID_ARG, "w and workspace must not be null");
  if ((uintptr_t)workspace & 255) return fail(DWBNQ_ERR_INVALID_ARG, "workspace must be 256-byte aligned");
  const int elem = d.dtype == DWBNQ_F32 ? 4 : 2;
  if ((uintptr_t)w & (elem - 1)) return fail(DWBNQ_ERR_INVALID_ARG, "w must be element-aligned");
  int st;
  const PwMode m = pw_mode(d, reinterpret_cast<const void *>(16), &st);  // the arithmetic does not depend on x
  if (st != DWBNQ_OK) return st;
  const int cstride = pw_coef_stride(d.c_out);
  const PwWorkspace ws = pw_workspace(d, workspace);
  const long long wsize = (long long)d.c_in * d.c_out;
  const long long work = wsize > cstride ? wsize : cstride;
  const unsigned blocks = (unsigned)((work + 255) / 256);
  if (d.dtype == DWBNQ_F32)
    pw_prepare_kernel<float><<<blocks, 256, 0, stream>>>(
        static_cast<const float *>(w), static_cast<const float *>(b), static_cast<const float *>(beta),
        static_cast<const float *>(gamma), static_cast<const float *>(mean), static_cast<const float *>(var), bn_eps,
        d.c_out, cstride, wsize, ws.coef, ws.w_a, m.math3 ? ws.w_b : nullptr, nullptr);
  else
    pw_prepare_kernel<__half><<<blocks, 256, 0, stream>>>(
        static_cast<const __half *>(w), static_cast<const __half *>(b), static_cast<const __half *>(beta),
        static_cast<const __half *>(gamma), static_cast<const __half *>(mean), static_cast<const __half *>(var), bn_eps,
        d.c_out, cstride, wsize, ws.coef, ws.w_a, nullptr, reinterpret_cast<__half *>(ws.w_b));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "pw_prepare_kernel launch");
  return DWBNQ_OK;
}

int pwconv_run(const dwbnq_pwconv_desc &d, const dwbnq_quant_desc *q, int has_bn, const void *x, void *y,
               void *workspace, int dev, cudaStream_t stream) {
  const int kind = q ? q->kind : DWBNQ_Q_NONE;
  if (kind != DWBNQ_Q_NONE && kind != DWBNQ_Q_FPQ && kind != DWBNQ_Q_POW2)
    return fail(DWBNQ_ERR_UNSUPPORTED, "pointwise convolution fuses FixedPointQuantize or Pow2Quantize only (kind %d)", kind);
  if (d.n == 0) return DWBNQ_OK;
  if (!x || !y || !workspace) return fail(DWBNQ_ERR_INVALID_ARG, "x, y and workspace must not be null");
  if ((uintptr_t)workspace & 255) return fail(DWBNQ_ERR_INVALID_ARG, "workspace must be 256-byte aligned");
  const int elem = d.dtype == DWBNQ_F32 ? 4 : 2;
  if (((uintptr_t)x | (uintptr_t)y) & (elem - 1)) return fail(DWBNQ_ERR_INVALID_ARG, "tensor pointers must be element-aligned");

  QuantArgs qa;
  std::memset(&qa, 0, sizeof(qa));
  int st = DWBNQ_OK;
  if (kind == DWBNQ_Q_FPQ) st = fill_fpq(&qa, q->sign, q->n, q->delta);
  else if (kind == DWBNQ_Q_POW2) st = fill_pow2(&qa, q->sign, q->with_zero, q->n, q->m, dev);
  if (st != DWBNQ_OK) return st;

  const int HW = d.h * d.w;
  const PwWorkspace wsp = pw_workspace(d, workspace);
  float *coef = wsp.coef, *w_hi = wsp.w_a, *w_lo = wsp.w_b;
  const PwMode mode = pw_mode(d, x, &st);
  if (st != DWBNQ_OK) return st;
  const bool tc = mode.tc, math3 = mode.math3;
  const void *mean = has_bn ? coef : nullptr;  // only its presence matters below

  if (!tc) {
    PwSimtArgs a;
    std::memset(&a, 0, sizeof(a));
    a.x = x; a.w = w_hi; a.y = y; a.coef = coef;
    a.HW = HW; a.Ci = d.c_in; a.Co = d.c_out; a.cpad = pw_coef_stride(d.c_out);
    a.pos_tiles = (HW + 63) / 64;
    a.has_bn = mean != nullptr; a.act = d.act; a.qkind = kind; a.q = qa;
    st = device_flag_ptr(dev, &a.flag);
    if (st != DWBNQ_OK) return st;
    const long long gx = d.n * a.pos_tiles;
    if (gx > 0x7fffffffLL) return fail(DWBNQ_ERR_UNSUPPORTED, "batch x position tiles beyond 2^31 - 1");
    const dim3 grid((unsigned)gx, (unsigned)((d.c_out + 63) / 64));
    if (d.dtype == DWBNQ_F32) pw_simt_kernel<float><<<grid, 256, 0, stream>>>(a);
    else pw_simt_kernel<__half><<<grid, 256, 0, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, "pw_simt_kernel launch");
    return DWBNQ_OK;
  }

  PwShape sh;
  st = pw_shape(d, x, math3, sm_count(dev), t_pw_max_ctas, &sh);
  if (st != DWBNQ_OK) return st;
  const PwGeom g = sh.g;
  const bool gather = sh.xmode != PW_X_TMA, scalar_gather = sh.xmode == PW_X_GATHER;
  PwArgs a;
  std::memset(&a, 0, sizeof(a));
  a.HW = HW; a.Ci = d.c_in; a.Co = d.c_out; a.N = d.n;
  a.npad = g.npad; a.co_tiles = g.co_tiles;
  a.pos_tiles = sh.pos_tiles;
  a.kchunks = sh.kchunks;
  a.x = x;
  a.total_pos = d.n * HW;
  a.total_tiles = sh.total_tiles;
  a.per_ct = sh.per_ct;
  a.stage_bytes = sh.stage_bytes;
  const int table_bytes = sh.table_bytes;
  a.ngroups = sh.ngroups;
  a.nacc = sh.nacc;
  a.stages = sh.stages;
  a.col_split = sh.col_split;
  a.coef = coef;
  a.cstride = pw_coef_stride(d.c_out);
  a.y = y;
  st = device_flag_ptr(dev, &a.flag);
  if (st != DWBNQ_OK) return st;
  a.has_bn = mean != nullptr; a.act = d.act; a.qkind = kind; a.q = qa;
  PwEncodeFn enc = pw_encode_fn();
  if (!enc) return fail(DWBNQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMap tx, tw, twl;
  std::memset(&tx, 0, sizeof(tx));
  const bool f16mma = !gather && d.dtype == DWBNQ_F16;  // binary16 operands through TMA, kind::f16
  if (f16mma) {
    const cuuint64_t gdim[3] = {(cuuint64_t)HW, (cuuint64_t)d.c_in, (cuuint64_t)d.n};
    const cuuint64_t gstr[2] = {(cuuint64_t)HW * 2, (cuuint64_t)HW * d.c_in * 2};
    const cuuint32_t box[3] = {64, 64, 1}, es[3] = {1, 1, 1};
    CUresult r = enc(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(x), gdim, gstr, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DWBNQ_ERR_CUDA, "cuTensorMapEncodeTiled(x, binary16) failed with CUresult %d", (int)r);
    const cuuint64_t wdim[2] = {(cuuint64_t)d.c_in, (cuuint64_t)d.c_out};
    const cuuint64_t wstr[1] = {(cuuint64_t)d.c_in * 2};
    const cuuint32_t wbox[2] = {64, (cuuint32_t)g.npad}, wes[2] = {1, 1};
    r = enc(&tw, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w_lo /* the binary16 copy */, wdim, wstr, wbox, wes,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DWBNQ_ERR_CUDA, "cuTensorMapEncodeTiled(w, binary16) failed with CUresult %d", (int)r);
    twl = tw;
  } else if (!gather) {
    const cuuint64_t gdim[3] = {(cuuint64_t)HW, (cuuint64_t)d.c_in, (cuuint64_t)d.n};
    const cuuint64_t gstr[2] = {(cuuint64_t)HW * 4, (cuuint64_t)HW * d.c_in * 4};
    const cuuint32_t box[3] = {32, (cuuint32_t)kPwKChunk, 1}, es[3] = {1, 1, 1};
    const CUresult r = enc(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(x), gdim, gstr, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DWBNQ_ERR_CUDA, "cuTensorMapEncodeTiled(x) failed with CUresult %d", (int)r);
  }
  for (int k = 0; k < 2 && !f16mma; ++k) {
    const void *src = (k && math3) ? w_lo : w_hi;
    const cuuint64_t gdim[2] = {(cuuint64_t)d.c_in, (cuuint64_t)d.c_out};
    const cuuint64_t gstr[1] = {(cuuint64_t)d.c_in * 4};
    const cuuint32_t box[2] = {(cuuint32_t)kPwKChunk, (cuuint32_t)g.npad}, es[2] = {1, 1};
    const CUresult r = enc(k ? &twl : &tw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(src), gdim, gstr, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DWBNQ_ERR_CUDA, "cuTensorMapEncodeTiled(w) failed with CUresult %d", (int)r);
  }
  int epi = PW_EPI_GENERIC;
  const bool fpq_u = kind == DWBNQ_Q_FPQ && qa.fpq_fast && qa.fpq_min == 0.0f;
  if (!a.has_bn && kind == DWBNQ_Q_NONE && d.act == DWBNQ_ACT_NONE) epi = PW_EPI_BIAS;
  else if (a.has_bn && fpq_u && d.act == DWBNQ_ACT_NONE) epi = PW_EPI_BN_FPQ;
  else if (a.has_bn && kind == DWBNQ_Q_FPQ && qa.fpq_fast && qa.fpq_min < 0.0f && d.act == DWBNQ_ACT_NONE) epi = PW_EPI_BN_FPQS;
  // ReLU6 yields a value in [0, 6] (a NaN becomes 0): inside an unsigned range that reaches 6 the
  // quantizer's own clamps change nothing
  else if (a.has_bn && fpq_u && d.act == DWBNQ_ACT_RELU6 && qa.fpq_max >= 6.0f) epi = PW_EPI_BN_RELU6_FPQ;
  const size_t smem = (size_t)a.stages * a.stage_bytes + table_bytes + 1024;
  const dim3 gd((unsigned)sh.grid);
  const cudaError_t e = f16mma ? launch_pw_tc<__half, PW_X_TMA, false>(epi, gd, smem, stream, tx, tw, twl, a)
                        : d.dtype == DWBNQ_F16
                            ? (scalar_gather ? launch_pw_tc<__half, PW_X_GATHER, false>(epi, gd, smem, stream, tx, tw, twl, a)
                                             : launch_pw_tc<__half, PW_X_GATHER4, false>(epi, gd, smem, stream, tx, tw, twl, a))
                        : gather && scalar_gather
                            ? (math3 ? launch_pw_tc<float, PW_X_GATHER, true>(epi, gd, smem, stream, tx, tw, twl, a)
                                     : launch_pw_tc<float, PW_X_GATHER, false>(epi, gd, smem, stream, tx, tw, twl, a))
                        : gather ? (math3 ? launch_pw_tc<float, PW_X_GATHER4, true>(epi, gd, smem, stream, tx, tw, twl, a)
                                          : launch_pw_tc<float, PW_X_GATHER4, false>(epi, gd, smem, stream, tx, tw, twl, a))
                                 : (math3 ? launch_pw_tc<float, PW_X_TMA, true>(epi, gd, smem, stream, tx, tw, twl, a)
                                          : launch_pw_tc<float, PW_X_TMA, false>(epi, gd, smem, stream, tx, tw, twl, a));
  if (e != cudaSuccess) return fail_cuda(e, "pw_tc_kernel launch");
  return DWBNQ_OK;
}

int launch_pwconv(const dwbnq_pwconv_desc &d, float bn_eps, const dwbnq_quant_desc *q, const void *x, const void *w,
                  const void *b, const void *beta, const void *gamma, const void *mean, const void *var, void *y,
                  void *workspace, int dev, cudaStream_t stream) {
  if (d.n == 0) return DWBNQ_OK;
  const int st = pwconv_prepare(d, bn_eps, w, b, beta, gamma, mean, var, workspace, stream);
  if (st != DWBNQ_OK) return st;
  return pwconv_run(d, q, mean != nullptr, x, y, workspace, dev, stream);
}

size_t pwconv_workspace_bytes(const dwbnq_pwconv_desc &d) {
  return align256((size_t)5 * pw_coef_stride(d.c_out) * 4) + 2 * align256((size_t)d.c_in * d.c_out * 4);
}
int pwconv_validate(const dwbnq_pwconv_desc *d) { return validate_pw(d); }
int pwconv_path(const dwbnq_pwconv_desc &d, const void *x, const void *w) {
  const int forced = forced_pw_path();
  (void)w;
  return forced == 0 ? 0 : (pw_tc_eligible(d, x, nullptr) ? 1 : 0);
}
int pwconv_tiling(const dwbnq_pwconv_desc &d, const void *x, int sms, int out[8]) {
  int st;
  const PwMode m = pw_mode(d, x, &st);
  if (st != DWBNQ_OK) return st;
  if (!m.tc) return fail(DWBNQ_ERR_UNSUPPORTED, "the descriptor goes to the plain FMA kernel, which has no tiling to report");
  PwShape s;
  st = pw_shape(d, x, m.math3, sms, t_pw_max_ctas, &s);
  if (st != DWBNQ_OK) return st;
  out[0] = s.g.npad; out[1] = s.g.co_tiles; out[2] = s.xmode; out[3] = s.total_tiles;
  out[4] = s.grid; out[5] = s.stages; out[6] = s.nacc; out[7] = s.col_split;
  return DWBNQ_OK;
}
void set_forced_pw_path(int p) { t_forced_pw = p; }
void set_pw_max_ctas(int n) { t_pw_max_ctas = n; }

}  // namespace dwbnq
