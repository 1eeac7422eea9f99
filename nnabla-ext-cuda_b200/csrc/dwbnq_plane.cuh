// Fused dw-conv(3x3, pad 1) -> BN -> quantizer for SMALL planes (7x7, 14x14, 28x28), where
// a row is narrower than a warp's worth of 16-byte vectors (and, for 7 / 14, its pitch is
// not a multiple of 16 bytes), so the strip decomposition of the tiled family wastes most
// of its instructions on halo tests and partial stores.
//
// One warp = one CTA = P consecutive (n, c) planes, which are contiguous in memory:
//   * lane 0 brings the whole tile in with ONE bulk async copy and, at the end, sends the
//     finished tile out with ONE bulk async store: global memory only ever sees full,
//     contiguous lines;
//   * stride 1 (fused_plane_kernel): a thread owns a block of R = 7 rows x W (7 or 14)
//     columns of one plane. Input rows stream through it one at a time: the row is loaded
//     from shared memory once, as pairs of horizontally adjacent elements, and feeds the
//     three output rows it touches (finishing row i-1, continuing row i, starting row i+1 -
//     which keeps every output's summation in the ky-major / kx-minor order of the
//     contract). Only two accumulator rows are live, the loop over rows is rolled (two
//     steps per trip) and there is no per-element halo test: plane-edge columns are
//     compile-time or per-thread predicated operands, the zero rows a predicated load.
//     Results overwrite the tile in place. Rows / columns read by one thread and written by
//     another are its neighbours' edges: the row below a block is copied to a private stash
//     before anything is written, the row above is read in the first step, neighbouring
//     columns are read one step before their owner overwrites them, and every step has a
//     warp barrier between its reads and its writes;
//   * stride 2 (fused_plane_s2_kernel): a thread owns a 14 x 14 input block = 7 x 7 outputs
//     and streams two input rows per output row; the (4x smaller) result goes to its own
//     compact tile.
// Arithmetic contract: the one of dwbnq_fused.cuh (bias-initialised accumulator, separately
// rounded product and sum, BN and quantizer of dwbnq_device.cuh). Halo taps enter as
// w * (+0.0); planes where that differs from skipping the tap (bias == -0.0, non-finite
// weights) are re-evaluated tap by tap by their threads after the fast pass.
#pragma once

#include "dwbnq_fused.cuh"

namespace dwbnq {

struct PlaneCfg {
  int P;        // planes per CTA = 32 / NRB
  int n_tiles;  // CTAs
  int bulk;     // x and y 16-byte aligned: the bulk copy engine may be used
};

constexpr int kPlaneRows = 7;  // rows per thread

// Stash row of a thread: [2 unused | left halo | W elements | right halo | pad], even size.
__host__ __device__ constexpr int plane_stash_elems(int W) { return (W + 4 + 1) / 2 * 2; }
// stride 1: tile | stash (NRB > 1) | weight pairs, row of zeros (5x5) | 8-bit codes of the
// tile (8-bit storage) | mbarrier
__host__ __device__ constexpr size_t plane_smem_bytes(int K, int W, int NRB, int NCB, int NBND, int elem_size,
                                                      bool code8 = false) {
  const int P = 32 / (NRB * NCB);
  const size_t tile_elems = (size_t)P * (kPlaneRows * NRB + (NBND > 1 ? 2 * (K / 2) : 0)) * (W * NCB);
  size_t s = tile_elems * elem_size;
  s = (s + 15) / 16 * 16;
  if (NRB > 1) s += (size_t)32 * (K / 2) * plane_stash_elems(W) * elem_size;
  s = (s + 15) / 16 * 16;
  if (K == 5) s += (size_t)P * 25 * 8 + 128;  // weight pairs, row of zeros
  if (code8) s += (tile_elems + 15) / 16 * 16;
  return s + 16;
}
// stride 2: input tile (with the row above a band) | output tile | codes (8-bit storage) | mbarrier
__host__ __device__ constexpr size_t plane_s2_smem_bytes(int NRB, int NCB, int NBND, int elem_size,
                                                         bool code8 = false) {
  const int P = 32 / (NRB * NCB);
  const size_t tile_elems = (size_t)P * (14 * NRB + (NBND > 1 ? 1 : 0)) * (14 * NCB);
  size_t s = tile_elems * elem_size;
  s = (s + 15) / 16 * 16;
  s += (size_t)P * (7 * NRB) * (7 * NCB) * elem_size;
  s = (s + 15) / 16 * 16;
  if (code8) s += (tile_elems + 15) / 16 * 16;
  return s + 16;
}

// ---- 8-bit storage: the tile travels as one byte per element ------------------------------
// The copy engine moves the codes; the warp expands them to fp32 in shared memory before the
// (unchanged) computation and packs the quantized results back to codes after it.
// n codes at src -> n floats at dst, value = code * delta. src 4-byte, dst 16-byte aligned.
// A byte b placed in the low mantissa bits of 2^23 is the float 2^23 + b, so
// fma(2^23 + b, delta, -2^23 * delta) = RN(b * delta): the conversion and the scaling are one
// instruction, bit-identical to (float)b * delta. Signed codes enter as b ^ 0x80 = code + 128.
__device__ __forceinline__ void plane_expand_codes(const unsigned char *src, float *dst, int n, float delta,
                                                   bool is_signed, int lane) {
  // (2^23 + 128) * delta is exact only for a power-of-two delta: other signed steps go one by one
  if (is_signed && (__float_as_uint(delta) & 0x007fffffu) != 0u) {
    for (int i = lane; i < n; i += 32) dst[i] = __fmul_rn((float)(signed char)src[i], delta);
    return;
  }
  const int nv = n >> 2;
  const unsigned int *s4 = reinterpret_cast<const unsigned int *>(src);
  float4 *d4 = reinterpret_cast<float4 *>(dst);
  const unsigned int flip = is_signed ? 0x80808080u : 0u;
  const float off = __fmul_rn(is_signed ? -8388736.0f : -8388608.0f, delta);  // -(2^23 [+ 128]) * delta
  for (int i = lane; i < nv; i += 32) {
    const unsigned int u = s4[i] ^ flip;
    float4 f;
    f.x = __fmaf_rn(__uint_as_float(__byte_perm(u, 0x4b000000u, 0x7440)), delta, off);
    f.y = __fmaf_rn(__uint_as_float(__byte_perm(u, 0x4b000000u, 0x7441)), delta, off);
    f.z = __fmaf_rn(__uint_as_float(__byte_perm(u, 0x4b000000u, 0x7442)), delta, off);
    f.w = __fmaf_rn(__uint_as_float(__byte_perm(u, 0x4b000000u, 0x7443)), delta, off);
    d4[i] = f;
  }
  for (int i = (nv << 2) + lane; i < n; i += 32) {
    const unsigned int b = (unsigned int)src[i] ^ (flip & 0xffu);
    dst[i] = __fmaf_rn(__uint_as_float(0x4b000000u | b), delta, off);
  }
}
// n quantized values k * delta at src -> their codes k (low 8 bits of the integer: int8 and
// uint8 alike) at dst. src 16-byte, dst 4-byte aligned. k = v * inv_delta is exact and
// |k| < 2^8, so fma(v, inv_delta, 1.5 * 2^23) holds k in its low mantissa byte (two's
// complement); a NaN has no code and is stored as 0.
__device__ __forceinline__ unsigned int plane_code_bits(float v, float inv_delta) {
  const float t = __fmaf_rn(v, inv_delta, 12582912.0f);
  return __float_as_uint(v == v ? t : 12582912.0f);
}
__device__ __forceinline__ void plane_pack_codes(const float *src, unsigned char *dst, int n, float inv_delta,
                                                 int lane) {
  const int nv = n >> 2;
  const float4 *s4 = reinterpret_cast<const float4 *>(src);
  unsigned int *d4 = reinterpret_cast<unsigned int *>(dst);
  for (int i = lane; i < nv; i += 32) {
    const float4 f = s4[i];
    const unsigned int lo = __byte_perm(plane_code_bits(f.x, inv_delta), plane_code_bits(f.y, inv_delta), 0x0040);
    const unsigned int hi = __byte_perm(plane_code_bits(f.z, inv_delta), plane_code_bits(f.w, inv_delta), 0x0040);
    d4[i] = __byte_perm(lo, hi, 0x5410);
  }
  for (int i = (nv << 2) + lane; i < n; i += 32) dst[i] = (unsigned char)(plane_code_bits(src[i], inv_delta) & 0xffu);
}

// Bulk async store shared -> global of `bytes` (multiple of 16, both sides 16-byte
// aligned); returns when the engine has read the shared-memory source.
__device__ __forceinline__ void bulk_store_1d_and_wait(void *dst, const void *src_smem,
                                                       unsigned int bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// One row of W elements at p (shared memory) as 2*NP floats, zeros beyond W and for
// !valid. Even W: pairs are 8-byte (float) / 4-byte (half) aligned and loaded whole.
template <typename T, int W>
__device__ __forceinline__ void plane_load_row(const T *p, bool valid, float *xv) {
  constexpr int NP = (W + 1) / 2;
  if (W % 2 == 0) {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      float2 t = make_float2(0.0f, 0.0f);
      if (valid) {
        if (sizeof(T) == 4) t = *reinterpret_cast<const float2 *>(p + 2 * j);
        else t = __half22float2(*reinterpret_cast<const __half2 *>(p + 2 * j));
      }
      xv[2 * j] = t.x;
      xv[2 * j + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j) xv[j] = valid ? Elem<T>::to_f32(p[j]) : 0.0f;
    xv[W] = 0.0f;
  }
}

template <typename T, int W>
__device__ __forceinline__ void plane_store_row(T *p, const float *o) {
  constexpr int NP = (W + 1) / 2;
  if (W % 2 == 0) {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      if (sizeof(T) == 4) *reinterpret_cast<float2 *>(p + 2 * j) = make_float2(o[2 * j], o[2 * j + 1]);
      else *reinterpret_cast<__half2 *>(p + 2 * j) = __floats2half2_rn(o[2 * j], o[2 * j + 1]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j) p[j] = Elem<T>::from_f32(o[j]);
  }
}

// Tap-by-tap evaluation of a rows x cols block of outputs of one plane from global memory
// (the rare planes whose halo taps must be skipped rather than added as zeros). Kept out of
// line: it is cold and several times the size of the fast path.
template <typename T, int QM>
__device__ __noinline__ void plane_exact_block(const FusedArgs &a, int plane, int ch, int oy0,
                                               int ox0, int nrows, int ncols, T *dst, int pitch,
                                               const MmCoef &mm, float *lo_out, float *hi_out) {
  float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
  const long long n = plane / a.OC;
#pragma unroll 1
  for (int r = 0; r < nrows; ++r) {
#pragma unroll 1
    for (int j = 0; j < ncols; ++j) {
      const float v = prequant_point<T>(a, n, ch, oy0 + r, ox0 + j);
      if (qm_reduces(QM)) {
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
      }
      if (qm_stores(QM)) dst[r * pitch + j] = Elem<T>::from_f32(quant_apply<QM>(v, a.q, mm));
    }
  }
  *lo_out = lo;
  *hi_out = hi;
}

// Quantizer epilogue on N values held in registers (QM_MM_REDUCE does not come here).
template <int QM, int N>
__device__ __forceinline__ void plane_quant(float *o, const QuantArgs &q, const MmCoef &mm) {
  if (QM == QM_FPQ_LEAN) {
    const FpqPacked f = make_fpq_packed(q);
#pragma unroll
    for (int p = 0; p < N / 2; ++p)
      unpack2(fpq_apply_fast_unsigned2(o[2 * p], o[2 * p + 1], q, f), o[2 * p], o[2 * p + 1]);
    if (N % 2) o[N - 1] = fpq_apply_fast<false>(o[N - 1], q);
  } else if (QM == QM_FPQ && q.fpq_fast) {
    if (q.fpq_min < 0.0f) {
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = fpq_apply_fast<true>(o[j], q);
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) o[j] = fpq_apply_fast<false>(o[j], q);
    }
  } else if (QM == QM_POW2) {
    pow2_apply_n<N>(o, q);
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) o[j] = quant_apply<QM>(o[j], q, mm);
  }
}

// Per-plane min / max of a thread group of TPP lanes (aligned, power of two) into the
// encoded per-channel slots. NaN never enters (fminf / fmaxf drop it), matching the
// element-wise reduction.
template <int TPP>
__device__ __forceinline__ void plane_reduce_minmax(const QuantArgs &q, int ch, float lo, float hi,
                                                    bool active, int lane) {
#pragma unroll
  for (int o = 1; o < TPP; o <<= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if (active && (lane % TPP) == 0) {
    atomicMin(q.mm_enc_min + ch, enc_ordered(lo));
    atomicMax(q.mm_enc_max + ch, enc_ordered(hi));
  }
}

// One tap on the accumulator. The contract rounds the product and the sum separately. For
// binary16 inputs the fp32 product of two 11-bit significands is exact (22 bits, and the
// exponent range of half squared stays inside fp32's normal range), so the fused
// multiply-add RN(w * x + acc) is bit for bit RN(RN(w * x) + acc) and one instruction does
// the work of two.
template <typename T>
__device__ __forceinline__ float tap_add(float acc, float w, float x) {
  if (sizeof(T) == 2) return __fmaf_rn(w, x, acc);
  return __fadd_rn(acc, __fmul_rn(w, x));
}
template <typename T>
__device__ __forceinline__ f32x2 tap_add2(f32x2 acc, f32x2 w, f32x2 x, f32x2 nz) {
  if (sizeof(T) == 2) return fma2(w, x, acc);
  return add2(acc, mul2(w, x, nz));
}

// ---- stride 1 ---------------------------------------------------------------------------
// Thread block of R x W outputs; a tile is NRB blocks high and NCB blocks wide. With
// NBND == 1 the tile is a whole plane (and a CTA takes 32 / (NRB * NCB) planes); with
// NBND > 1 a plane is cut into NBND bands of full-width rows, one band per CTA, and the
// copy brings the row above and the row below the band along (they are contiguous with it).
// Compiled for 16 one-warp CTAs per SM (128 registers).
template <typename T, int W, int NRB, int NCB, int NBND, int QM, bool IO8 = false>
__global__ void __launch_bounds__(32, 16)
    fused_plane_kernel(const __grid_constant__ FusedArgs a, const PlaneCfg c) {
  static_assert(NCB == 1 || W % 2 == 0, "column blocks need an even block width");
  static_assert(NBND == 1 || NRB * NCB == 32, "a band is one warp's worth of blocks");
  static_assert(!IO8 || (sizeof(T) == 4 && (QM == QM_FPQ || QM == QM_FPQ_LEAN)),
                "8-bit storage: fp32 arithmetic, FixedPointQuantize codes");
  constexpr int R = kPlaneRows;
  constexpr int TB = R * NRB;        // rows per tile
  constexpr int H = TB * NBND;       // plane height
  constexpr int PW = W * NCB;        // plane width
  constexpr int PE = H * PW;         // elements per plane
  constexpr int HALO = NBND > 1 ? 1 : 0;  // row slots above / below the band
  constexpr int TE = (TB + 2 * HALO) * PW;  // shared-memory elements per plane of the tile
  constexpr int NP = (W + 1) / 2;    // output pairs per row
  constexpr int TPP = NRB * NCB;     // threads per plane
  constexpr int P = 32 / TPP;        // planes per CTA
  constexpr int SW = plane_stash_elems(W);

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *tile = reinterpret_cast<T *>(smem_raw);
  constexpr size_t tile_bytes = ((size_t)P * TE * sizeof(T) + 15) / 16 * 16;
  T *stash = reinterpret_cast<T *>(smem_raw + tile_bytes);
  constexpr size_t stash_bytes = NRB > 1 ? ((size_t)32 * SW * sizeof(T) + 15) / 16 * 16 : 0;
  // 8-bit storage: the codes of the tile, same element layout as the tile, one byte each
  unsigned char *codes = smem_raw + tile_bytes + stash_bytes;
  constexpr size_t codes_bytes = IO8 ? ((size_t)P * TE + 15) / 16 * 16 : 0;
  unsigned long long *bar =
      reinterpret_cast<unsigned long long *>(smem_raw + tile_bytes + stash_bytes + codes_bytes);
  constexpr int ESZ = IO8 ? 1 : (int)sizeof(T);  // bytes per element in global memory

  const int lane = threadIdx.x;
  const int n_planes = (int)(a.n * a.OC);
  const int plane0 = (NBND > 1 ? blockIdx.x / NBND : blockIdx.x) * P;
  const int r0 = NBND > 1 ? (blockIdx.x % NBND) * TB : 0;  // first plane row of the tile
  const int pv = min(P, n_planes - plane0);
  // what comes in (band: with the rows above / below it that exist) and what goes out
  const int in_first = NBND > 1 ? max(r0 - 1, 0) : 0;
  const int in_rows = NBND > 1 ? min(r0 + TB + 1, H) - in_first : pv * H;
  const unsigned char *in_src = static_cast<const unsigned char *>(a.x) +
                                ((long long)plane0 * PE + (long long)in_first * PW) * ESZ;
  const int in_off = NBND > 1 ? (in_first - (r0 - 1)) * PW : 0;  // tile element the copy starts at
  T *in_dst = tile + in_off;
  const int n_in = in_rows * PW, n_out = (NBND > 1 ? TB : pv * H) * PW;
  const unsigned int bytes = (unsigned int)(n_in * ESZ);
  const unsigned int obytes = (unsigned int)(n_out * ESZ);
  const bool async_tile = c.bulk != 0 && (bytes % 16) == 0 && (obytes % 16) == 0;

  pdl_launch_dependents();
  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  pdl_wait_for_predecessor();  // nothing global is read or written before this point
  if (lane == 0) {
    if (async_tile) {
      mbar_expect_tx(bar, bytes);
      if (IO8) bulk_load_1d(codes + in_off, in_src, bytes, bar);
      else bulk_load_1d(in_dst, in_src, bytes, bar);
    }
  }

  // ---- this thread's plane, block and per-channel operands (the copy is in flight) -------
  const int pl = lane / TPP;
  const int rb = (lane / NCB) % NRB;
  const int cb = lane % NCB;
  const bool active = pl < pv;
  const int plane = active ? plane0 + pl : n_planes - 1;
  const int ch = plane % a.OC;
  const bool has_left = NCB > 1 && cb > 0;
  const bool has_right = NCB > 1 && cb + 1 < NCB;
  const f32x2 nz = negzero2();
  f32x2 w2[9];
  bool exact = false;
  {
    const T *w = static_cast<const T *>(a.w) + (long long)ch * 9;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      const float wv = Elem<T>::to_f32(w[tap_index(a, i, 9)]);
      exact = exact || !(fabsf(wv) <= 3.402823466e38f);
      w2[i] = splat2(wv);
      pin(w2[i]);
    }
  }
  const float bv = a.b ? Elem<T>::to_f32(static_cast<const T *>(a.b)[ch]) : 0.0f;
  exact = exact || __float_as_uint(bv) == 0x80000000u;
  f32x2 bias2 = splat2(bv);
  pin(bias2);
  BnPacked bnp;
  if (QM == QM_FPQ_LEAN || a.has_bn) bnp = make_bn_packed(load_bn<T>(a, ch), nz);
  const MmCoef mm = load_mm<QM>(a, ch);

  if (!async_tile) {
    if (IO8) {
      for (int i = lane; i < n_in; i += 32) codes[in_off + i] = in_src[i];
    } else {
      const T *src_t = reinterpret_cast<const T *>(in_src);
      for (int i = lane; i < n_in; i += 32) in_dst[i] = src_t[i];
    }
  }
  __syncwarp();  // barrier initialisation and thread-copied data are visible
  if (async_tile && !mbar_wait_bounded(bar, 0)) {
    if (a.flag) atomicExch(a.flag, 1);
    return;
  }
  if (IO8) {  // codes -> fp32 values, in the tile's own layout
    plane_expand_codes(codes + in_off, reinterpret_cast<float *>(in_dst), n_in, a.code_in_delta,
                       a.code_in_signed != 0, lane);
    __syncwarp();
  }

  // this thread's R x W block, overwritten in place (row pitch PW)
  T *rows = tile + pl * TE + (HALO + rb * R) * PW + cb * W;
  // The row below the block belongs to the next thread, which overwrites it early: keep a
  // copy, laid out like a tile row (left halo at [-1], right halo at [W]).
  T *my_stash = stash + lane * SW + 2;
  if (NRB > 1) {
    if (rb + 1 < NRB) {
      const T *below = rows + R * PW;
      float xv[2 * NP];
      plane_load_row<T, W>(below, true, xv);
      plane_store_row<T, W>(my_stash, xv);
      if (has_left) my_stash[-1] = below[-1];
      if (has_right) my_stash[W] = below[W];
    }
    __syncwarp();
  }

  float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
  f32x2 acc0[NP], acc1[NP];

  // One step = one input row k (plane row rb*R - 1 + k): finishes output row k-2 held in
  // `fin`, continues output row k-1 held in `mid`, starts output row k in `fin`.
  auto step = [&](int k, f32x2 *fin, f32x2 *mid) {
    const int gi = r0 + rb * R - 1 + k;
    const bool valid = gi >= 0 && gi < H;
    // the row below the block: the stash, or (last block of a band) the band's extra row
    const T *src = (NRB > 1 && k == R + 1 && rb + 1 < NRB) ? my_stash : rows + (k - 1) * PW;
    float xv[2 * NP];
    plane_load_row<T, W>(src, valid, xv);
    float xl = 0.0f, xr = 0.0f;  // the neighbours' edge columns (zero at the plane edge)
    if (NCB > 1) {
      if (valid && has_left) xl = Elem<T>::to_f32(src[-1]);
      if (valid && has_right) xr = Elem<T>::to_f32(src[W]);
    }
    // Reads of this step come before any write of this step: the row above the block is the
    // upper neighbour's last row (written in its last step), and a neighbour's edge column
    // of row k-1 is overwritten by its owner one step later.
    __syncwarp();
    // single-block planes: rows -1 and H are zero for every lane, their taps are skipped
    const bool zero_row = NRB == 1 && NBND == 1 && (k == 0 || k == R + 1);
    f32x2 E[NP], L[NP + 1];
#pragma unroll
    for (int j = 0; j < NP; ++j) E[j] = pack2(xv[2 * j], xv[2 * j + 1]);
#pragma unroll
    for (int j = 0; j <= NP; ++j)
      L[j] = pack2(j == 0 ? xl : xv[2 * j - 1], j < NP ? xv[2 * j] : xr);
    constexpr bool LAST_L_ZERO = (W % 2) != 0;  // odd W: L[NP] = (0, 0)

    auto taps = [&](f32x2 *acc, int ky, bool init) {
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        f32x2 v = init ? bias2 : acc[p];
        v = tap_add2<T>(v, w2[ky * 3 + 0], L[p], nz);
        v = tap_add2<T>(v, w2[ky * 3 + 1], E[p], nz);
        if (!(LAST_L_ZERO && p == NP - 1)) v = tap_add2<T>(v, w2[ky * 3 + 2], L[p + 1], nz);
        acc[p] = v;
      }
    };

    if (k >= 2) {
      if (!zero_row) taps(fin, 2, false);
      if (QM == QM_FPQ_LEAN || a.has_bn) bn_apply_packed<NP>(fin, bnp);
      float o[2 * NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) unpack2(fin[p], o[2 * p], o[2 * p + 1]);
      if (qm_reduces(QM)) {
#pragma unroll
        for (int j = 0; j < W; ++j) {
          lo = fminf(lo, o[j]);
          hi = fmaxf(hi, o[j]);
        }
      }
      if (qm_stores(QM)) {
        plane_quant<QM, W>(o, a.q, mm);
        if (active) plane_store_row<T, W>(rows + (k - 2) * PW, o);
      }
    }
    if (k >= 1 && k <= R) taps(mid, 1, false);
    if (k <= R - 1) {
      if (zero_row) {
#pragma unroll
        for (int p = 0; p < NP; ++p) fin[p] = bias2;
      } else {
        taps(fin, 0, true);
      }
    }
  };

#pragma unroll 1
  for (int k = 0; k < R + 2; k += 2) {
    step(k, acc0, acc1);
    if (k + 1 < R + 2) step(k + 1, acc1, acc0);
  }

  // ---- planes that need tap-skipping semantics: exact re-evaluation from global memory ----
  if (exact && active)
    plane_exact_block<T, QM>(a, plane, ch, r0 + rb * R, cb * W, R, W, rows, PW, mm, &lo, &hi);

  if (qm_reduces(QM)) plane_reduce_minmax<TPP>(a.q, ch, lo, hi, active, lane);
  if (!qm_stores(QM)) return;

  // ---- the finished tile leaves in one piece ------------------------------------------------
  unsigned char *dst = static_cast<unsigned char *>(a.y) + ((long long)plane0 * PE + (long long)r0 * PW) * ESZ;
  const T *out_src = tile + HALO * PW;
  if (IO8) {  // quantized values -> codes (the input codes are spent: their buffer is reused)
    __syncwarp();
    plane_pack_codes(reinterpret_cast<const float *>(out_src), codes, n_out, a.q.fpq_inv_delta, lane);
  }
  const void *out_bytes = IO8 ? static_cast<const void *>(codes) : static_cast<const void *>(out_src);
  if (async_tile) {
    fence_proxy_async_smem();  // this thread's shared-memory writes, for the copy engine
    __syncwarp();
    if (lane == 0) bulk_store_1d_and_wait(dst, out_bytes, obytes);
  } else {
    __syncwarp();
    if (IO8) {
      for (int i = lane; i < n_out; i += 32) dst[i] = codes[i];
    } else {
      T *dst_t = reinterpret_cast<T *>(dst);
      for (int i = lane; i < n_out; i += 32) dst_t[i] = out_src[i];
    }
  }
}

// ---- stride 1, K x K ------------------------------------------------------------------
// The same scheme for a K x K convolution (K = 3 or 5, pad K/2; instantiated for 5x5, the
// 3x3 case keeps the hand-scheduled kernel above, which is a few percent faster): thread
// block of R x W outputs; a tile is NRB
// blocks high and NCB blocks wide. With NBND == 1 the tile is a whole plane (and a CTA takes
// 32 / (NRB * NCB) planes); with NBND > 1 a plane is cut into NBND bands of full-width rows,
// one band per CTA, and the copy brings the K/2 rows above and below the band along (they
// are contiguous with it).
//
// Step k loads input row k - K/2 of the block and adds its ky = m taps to output row k - m
// for m = K-1 .. 0: output row j starts at step j (from the bias) and is finished, BN'd,
// quantized and stored at step j + K - 1. Row j lives in accumulator set j mod (K-1): the
// row finished in a step hands its registers to the row started in the same step, so K-1
// sets are live and the loop is unrolled K-1 steps per trip to keep the set indices static.
// Compiled for 16 one-warp CTAs per SM (128 registers).
// Compiled for 12 one-warp CTAs per SM: the tile, stash and weight pairs of a 56 x 56 fp32
// plane (17.5 KB) leave room for no more, and the registers this frees (140 instead of 128)
// save moves.
template <typename T, int K, int W, int NRB, int NCB, int NBND, int QM>
__global__ void __launch_bounds__(32, K == 5 ? 12 : 16)
    fused_plane_kxk_kernel(const __grid_constant__ FusedArgs a, const PlaneCfg c) {
  static_assert(K == 3 || K == 5, "3x3 or 5x5");
  static_assert(NCB == 1 || W % 2 == 0, "column blocks need an even block width");
  static_assert(K == 3 || W % 2 == 0, "5x5 needs an even block width");
  static_assert(NBND == 1 || NRB * NCB == 32, "a band is one warp's worth of blocks");
  constexpr int R = kPlaneRows;
  constexpr int PAD = K / 2;
  constexpr int KK = K * K;
  constexpr int NSET = K - 1;        // live accumulator rows
  constexpr int NSTEP = R + K - 1;   // input rows a block consumes
  constexpr int TB = R * NRB;        // rows per tile
  constexpr int H = TB * NBND;       // plane height
  constexpr int PW = W * NCB;        // plane width
  constexpr int PE = H * PW;         // elements per plane
  constexpr int HALO = NBND > 1 ? PAD : 0;  // row slots above / below the band
  constexpr int TE = (TB + 2 * HALO) * PW;  // shared-memory elements per plane of the tile
  constexpr int NP = (W + 1) / 2;    // output pairs per row
  constexpr int EH = PAD / 2;        // pairs of neighbour columns at even offsets (5x5: 1)
  constexpr int TPP = NRB * NCB;     // threads per plane
  constexpr int P = 32 / TPP;        // planes per CTA
  constexpr int SW = plane_stash_elems(W);
  constexpr bool W_SMEM = K == 5;    // 5x5: the 25 weight pairs live in shared memory
  // 5x5: one step in the loop body, accumulator rows shifted by register moves (a fourfold
  // unrolled body would not fit the instruction cache)
  constexpr bool ROTATE = K == 5;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *tile = reinterpret_cast<T *>(smem_raw);
  constexpr size_t tile_bytes = ((size_t)P * TE * sizeof(T) + 15) / 16 * 16;
  T *stash = reinterpret_cast<T *>(smem_raw + tile_bytes);
  constexpr size_t stash_bytes = NRB > 1 ? ((size_t)32 * PAD * SW * sizeof(T) + 15) / 16 * 16 : 0;
  f32x2 *wsm = reinterpret_cast<f32x2 *>(smem_raw + tile_bytes + stash_bytes);
  constexpr size_t wsm_bytes = W_SMEM ? (size_t)P * KK * sizeof(f32x2) : 0;
  // 5x5: 128 bytes of zeros that stand in for a row (or a neighbour's columns) outside the plane
  constexpr size_t zrow_bytes = K == 5 ? 128 : 0;
  T *zrow = reinterpret_cast<T *>(smem_raw + tile_bytes + stash_bytes + wsm_bytes);
  unsigned long long *bar =
      reinterpret_cast<unsigned long long *>(smem_raw + tile_bytes + stash_bytes + wsm_bytes + zrow_bytes);

  const int lane = threadIdx.x;
  if (K == 5) reinterpret_cast<float *>(zrow)[lane] = 0.0f;
  const int n_planes = (int)(a.n * a.OC);
  const int plane0 = (NBND > 1 ? blockIdx.x / NBND : blockIdx.x) * P;
  const int r0 = NBND > 1 ? (blockIdx.x % NBND) * TB : 0;  // first plane row of the tile
  const int pv = min(P, n_planes - plane0);
  T *y = static_cast<T *>(a.y);
  // what comes in (band: with the rows above / below it that exist) and what goes out
  const int in_first = NBND > 1 ? max(r0 - PAD, 0) : 0;
  const int in_rows = NBND > 1 ? min(r0 + TB + PAD, H) - in_first : pv * H;
  const T *in_src = static_cast<const T *>(a.x) + (long long)plane0 * PE + (long long)in_first * PW;
  T *in_dst = tile + (NBND > 1 ? (in_first - (r0 - PAD)) * PW : 0);
  const unsigned int bytes = (unsigned int)(in_rows * PW * sizeof(T));
  const unsigned int obytes = (unsigned int)((NBND > 1 ? TB : pv * H) * PW * sizeof(T));
  const bool async_tile = c.bulk != 0 && (bytes % 16) == 0 && (obytes % 16) == 0;

  pdl_launch_dependents();
  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  pdl_wait_for_predecessor();  // nothing global is read or written before this point
  if (lane == 0) {
    if (async_tile) {
      mbar_expect_tx(bar, bytes);
      bulk_load_1d(in_dst, in_src, bytes, bar);
    }
  }

  // ---- this thread's plane, block and per-channel operands (the copy is in flight) -------
  const int pl = lane / TPP;
  const int rb = (lane / NCB) % NRB;
  const int cb = lane % NCB;
  const bool active = pl < pv;
  const int plane = active ? plane0 + pl : n_planes - 1;
  const int ch = plane % a.OC;
  const bool has_left = NCB > 1 && cb > 0;
  const bool has_right = NCB > 1 && cb + 1 < NCB;
  const f32x2 nz = negzero2();
  f32x2 w2[W_SMEM ? 1 : KK];
  const f32x2 *wpl = wsm + pl * KK;
  bool exact = false;
  {
    const T *w = static_cast<const T *>(a.w) + (long long)ch * KK;
    if (W_SMEM) {
      // every thread checks all weights of its plane; the plane's threads share the stores
      for (int i = 0; i < KK; ++i) {
        const float wv = Elem<T>::to_f32(w[tap_index(a, i, KK)]);
        exact = exact || !(fabsf(wv) <= 3.402823466e38f);
        if (i % TPP == lane % TPP) wsm[pl * KK + i] = splat2(wv);
      }
    } else {
#pragma unroll
      for (int i = 0; i < KK; ++i) {
        const float wv = Elem<T>::to_f32(w[tap_index(a, i, KK)]);
        exact = exact || !(fabsf(wv) <= 3.402823466e38f);
        w2[i] = splat2(wv);
        pin(w2[i]);
      }
    }
  }
  const float bv = a.b ? Elem<T>::to_f32(static_cast<const T *>(a.b)[ch]) : 0.0f;
  exact = exact || __float_as_uint(bv) == 0x80000000u;
  f32x2 bias2 = splat2(bv);
  pin(bias2);
  BnPacked bnp;
  if (QM == QM_FPQ_LEAN || a.has_bn) bnp = make_bn_packed(load_bn<T>(a, ch), nz);
  const MmCoef mm = load_mm<QM>(a, ch);

  if (!async_tile) {
    const int n = in_rows * PW;
    for (int i = lane; i < n; i += 32) in_dst[i] = in_src[i];
  }
  __syncwarp();  // barrier initialisation, weight pairs and thread-copied data are visible
  if (async_tile && !mbar_wait_bounded(bar, 0)) {
    if (a.flag) atomicExch(a.flag, 1);
    return;
  }

  // this thread's R x W block, overwritten in place (row pitch PW)
  T *rows = tile + pl * TE + (HALO + rb * R) * PW + cb * W;
  // The PAD rows below the block belong to the next thread, which overwrites them early:
  // keep a copy, laid out like tile rows (left halo at [-PAD..-1], right halo at [W..]).
  T *my_stash = stash + lane * (PAD * SW) + 2;
  if (NRB > 1) {
    if (rb + 1 < NRB) {
#pragma unroll
      for (int h = 0; h < PAD; ++h) {
        const T *below = rows + (R + h) * PW;
        T *st = my_stash + h * SW;
        float xv[2 * NP];
        plane_load_row<T, W>(below, true, xv);
        plane_store_row<T, W>(st, xv);
#pragma unroll
        for (int e = 1; e <= PAD; ++e) {
          if (has_left) st[-e] = below[-e];
          if (has_right) st[W - 1 + e] = below[W - 1 + e];
        }
      }
    }
    __syncwarp();
  }

  float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);
  f32x2 acc[NSET][NP];

  // u = k mod NSET is a compile-time constant at every call site.
  auto step = [&](int k, auto uc) {
    constexpr int u = decltype(uc)::value;
    const int gi = r0 + rb * R - PAD + k;  // plane row of this step's input row
    const bool valid = gi >= 0 && gi < H;
    // rows below the block: the stash, or (last block of a band) the band's extra rows
    const T *src = (NRB > 1 && k >= R + PAD && rb + 1 < NRB) ? my_stash + (k - R - PAD) * SW
                                                              : rows + (k - PAD) * PW;
    // xs[PAD + j] = element j of the row, j = -PAD .. W + PAD - 1 (zeros outside the plane)
    float xs[2 * NP + 2 * PAD + 1];
    f32x2 Lm[NP + 1];  // 5x5: the odd-offset pairs (x[2j-1], x[2j]), loaded as such
    if (K == 5 && W % 2 == 0) {
      // Unconditional loads: a row (or a neighbour's columns) outside the plane is read from
      // the row of zeros instead, chosen by pointer, so the step has no per-load predicate
      // (the compiler turned each predicated load into a branch); the odd-offset pairs are
      // loaded straight into register pairs instead of being assembled with moves.
      const T *zc = zrow + 8;
      const T *rp = valid ? src : zc;
      const T *lp = (NCB > 1 && valid && has_left) ? src : zc;
      const T *rq = (NCB > 1 && valid && has_right) ? src : zc;
      plane_load_row<T, 2>(lp - 2, true, xs);
      plane_load_row<T, W>(rp, true, xs + PAD);
      plane_load_row<T, 2>(rq + W, true, xs + PAD + W);
#pragma unroll
      for (int j = 0; j <= NP; ++j) {
        const float a0 = Elem<T>::to_f32(j == 0 ? lp[-1] : rp[2 * j - 1]);
        const float a1 = Elem<T>::to_f32(j == NP ? rq[W] : rp[2 * j]);
        Lm[j] = pack2(a0, a1);
      }
    } else {
      plane_load_row<T, W>(src, valid, xs + PAD);
#pragma unroll
      for (int e = 1; e <= PAD; ++e) {
        xs[PAD - e] = 0.0f;
        if (W % 2 == 0) xs[PAD + W - 1 + e] = 0.0f;
        if (NCB > 1) {
          if (valid && has_left) xs[PAD - e] = Elem<T>::to_f32(src[-e]);
          if (valid && has_right) xs[PAD + W - 1 + e] = Elem<T>::to_f32(src[W - 1 + e]);
        }
      }
      if (W % 2 != 0) xs[PAD + W + 1] = 0.0f;
    }
    // Reads of this step come before any write of this step: rows above the block are the
    // upper neighbour's last rows (written in its last steps), and a neighbour's edge columns
    // of this row are overwritten by their owner K-1 steps later.
    __syncwarp();
    // single-block planes: rows outside the plane are zero for every lane, their taps are skipped
    const bool zero_row = NRB == 1 && NBND == 1 && (k < PAD || k >= R + PAD);
    // pairs of adjacent elements: E[EH + j] = (x[2j], x[2j+1]), L[j] = (x[2j-1], x[2j])
    f32x2 E[NP + 2 * EH], L[NP + 1];
#pragma unroll
    for (int j = -EH; j < NP + EH; ++j) E[EH + j] = pack2(xs[PAD + 2 * j], xs[PAD + 2 * j + 1]);
#pragma unroll
    for (int j = 0; j <= NP; ++j)
      L[j] = (K == 5 && W % 2 == 0) ? Lm[j] : pack2(xs[PAD + 2 * j - 1], xs[PAD + 2 * j]);
    constexpr bool LAST_L_ZERO = (W % 2) != 0;  // odd W (3x3 only): L[NP] = (0, 0)

    // ky = m taps of this input row onto the accumulator row that started m steps ago
    // (x[2p+d], x[2p+d+1]) for column offset d: even d -> E[p + d/2], odd d -> L[p + (d+1)/2]
    auto taps = [&](f32x2 *ar, int ky, bool init) {
      if (W_SMEM) {
#pragma unroll
        for (int kx = 0; kx < K; ++kx) {
          const f32x2 wv = wpl[ky * K + kx];
          const int d = kx - PAD;
#pragma unroll
          for (int p = 0; p < NP; ++p) {
            const f32x2 xv2 = (d % 2 == 0) ? E[EH + p + d / 2] : L[p + (d + 1) / 2];
            ar[p] = tap_add2<T>((init && kx == 0) ? bias2 : ar[p], wv, xv2, nz);
          }
        }
      } else {
#pragma unroll
        for (int p = 0; p < NP; ++p) {
          f32x2 v = init ? bias2 : ar[p];
#pragma unroll
          for (int kx = 0; kx < K; ++kx) {
            const int d = kx - PAD;
            if (LAST_L_ZERO && p == NP - 1 && d == 1) continue;
            const f32x2 xv2 = (d % 2 == 0) ? E[EH + p + d / 2] : L[p + (d + 1) / 2];
            v = tap_add2<T>(v, w2[W_SMEM ? 0 : ky * K + kx], xv2, nz);
          }
          ar[p] = v;
        }
      }
    };

    if (k >= K - 1) {  // finish output row k - (K-1)
      f32x2 *fin = acc[ROTATE ? 0 : u];
      if (!zero_row) taps(fin, K - 1, false);
      if (QM == QM_FPQ_LEAN || a.has_bn) bn_apply_packed<NP>(fin, bnp);
      float o[2 * NP];
#pragma unroll
      for (int p = 0; p < NP; ++p) unpack2(fin[p], o[2 * p], o[2 * p + 1]);
      if (qm_reduces(QM)) {
#pragma unroll
        for (int j = 0; j < W; ++j) {
          lo = fminf(lo, o[j]);
          hi = fmaxf(hi, o[j]);
        }
      }
      if (qm_stores(QM)) {
        plane_quant<QM, W>(o, a.q, mm);
        // (a lane without a plane writes into its own, never copied-out part of the tile)
        if (K == 5 || active) plane_store_row<T, W>(rows + (k - (K - 1)) * PW, o);
      }
    }
#pragma unroll
    for (int m = K - 2; m >= 1; --m) {  // rows in the middle of their accumulation
      if (k - m >= 0 && k - m < R && !zero_row)
        taps(acc[ROTATE ? K - 1 - m : (u - m + NSET * 2) % NSET], m, false);
    }
    if (ROTATE) {  // row j moves from set s+1 to set s; the new row takes the last set
#pragma unroll
      for (int sft = 0; sft + 1 < NSET; ++sft) {
#pragma unroll
        for (int p = 0; p < NP; ++p) acc[sft][p] = acc[sft + 1][p];
      }
    }
    if (k < R) {  // start output row k
      f32x2 *st = acc[ROTATE ? NSET - 1 : u];
      if (zero_row) {
#pragma unroll
        for (int p = 0; p < NP; ++p) st[p] = bias2;
      } else {
        taps(st, 0, true);
      }
    }
  };

  if (ROTATE) {
#pragma unroll 1
    for (int k = 0; k < NSTEP; ++k) step(k, IntC<0>{});
  } else {
#pragma unroll 1
    for (int k0 = 0; k0 < NSTEP; k0 += NSET) {
      static_loop<NSET>([&](auto uc) {
        constexpr int u = decltype(uc)::value;
        if (k0 + u < NSTEP) step(k0 + u, uc);
      });
    }
  }

  // ---- planes that need tap-skipping semantics: exact re-evaluation from global memory ----
  if (exact && active)
    plane_exact_block<T, QM>(a, plane, ch, r0 + rb * R, cb * W, R, W, rows, PW, mm, &lo, &hi);

  if (qm_reduces(QM)) plane_reduce_minmax<TPP>(a.q, ch, lo, hi, active, lane);
  if (!qm_stores(QM)) return;

  // ---- the finished tile leaves in one piece ------------------------------------------------
  T *dst = y + (long long)plane0 * PE + (long long)r0 * PW;
  const T *out_src = tile + HALO * PW;
  if (async_tile) {
    fence_proxy_async_smem();  // this thread's shared-memory writes, for the copy engine
    __syncwarp();
    if (lane == 0) bulk_store_1d_and_wait(dst, out_src, obytes);
  } else {
    __syncwarp();
    const int n = (NBND > 1 ? TB : pv * H) * PW;
    for (int i = lane; i < n; i += 32) dst[i] = out_src[i];
  }
}

// ---- 7x7 planes, 3x3 stride 1: two planes per thread --------------------------------------
// A 7-wide row has an odd number of elements, so pairing neighbours along the row wastes a
// lane and needs scalar loads. Here the two lanes of a pair are the SAME position of two
// different planes (thread t owns planes t and t + 32 of a 64-plane tile): the weights and
// BN operands of a pair are (channel of plane t, channel of plane t + 32), a shifted tap is
// just another column, and - with whole planes per thread - every halo tap is skipped at
// compile time (columns) or by a uniform test (rows), which is the contract's own rule: no
// zero padding enters, so there is no exact-evaluation fall-back, no stash and no barrier
// inside the loop. Input rows stream through the thread as in fused_plane_kernel.
template <typename T, int QM, bool IO8 = false>
__global__ void __launch_bounds__(32, 16)
    fused_plane_pair7_kernel(const __grid_constant__ FusedArgs a, const PlaneCfg c) {
  constexpr int W = 7, H = 7, PE = 49, P = 64;
  static_assert(!IO8 || (sizeof(T) == 4 && (QM == QM_FPQ || QM == QM_FPQ_LEAN)),
                "8-bit storage: fp32 arithmetic, FixedPointQuantize codes");

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *tile = reinterpret_cast<T *>(smem_raw);
  constexpr size_t tile_bytes = ((size_t)P * PE * sizeof(T) + 15) / 16 * 16;
  unsigned char *codes = smem_raw + tile_bytes;  // 8-bit storage: the tile's codes
  constexpr size_t codes_bytes = IO8 ? ((size_t)P * PE + 15) / 16 * 16 : 0;
  unsigned long long *bar = reinterpret_cast<unsigned long long *>(smem_raw + tile_bytes + codes_bytes);
  constexpr int ESZ = IO8 ? 1 : (int)sizeof(T);

  const int lane = threadIdx.x;
  const int n_planes = (int)(a.n * a.OC);
  const int plane0 = blockIdx.x * P;
  const int pv = min(P, n_planes - plane0);
  const unsigned char *in_src = static_cast<const unsigned char *>(a.x) + (long long)plane0 * PE * ESZ;
  unsigned char *dst = static_cast<unsigned char *>(a.y) + (long long)plane0 * PE * ESZ;
  const unsigned int bytes = (unsigned int)(pv * PE * ESZ);
  const bool async_tile = c.bulk != 0 && (bytes % 16) == 0;

  pdl_launch_dependents();
  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  pdl_wait_for_predecessor();  // nothing global is read or written before this point
  if (lane == 0) {
    if (async_tile) {
      mbar_expect_tx(bar, bytes);
      bulk_load_1d(IO8 ? static_cast<void *>(codes) : static_cast<void *>(tile), in_src, bytes, bar);
    }
  }

  // planes (lane, lane + 32) -> the (low, high) lanes of every pair
  const bool act0 = lane < pv, act1 = lane + 32 < pv;
  const int ch0 = (act0 ? plane0 + lane : n_planes - 1) % a.OC;
  const int ch1 = (act1 ? plane0 + lane + 32 : n_planes - 1) % a.OC;
  const f32x2 nz = negzero2();
  f32x2 w2[9];
  {
    const T *w0 = static_cast<const T *>(a.w) + (long long)ch0 * 9;
    const T *w1 = static_cast<const T *>(a.w) + (long long)ch1 * 9;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      w2[i] = pack2(Elem<T>::to_f32(w0[tap_index(a, i, 9)]), Elem<T>::to_f32(w1[tap_index(a, i, 9)]));
      pin(w2[i]);
    }
  }
  const T *bp = static_cast<const T *>(a.b);
  f32x2 bias2 = pack2(bp ? Elem<T>::to_f32(bp[ch0]) : 0.0f, bp ? Elem<T>::to_f32(bp[ch1]) : 0.0f);
  pin(bias2);
  BnPacked bnp;
  if (QM == QM_FPQ_LEAN || a.has_bn) bnp = make_bn_packed2(load_bn<T>(a, ch0), load_bn<T>(a, ch1), nz);
  const MmCoef mm0 = load_mm<QM>(a, ch0), mm1 = load_mm<QM>(a, ch1);

  if (!async_tile) {
    const int n = pv * PE;
    if (IO8) {
      for (int i = lane; i < n; i += 32) codes[i] = in_src[i];
    } else {
      const T *src_t = reinterpret_cast<const T *>(in_src);
      for (int i = lane; i < n; i += 32) tile[i] = src_t[i];
    }
  }
  __syncwarp();
  if (async_tile && !mbar_wait_bounded(bar, 0)) {
    if (a.flag) atomicExch(a.flag, 1);
    return;
  }
  if (IO8) {
    plane_expand_codes(codes, reinterpret_cast<float *>(tile), pv * PE, a.code_in_delta, a.code_in_signed != 0, lane);
    __syncwarp();
  }

  T *p0 = tile + lane * PE;         // lane stride 49 words: conflict-free
  T *p1 = tile + (lane + 32) * PE;
  float lo0 = __uint_as_float(0x7f800000u), hi0 = __uint_as_float(0xff800000u), lo1 = lo0, hi1 = hi0;
  f32x2 acc0[W], acc1[W];

  // step k: input row k - 1 finishes output row k - 2 (ky = 2), continues row k - 1 (ky = 1)
  // and starts row k (ky = 0); rows -1 and 7 do not exist and their taps are skipped
  auto step = [&](int k, f32x2 *fin, f32x2 *mid) {
    const bool have_row = k >= 1 && k <= H;
    f32x2 X[W];
    if (have_row) {
#pragma unroll
      for (int j = 0; j < W; ++j)
        X[j] = pack2(Elem<T>::to_f32(p0[(k - 1) * W + j]), Elem<T>::to_f32(p1[(k - 1) * W + j]));
    }
    auto taps = [&](f32x2 *acc, int ky, bool init) {
#pragma unroll
      for (int j = 0; j < W; ++j) {
        f32x2 v = init ? bias2 : acc[j];
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
          if (j + kx - 1 < 0 || j + kx - 1 >= W) continue;  // outside the plane: tap skipped
          v = tap_add2<T>(v, w2[ky * 3 + kx], X[j + kx - 1], nz);
        }
        acc[j] = v;
      }
    };
    if (k >= 2) {
      if (have_row) taps(fin, 2, false);
      if (QM == QM_FPQ_LEAN || a.has_bn) bn_apply_packed<W>(fin, bnp);
      float o[2 * W];  // o[2j] = plane 0, o[2j + 1] = plane 1, column j
#pragma unroll
      for (int j = 0; j < W; ++j) unpack2(fin[j], o[2 * j], o[2 * j + 1]);
      if (qm_reduces(QM)) {
#pragma unroll
        for (int j = 0; j < W; ++j) {
          lo0 = fminf(lo0, o[2 * j]);
          hi0 = fmaxf(hi0, o[2 * j]);
          lo1 = fminf(lo1, o[2 * j + 1]);
          hi1 = fmaxf(hi1, o[2 * j + 1]);
        }
      }
      if (qm_stores(QM)) {
        if (QM == QM_MM_APPLY) {
#pragma unroll
          for (int j = 0; j < W; ++j) {
            o[2 * j] = mm_apply(o[2 * j], mm0);
            o[2 * j + 1] = mm_apply(o[2 * j + 1], mm1);
          }
        } else {
          plane_quant<QM, 2 * W>(o, a.q, mm0);
        }
#pragma unroll
        for (int j = 0; j < W; ++j) {
          if (act0) p0[(k - 2) * W + j] = Elem<T>::from_f32(o[2 * j]);
          if (act1) p1[(k - 2) * W + j] = Elem<T>::from_f32(o[2 * j + 1]);
        }
      }
    }
    if (k >= 1 && k <= H && have_row) taps(mid, 1, false);
    if (k <= H - 1) {
      if (have_row) {
        taps(fin, 0, true);
      } else {
#pragma unroll
        for (int j = 0; j < W; ++j) fin[j] = bias2;
      }
    }
  };

#pragma unroll 1
  for (int k = 0; k < H + 2; k += 2) {
    step(k, acc0, acc1);
    if (k + 1 < H + 2) step(k + 1, acc1, acc0);
  }

  if (qm_reduces(QM)) {
    if (act0) {
      atomicMin(a.q.mm_enc_min + ch0, enc_ordered(lo0));
      atomicMax(a.q.mm_enc_max + ch0, enc_ordered(hi0));
    }
    if (act1) {
      atomicMin(a.q.mm_enc_min + ch1, enc_ordered(lo1));
      atomicMax(a.q.mm_enc_max + ch1, enc_ordered(hi1));
    }
  }
  if (!qm_stores(QM)) return;

  if (IO8) {
    __syncwarp();
    plane_pack_codes(reinterpret_cast<const float *>(tile), codes, pv * PE, a.q.fpq_inv_delta, lane);
  }
  const void *out_bytes = IO8 ? static_cast<const void *>(codes) : static_cast<const void *>(tile);
  if (async_tile) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) bulk_store_1d_and_wait(dst, out_bytes, bytes);
  } else {
    __syncwarp();
    const int n = pv * PE;
    if (IO8) {
      for (int i = lane; i < n; i += 32) dst[i] = codes[i];
    } else {
      T *dst_t = reinterpret_cast<T *>(dst);
      for (int i = lane; i < n; i += 32) dst_t[i] = tile[i];
    }
  }
}
__host__ __device__ constexpr size_t plane_pair7_smem_bytes(int elem_size, bool code8 = false) {
  return ((size_t)64 * 49 * elem_size + 15) / 16 * 16 + (code8 ? ((size_t)64 * 49 + 15) / 16 * 16 : 0) + 16;
}

// ---- stride 2 ---------------------------------------------------------------------------
// Thread block of 14 x 14 inputs = 7 x 7 outputs; a tile is NRB x NCB blocks: whole planes
// (NBND == 1) or one band of 14 * NRB full-width input rows plus the row above it
// (NBND > 1). Taps are scalar (the two outputs of a packed pair would need operands two
// elements apart, which costs more moves than it saves), BN is packed. The traffic per
// output is 2.5 times that of stride 1, so the arithmetic has issue slots to spare.
template <typename T, int NRB, int NCB, int NBND, int QM, bool IO8 = false>
__global__ void __launch_bounds__(32, 7)
    fused_plane_s2_kernel(const __grid_constant__ FusedArgs a, const PlaneCfg c) {
  static_assert(NBND == 1 || NRB * NCB == 32, "a band is one warp's worth of blocks");
  static_assert(!IO8 || (sizeof(T) == 4 && (QM == QM_FPQ || QM == QM_FPQ_LEAN)),
                "8-bit storage: fp32 arithmetic, FixedPointQuantize codes");
  constexpr int BW = 14;             // input block edge
  constexpr int OB = 7;              // output block edge
  constexpr int PW = BW * NCB;       // input plane width
  constexpr int TBI = BW * NRB;      // input rows per tile
  constexpr int H = TBI * NBND;      // input plane height
  constexpr int PE = H * PW;
  constexpr int HALO = NBND > 1 ? 1 : 0;
  constexpr int TE = (TBI + HALO) * PW;  // shared-memory elements per plane of the input tile
  constexpr int OW = OB * NCB;       // output plane width
  constexpr int TBO = OB * NRB;      // output rows per tile
  constexpr int OE = TBO * NBND * OW;
  constexpr int OTE = TBO * OW;      // elements per plane of the output tile
  constexpr int TPP = NRB * NCB;
  constexpr int P = 32 / TPP;
  constexpr int NPO = (OB + 1) / 2;  // output pairs (one dummy lane)

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *tile = reinterpret_cast<T *>(smem_raw);
  constexpr size_t tile_bytes = ((size_t)P * TE * sizeof(T) + 15) / 16 * 16;
  T *otile = reinterpret_cast<T *>(smem_raw + tile_bytes);
  constexpr size_t otile_bytes = ((size_t)P * OTE * sizeof(T) + 15) / 16 * 16;
  // 8-bit storage: the input tile's codes; the (smaller) output tile's codes reuse the buffer
  unsigned char *codes = smem_raw + tile_bytes + otile_bytes;
  constexpr size_t codes_bytes = IO8 ? ((size_t)P * TE + 15) / 16 * 16 : 0;
  unsigned long long *bar =
      reinterpret_cast<unsigned long long *>(smem_raw + tile_bytes + otile_bytes + codes_bytes);
  constexpr int ESZ = IO8 ? 1 : (int)sizeof(T);

  const int lane = threadIdx.x;
  const int n_planes = (int)(a.n * a.OC);
  const int plane0 = (NBND > 1 ? blockIdx.x / NBND : blockIdx.x) * P;
  const int band = NBND > 1 ? blockIdx.x % NBND : 0;
  const int r0 = band * TBI;  // first input row of the tile
  const int pv = min(P, n_planes - plane0);
  const int in_first = NBND > 1 ? max(r0 - 1, 0) : 0;
  const int in_rows = NBND > 1 ? r0 + TBI - in_first : pv * H;
  const unsigned char *in_src = static_cast<const unsigned char *>(a.x) +
                                ((long long)plane0 * PE + (long long)in_first * PW) * ESZ;
  const int in_off = NBND > 1 ? (in_first - (r0 - 1)) * PW : 0;
  T *in_dst = tile + in_off;
  const int n_in = in_rows * PW;
  const unsigned int bytes = (unsigned int)(n_in * ESZ);
  const int out_elems = (NBND > 1 ? 1 : pv) * OTE;
  const unsigned int obytes = (unsigned int)(out_elems * ESZ);
  const bool async_tile = c.bulk != 0 && (bytes % 16) == 0 && (obytes % 16) == 0;

  pdl_launch_dependents();
  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  pdl_wait_for_predecessor();  // nothing global is read or written before this point
  if (lane == 0) {
    if (async_tile) {
      mbar_expect_tx(bar, bytes);
      if (IO8) bulk_load_1d(codes + in_off, in_src, bytes, bar);
      else bulk_load_1d(in_dst, in_src, bytes, bar);
    }
  }

  const int pl = lane / TPP;
  const int rb = (lane / NCB) % NRB;
  const int cb = lane % NCB;
  const bool active = pl < pv;
  const int plane = active ? plane0 + pl : n_planes - 1;
  const int ch = plane % a.OC;
  const bool has_left = NCB > 1 && cb > 0;
  const f32x2 nz = negzero2();
  float wr[9];
  bool exact = false;
  {
    const T *w = static_cast<const T *>(a.w) + (long long)ch * 9;
#pragma unroll
    for (int i = 0; i < 9; ++i) {
      wr[i] = Elem<T>::to_f32(w[tap_index(a, i, 9)]);
      exact = exact || !(fabsf(wr[i]) <= 3.402823466e38f);
      pin(wr[i]);
    }
  }
  float bv = a.b ? Elem<T>::to_f32(static_cast<const T *>(a.b)[ch]) : 0.0f;
  exact = exact || __float_as_uint(bv) == 0x80000000u;
  pin(bv);
  BnPacked bnp;
  if (QM == QM_FPQ_LEAN || a.has_bn) bnp = make_bn_packed(load_bn<T>(a, ch), nz);
  const MmCoef mm = load_mm<QM>(a, ch);

  if (!async_tile) {
    if (IO8) {
      for (int i = lane; i < n_in; i += 32) codes[in_off + i] = in_src[i];
    } else {
      const T *src_t = reinterpret_cast<const T *>(in_src);
      for (int i = lane; i < n_in; i += 32) in_dst[i] = src_t[i];
    }
  }
  __syncwarp();
  if (async_tile && !mbar_wait_bounded(bar, 0)) {
    if (a.flag) atomicExch(a.flag, 1);
    return;
  }
  if (IO8) {
    plane_expand_codes(codes + in_off, reinterpret_cast<float *>(in_dst), n_in, a.code_in_delta,
                       a.code_in_signed != 0, lane);
    __syncwarp();
  }

  const T *rows = tile + pl * TE + (HALO + rb * BW) * PW + cb * BW;  // this thread's 14 x 14 inputs
  T *orows = otile + pl * OTE + rb * (OB * OW) + cb * OB;            // its 7 x 7 outputs
  float lo = __uint_as_float(0x7f800000u), hi = __uint_as_float(0xff800000u);

  // xv[0] = the column left of the block, xv[1..14] = the block's row
  auto load_row = [&](const T *p, bool valid, float *xv) {
    plane_load_row<T, BW>(p, valid, xv + 1);
    xv[0] = 0.0f;
    if (NCB > 1) {
      if (valid && has_left) xv[0] = Elem<T>::to_f32(p[-1]);
    }
  };
  auto taps = [&](float *acc, const float *xv, int ky, bool init) {
#pragma unroll
    for (int j = 0; j < OB; ++j) {
      float v = init ? bv : acc[j];
      v = tap_add<T>(v, wr[ky * 3 + 0], xv[2 * j]);
      v = tap_add<T>(v, wr[ky * 3 + 1], xv[2 * j + 1]);
      v = tap_add<T>(v, wr[ky * 3 + 2], xv[2 * j + 2]);
      acc[j] = v;
    }
  };

  float acc[OB];
  {
    // the row above the block: zero above the plane (skipped when no block has a row above)
    if (NRB == 1 && NBND == 1) {
#pragma unroll
      for (int j = 0; j < OB; ++j) acc[j] = bv;
    } else {
      float xv[BW + 2];
      load_row(rows - PW, r0 + rb * BW > 0, xv);
      taps(acc, xv, 0, true);
    }
  }
#pragma unroll 1
  for (int t = 0; t < OB; ++t) {
    float xv[BW + 2];
    load_row(rows + (2 * t) * PW, true, xv);
    taps(acc, xv, 1, false);
    load_row(rows + (2 * t + 1) * PW, true, xv);
    taps(acc, xv, 2, false);
    f32x2 pr[NPO];
#pragma unroll
    for (int p = 0; p < NPO; ++p) pr[p] = pack2(acc[2 * p], 2 * p + 1 < OB ? acc[2 * p + 1] : acc[2 * p]);
    if (QM == QM_FPQ_LEAN || a.has_bn) bn_apply_packed<NPO>(pr, bnp);
    float o[2 * NPO];
#pragma unroll
    for (int p = 0; p < NPO; ++p) unpack2(pr[p], o[2 * p], o[2 * p + 1]);
    if (qm_reduces(QM)) {
#pragma unroll
      for (int j = 0; j < OB; ++j) {
        lo = fminf(lo, o[j]);
        hi = fmaxf(hi, o[j]);
      }
    }
    if (qm_stores(QM)) {
      plane_quant<QM, OB>(o, a.q, mm);
#pragma unroll
      for (int j = 0; j < OB; ++j) orows[t * OW + j] = Elem<T>::from_f32(o[j]);
    }
    taps(acc, xv, 0, true);  // the next output row starts from this step's odd input row
  }

  if (exact && active)
    plane_exact_block<T, QM>(a, plane, ch, band * TBO + rb * OB, cb * OB, OB, OB, orows, OW, mm, &lo, &hi);

  if (qm_reduces(QM)) plane_reduce_minmax<TPP>(a.q, ch, lo, hi, active, lane);
  if (!qm_stores(QM)) return;

  unsigned char *dst = static_cast<unsigned char *>(a.y) + ((long long)plane0 * OE + (long long)band * OTE) * ESZ;
  if (IO8) {
    __syncwarp();
    plane_pack_codes(reinterpret_cast<const float *>(otile), codes, out_elems, a.q.fpq_inv_delta, lane);
  }
  const void *out_bytes = IO8 ? static_cast<const void *>(codes) : static_cast<const void *>(otile);
  if (async_tile) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) bulk_store_1d_and_wait(dst, out_bytes, obytes);
  } else {
    __syncwarp();
    if (IO8) {
      for (int i = lane; i < out_elems; i += 32) dst[i] = codes[i];
    } else {
      T *dst_t = reinterpret_cast<T *>(dst);
      for (int i = lane; i < out_elems; i += 32) dst_t[i] = otile[i];
    }
  }
}

// Host-side entry (fused_plane.cu).
cudaError_t launch_plane(int dtype, int k, int hw, int stride, int qm, const FusedArgs &a,
                         const PlaneCfg &c, cudaStream_t stream);
// Whether 8-bit storage has a plane-kernel instantiation for this shape and mode.
bool plane_has_code8(int dtype, int k, int hw, int stride, int qm);
// Geometry of the instantiation for a square hw x hw plane, kernel size and stride; tpp == 0
// if there is none.
struct PlaneGeom {
  int tpp;    // threads per plane (banded: per band)
  int bands;  // bands per plane (1 = whole planes)
  int w, nrb, ncb;
};
__host__ inline PlaneGeom plane_geom(int k, int h, int w, int stride) {
  PlaneGeom g = {0, 1, 0, 0, 0};
  if (h != w) return g;
  if (stride == 1 && (k == 3 || k == 5)) {
    if (w == 7 && k == 3) g = {1, 1, 7, 1, 1};
    else if (w == 14) g = {2, 1, 14, 2, 1};
    else if (w == 28) g = {8, 1, 14, 4, 2};
    else if (w == 56) g = {32, 1, 14, 8, 4};
    else if (w == 112) g = {32, 4, 14, 4, 8};
  } else if (stride == 2 && k == 3) {
    if (w == 14) g = {1, 1, 14, 1, 1};
    else if (w == 28) g = {4, 1, 14, 2, 2};
    else if (w == 56) g = {16, 1, 14, 4, 4};
    else if (w == 112) g = {32, 2, 14, 4, 8};
  }
  return g;
}
__host__ inline size_t plane_launch_smem(int k, int hw, int stride, int elem_size, bool code8 = false) {
  const PlaneGeom g = plane_geom(k, hw, hw, stride);
  if (stride == 1 && k == 3 && hw == 7) return plane_pair7_smem_bytes(elem_size, code8);
  if (stride == 1) return plane_smem_bytes(k, g.w, g.nrb, g.ncb, g.bands, elem_size, code8);
  return plane_s2_smem_bytes(g.nrb, g.ncb, g.bands, elem_size, code8);
}

}  // namespace dwbnq
