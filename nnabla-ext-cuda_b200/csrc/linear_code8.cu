// QuantizeLinear / DequantizeLinear with the integer result kept as 8-bit codes: the way into
// and out of the 8-bit storage of quantized activations.
//
// Arithmetic (scalar scale and zero point), the steps and order of the reference composite
// whose CUDA hooks are src/nbla/cuda/function/generic/quantize_linear.cu:22-74:
//   QuantizeLinear   t = x / scale; t = t + zero_point; t = round(t); t = saturate(t)
//                    round = half away from zero (kernel_std_round, :33-35) or half to even
//                    (kernel_round_half_to_even, :37-47: r = round(t); |t - r| == 0.5 ?
//                    round(t * 0.5) * 2 : r); saturate = clamp to [min_range, max_range] (:22-31)
//   DequantizeLinear y = (code - zero_point) * scale   (dequantize_linear.cu:22-27 + core)
// Every operation is a rounded fp32 operation (binary16 tensors are up-cast first and the
// result rounded once). A NaN has no code and is stored as 0.
#include "dwbnq_internal.h"

namespace dwbnq {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ int quantize_one(float x, float scale, float zp, int half_even, float lo, float hi) {
  float t = __fadd_rn(__fdiv_rn(x, scale), zp);
  const float r = roundf(t);
  if (half_even && fabsf(__fsub_rn(t, r)) == 0.5f) t = __fmul_rn(roundf(__fmul_rn(t, 0.5f)), 2.0f);
  else t = r;
  if (t < lo) t = lo;
  else if (t > hi) t = hi;
  return __float2int_rn(t);  // t is an integer (or NaN -> 0)
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
    quantize_linear_code8_kernel(const T *__restrict__ x, unsigned char *__restrict__ codes, long long size,
                                 int vec_ok, float scale, float zp, int half_even, float lo, float hi) {
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  constexpr int S = Elem<T>::VEC;  // elements per 16-byte load
  const long long n_vec = vec_ok ? size / S : 0;
  for (long long v = tid; v < n_vec; v += step) {
    float e[S];
    Vec16<T>::load_stream(x + v * S, e);
    unsigned int w[S / 4];
#pragma unroll
    for (int g = 0; g < S / 4; ++g) {
      unsigned int u = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        u |= ((unsigned int)quantize_one(e[4 * g + j], scale, zp, half_even, lo, hi) & 0xffu) << (8 * j);
      w[g] = u;
    }
    if (S == 4) reinterpret_cast<unsigned int *>(codes)[v] = w[0];
    else reinterpret_cast<uint2 *>(codes)[v] = make_uint2(w[0], w[S / 4 - 1]);
  }
  for (long long i = n_vec * S + tid; i < size; i += step)
    codes[i] = (unsigned char)((unsigned int)quantize_one(Elem<T>::to_f32(x[i]), scale, zp, half_even, lo, hi) & 0xffu);
}

template <typename T, bool SIGNED>
__global__ void __launch_bounds__(kThreads)
    dequantize_linear_code8_kernel(const unsigned char *__restrict__ codes, T *__restrict__ y, long long size,
                                   int vec_ok, float scale, float zp) {
  pdl_launch_dependents();
  pdl_wait_for_predecessor();
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  constexpr int S = Elem<T>::VEC;
  const long long n_vec = vec_ok ? size / S : 0;
  auto one = [&](unsigned int c) {
    const float k = SIGNED ? (float)(signed char)c : (float)c;
    return __fmul_rn(__fsub_rn(k, zp), scale);
  };
  for (long long v = tid; v < n_vec; v += step) {
    unsigned int w[2];
    if (S == 4) {
      w[0] = reinterpret_cast<const unsigned int *>(codes)[v];
      w[1] = 0;
    } else {
      const uint2 t = reinterpret_cast<const uint2 *>(codes)[v];
      w[0] = t.x;
      w[1] = t.y;
    }
    float e[S];
#pragma unroll
    for (int j = 0; j < S; ++j) e[j] = one((w[j / 4] >> (8 * (j % 4))) & 0xffu);
    Vec16<T>::store_stream(y + v * S, e);
  }
  for (long long i = n_vec * S + tid; i < size; i += step) y[i] = Elem<T>::from_f32(one(codes[i]));
}

unsigned int grid_for(long long items) {
  long long blocks = (items + kThreads - 1) / kThreads;
  const long long cap = (long long)sm_count(-1) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned int)blocks;
}

inline bool aligned_to(const void *p, int n) { return (reinterpret_cast<uintptr_t>(p) % n) == 0; }

}  // namespace

int launch_quantize_linear_code8(int dtype, long long size, float scale, int zero_point, int round_mode,
                                 int min_range, int max_range, const void *x, void *codes, cudaStream_t stream) {
  const int S = dtype == DWBNQ_F32 ? 4 : 8;
  const int vec_ok = aligned_to(x, 16) && aligned_to(codes, S);
  const int he = round_mode == DWBNQ_ROUND_HALF_TO_EVEN;
  cudaError_t e;
  if (dtype == DWBNQ_F32)
    e = launch_pdl(quantize_linear_code8_kernel<float>, dim3(grid_for((size + S - 1) / S)), dim3(kThreads), 0, stream,
                   static_cast<const float *>(x), static_cast<unsigned char *>(codes), size, vec_ok, scale,
                   (float)zero_point, he, (float)min_range, (float)max_range);
  else
    e = launch_pdl(quantize_linear_code8_kernel<__half>, dim3(grid_for((size + S - 1) / S)), dim3(kThreads), 0, stream,
                   static_cast<const __half *>(x), static_cast<unsigned char *>(codes), size, vec_ok, scale,
                   (float)zero_point, he, (float)min_range, (float)max_range);
  if (e != cudaSuccess) return fail_cuda(e, "quantize_linear_code8_kernel launch");
  return DWBNQ_OK;
}

int launch_dequantize_linear_code8(int dtype, long long size, float scale, int zero_point, int codes_signed,
                                   const void *codes, void *y, cudaStream_t stream) {
  const int S = dtype == DWBNQ_F32 ? 4 : 8;
  const int vec_ok = aligned_to(y, 16) && aligned_to(codes, S);
  const unsigned int grid = grid_for((size + S - 1) / S);
  const unsigned char *c = static_cast<const unsigned char *>(codes);
  cudaError_t e;
  if (dtype == DWBNQ_F32) {
    e = codes_signed ? launch_pdl(dequantize_linear_code8_kernel<float, true>, dim3(grid), dim3(kThreads), 0, stream, c,
                                  static_cast<float *>(y), size, vec_ok, scale, (float)zero_point)
                     : launch_pdl(dequantize_linear_code8_kernel<float, false>, dim3(grid), dim3(kThreads), 0, stream, c,
                                  static_cast<float *>(y), size, vec_ok, scale, (float)zero_point);
  } else {
    e = codes_signed ? launch_pdl(dequantize_linear_code8_kernel<__half, true>, dim3(grid), dim3(kThreads), 0, stream, c,
                                  static_cast<__half *>(y), size, vec_ok, scale, (float)zero_point)
                     : launch_pdl(dequantize_linear_code8_kernel<__half, false>, dim3(grid), dim3(kThreads), 0, stream, c,
                                  static_cast<__half *>(y), size, vec_ok, scale, (float)zero_point);
  }
  if (e != cudaSuccess) return fail_cuda(e, "dequantize_linear_code8_kernel launch");
  return DWBNQ_OK;
}

}  // namespace dwbnq
