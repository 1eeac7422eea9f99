/*
 * dwbnq - C ABI of the B200 (sm_100a) quantized depthwise-CNN inference path:
 * DepthwiseConvolution forward -> BatchNormalization (batch_stat=false) ->
 * FixedPointQuantize | Pow2Quantize | MinMaxQuantize forward, plus the pointwise
 * convolutions around it.
 *
 * Conventions (they mirror how nnabla-ext-cuda's function classes touch memory):
 *  - every data pointer is a DEVICE pointer owned by the caller and valid for the
 *    duration of the call (the reference obtains them with
 *    Variable::get_data_pointer<Tc>(ctx) / cast_data_and_get_pointer<Tc>(ctx, true),
 *    src/nbla/cuda/function/generic/depthwise_convolution.cu:445-449);
 *  - nothing is allocated or freed on the caller's behalf; ops that need scratch take a
 *    caller-provided workspace whose size dwbnq_workspace_bytes() reports;
 *  - `device` is the CUDA device ordinal the pointers live on (-1 = the calling
 *    thread's current device); the call makes it current like the reference's
 *    cuda_set_device(device_) (src/nbla/cuda/common.cpp:20-26);
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream the
 *    reference launches on, include/nbla/cuda/common.hpp:377-382); calls are
 *    asynchronous with respect to the host unless stated otherwise;
 *  - every function returns a dwbnq_status; on failure dwbnq_last_error_string() gives
 *    the message for the calling thread. No C++ exception crosses this boundary (the
 *    reference raises nbla::Exception through NBLA_CHECK / NBLA_CUDA_CHECK,
 *    include/nbla/cuda/common.hpp:70-85; the plugin shim converts a status to one);
 *  - there is no CPU fallback: without a usable CUDA device compute calls fail with
 *    DWBNQ_ERR_CUDA.
 *  - dtype DWBNQ_F16: tensors and parameters are IEEE binary16 in memory, arithmetic is
 *    fp32 and the result is rounded to binary16 once at the store.
 */
#ifndef DWBNQ_H_
#define DWBNQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with hidden visibility */
#endif

#define DWBNQ_ABI_VERSION 1

typedef enum dwbnq_status {
  DWBNQ_OK = 0,
  DWBNQ_ERR_INVALID_ARG = 1, /* null pointer, non-positive size, bad enum ...        */
  DWBNQ_ERR_UNSUPPORTED = 2, /* a configuration the reference rejects too             */
  DWBNQ_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed (message has why)   */
  DWBNQ_ERR_NCCL = 4,        /* NCCL missing or a collective failed                   */
  DWBNQ_ERR_TIMEOUT = 5,     /* a bounded wait ran out (collective or device barrier) */
  DWBNQ_ERR_DEVICE_FLAG = 6  /* a kernel recorded an internal error (bounded wait)    */
} dwbnq_status;

typedef enum dwbnq_dtype { DWBNQ_F32 = 0, DWBNQ_F16 = 1 } dwbnq_dtype;

typedef enum dwbnq_quant_kind {
  DWBNQ_Q_NONE = 0,  /* conv (+BN) only                                   */
  DWBNQ_Q_FPQ = 1,   /* FixedPointQuantize                                */
  DWBNQ_Q_POW2 = 2,  /* Pow2Quantize                                      */
  DWBNQ_Q_MINMAX = 3 /* MinMaxQuantize with per-channel ranges [1,C,1,1]  */
} dwbnq_quant_kind;

/* Geometry of a DepthwiseConvolution, i.e. the constructor arguments of
 * DepthwiseConvolutionCuda(ctx, base_axis, pad, stride, dilation, multiplier)
 * (include/nbla/cuda/function/depthwise_convolution.hpp:27-32) plus the input shape the
 * base class derives in setup_impl. Layout is NCHW; a 1-D convolution is h = kh = 1. */
typedef struct dwbnq_conv_desc {
  int32_t dtype;      /* dwbnq_dtype                                          */
  int32_t c;          /* input channels                                       */
  int64_t n;          /* product of the axes before base_axis (the batch)     */
  int32_t h, w;       /* input spatial size                                   */
  int32_t kh, kw;     /* kernel                                               */
  int32_t stride_h, stride_w;
  int32_t pad_h, pad_w;
  int32_t dil_h, dil_w;
  int32_t multiplier; /* output channels = c * multiplier                     */
} dwbnq_conv_desc;

/* Quantizer constructor arguments.
 *  FPQ   : FixedPointQuantizeCuda(ctx, sign, n, delta, ste_fine_grained)
 *          (include/nbla/cuda/function/fixed_point_quantize.hpp:35-38)
 *  POW2  : Pow2QuantizeCuda(ctx, sign, with_zero, n, m, ste_fine_grained)
 *          (include/nbla/cuda/function/pow2_quantize.hpp:34-37)
 *  MINMAX: MinMaxQuantizeCuda(ctx, decay, x_min_max, ema, ste_fine_grained, eps)
 *          (include/nbla/cuda/function/min_max_quantize.hpp:27-30)
 * ste_fine_grained only affects backward and is not carried. */
typedef struct dwbnq_quant_desc {
  int32_t kind; /* dwbnq_quant_kind */
  int32_t sign;
  int32_t n;
  float delta;       /* FPQ                      */
  int32_t with_zero; /* POW2                     */
  int32_t m;         /* POW2                     */
  float decay;       /* MINMAX (used when ema)   */
  float eps;         /* MINMAX range nudge       */
  int32_t x_min_max; /* MINMAX                   */
  int32_t ema;       /* MINMAX                   */
} dwbnq_quant_desc;

/* Per-channel MinMaxQuantize tensors (inputs 1..4 of the function; qr_min / qr_max are
 * updated in place when x_min_max is set, like the reference writes them back,
 * src/nbla/cuda/function/generic/min_max_quantize.cu:63-69). All hold `channels`
 * elements of the call's dtype. */
typedef struct dwbnq_minmax_ptrs {
  void *qr_min;
  void *qr_max;
  const void *ql_min;
  const void *ql_max;
} dwbnq_minmax_ptrs;

/* ---- library ------------------------------------------------------------------ */

int dwbnq_version(void);
const char *dwbnq_last_error_string(void);
/* Number of CUDA devices visible (0 when there is no driver/GPU). Never fails. */
int dwbnq_device_count(void);
/* Reads and clears the per-device flag kernels set when one of their bounded waits ran
 * out. Synchronises the device. DWBNQ_OK when clear, DWBNQ_ERR_DEVICE_FLAG when set. */
int dwbnq_check_device_flag(int device);

/* ---- shape / parameter helpers (host only, no CUDA) ----------------------------- */

/* Output spatial size the base class computes in setup_impl:
 * o = (i + 2p - d(k-1) - 1) / s + 1. Fails with DWBNQ_ERR_INVALID_ARG on a bad desc
 * and DWBNQ_ERR_UNSUPPORTED when c*multiplier*kh*kw > 65536, the limit the reference
 * enforces (depthwise_convolution.cu:381), or when a padded input plane or an output plane
 * holds more than 2^31-1 elements (planes are indexed with 32-bit integers). ho and wo may
 * each be NULL (not written). */
int dwbnq_conv_out_shape(const dwbnq_conv_desc *desc, int32_t *ho, int32_t *wo);
/* max_ / min_ members of FixedPointQuantize for (sign, n, delta). */
int dwbnq_fpq_range(int sign, int n, float delta, float *max_out, float *min_out);
/* p_max_ / p_min_ / pruning_threshold_ members of Pow2Quantize. */
int dwbnq_pow2q_range(int sign, int with_zero, int n, int m, float *p_max, float *p_min,
                      float *pruning_threshold);
/* Pow2Quantize needs round(log2f(|x|)) exactly as the host libm rounds it. The library
 * keeps, per binade e in [-149, 127], the smallest float bit pattern whose rounded
 * log2 is e+1 (found with the host libm by bisection) and decides with integer
 * compares on the device. This copies the 277-entry table (index e+149). */
int dwbnq_pow2q_threshold_table(uint32_t *table277);
/* Bytes of device scratch the MINMAX entry points need for `channels` channels. */
size_t dwbnq_workspace_bytes(int32_t channels);

/* ---- the five registered function classes, one entry point each ------------------ */

/* DepthwiseConvolutionCuda<T>::forward_impl
 * (src/nbla/cuda/function/generic/depthwise_convolution.cu:435-489).
 * x [n,c,h,w]; w [c*mult,kh,kw]; b [c*mult] or NULL; y [n,c*mult,ho,wo]. */
int dwbnq_dwconv_fwd(const dwbnq_conv_desc *desc, const void *x, const void *w,
                     const void *b, void *y, int device, void *stream);

/* BatchNormalizationCuda<T>::forward_impl_global, i.e. batch_stat=false
 * (src/nbla/cuda/function/generic/batch_normalization.cu:174-199). x is viewed as
 * [size0, size1, size2] with the channel axis = size1; beta / gamma may be NULL
 * (no_bias / no_scale); mean, var (and beta, gamma) hold size1 elements. */
int dwbnq_bn_infer_fwd(int dtype, int64_t size0, int64_t size1, int64_t size2, float eps,
                       const void *x, const void *beta, const void *gamma, const void *mean,
                       const void *var, void *y, int device, void *stream);

/* FixedPointQuantizeCuda<T>::forward_impl
 * (src/nbla/cuda/function/generic/fixed_point_quantize.cu:51-61). y may alias x. */
int dwbnq_fpq_fwd(int dtype, int64_t size, int sign, int n, float delta, const void *x,
                  void *y, int device, void *stream);

/* Pow2QuantizeCuda<T>::forward_impl
 * (src/nbla/cuda/function/generic/pow2_quantize.cu:65-77). y may alias x. */
int dwbnq_pow2q_fwd(int dtype, int64_t size, int sign, int with_zero, int n, int m,
                    const void *x, void *y, int device, void *stream);

/* MinMaxQuantize forward (core composite + the MinMaxQuantizeCuda hooks,
 * src/nbla/cuda/function/generic/min_max_quantize.cu:29-90) for x viewed as
 * [size0, channels, size2] and ranges of shape [1, channels, 1, 1].
 * `workspace`: dwbnq_workspace_bytes(channels) bytes of device memory, 256-byte
 * aligned, contents irrelevant on entry. `comm`: NULL, or a dwbnq communicator over
 * which the per-channel min/max are all-reduced (for a batch sharded across GPUs) when
 * q->x_min_max is set. y may alias x. */
int dwbnq_minmaxq_fwd(int dtype, int64_t size0, int32_t channels, int64_t size2,
                      const dwbnq_quant_desc *q, const void *x, const dwbnq_minmax_ptrs *mm,
                      void *y, void *workspace, void *comm, int device, void *stream);

/* MinMaxQuantize forward without a workspace argument. It has no counterpart in the
 * reference. It exists for callers that cannot supply scratch memory at the point of the
 * call - a function object of a framework whose own allocator already holds the whole
 * device, a serving loop that is not allowed to reach the allocator while it runs, a
 * plugin hook that receives nothing but tensor pointers. The scratch lives in a fixed
 * device array inside the library instead (7 words per channel, DWBNQ_STATIC_MAX_CHANNELS
 * channels, 112 KiB on every GPU that loads the library, held until the process exits).
 *  - channels > DWBNQ_STATIC_MAX_CHANNELS fails with DWBNQ_ERR_UNSUPPORTED;
 *  - no cudaMalloc / cudaFree or other allocating call is made, here or in the kernels;
 *  - the first call on each device looks up the array's device address; make that first
 *    call before starting any stream capture on the device;
 *  - all calls on a device share the one array: calls that may overlap on the GPU (different
 *    streams, different host threads) race on it - serialise them or use
 *    dwbnq_minmaxq_fwd with separate workspaces; there is no `comm` either: a batch
 *    sharded over several GPUs needs dwbnq_minmaxq_fwd.
 * Results are identical to dwbnq_minmaxq_fwd with comm == NULL. */
#define DWBNQ_STATIC_MAX_CHANNELS 4096
int dwbnq_minmaxq_fwd_static(int dtype, int64_t size0, int32_t channels, int64_t size2,
                             const dwbnq_quant_desc *q, const void *x, const dwbnq_minmax_ptrs *mm,
                             void *y, int device, void *stream);

/* ---- the fused layer: what the graph pass rewrites dw-conv -> BN -> quantizer into -- */

/* y = Quantize(BN_inference(DepthwiseConvolution(x))). No counterpart kernel exists in
 * the reference (it runs the three classes above back to back); the arithmetic is the
 * exact composition of the three, so the result is bit-identical to the unfused chain.
 * bn_mean == NULL skips BatchNormalization (then bn_var / beta / gamma are ignored);
 * q == NULL or kind NONE skips the quantizer. For MINMAX `mm` and `workspace` are
 * required and `comm` is as in dwbnq_minmaxq_fwd; the activation is reduced in a first
 * pass over x and quantized in a second one (nothing but `workspace` is written
 * besides y and qr_min / qr_max). */
int dwbnq_fused_fwd(const dwbnq_conv_desc *desc, float bn_eps, const dwbnq_quant_desc *q,
                    const void *x, const void *w, const void *b, const void *bn_beta,
                    const void *bn_gamma, const void *bn_mean, const void *bn_var,
                    const dwbnq_minmax_ptrs *mm, void *y, void *workspace, void *comm,
                    int device, void *stream);

/* ---- training side: backward of the quantizers and of the convolution ------------------- */

/* FixedPointQuantizeCuda<T>::backward_impl, the straight-through estimator
 * (src/nbla/cuda/function/generic/fixed_point_quantize.cu:63-128): dx = dy, or with
 * ste_fine_grained dx = dy where min <= x <= max and 0 elsewhere; `accum` adds to dx instead
 * (clipped elements are then left untouched). x may be NULL without ste_fine_grained. */
int dwbnq_fpq_bwd(int dtype, int64_t size, int sign, int n, float delta, int ste_fine_grained,
                  int accum, const void *x, const void *dy, void *dx, int device, void *stream);
/* Pow2QuantizeCuda<T>::backward_impl (src/nbla/cuda/function/generic/pow2_quantize.cu:79-160):
 * dx (+)= c * dy with c = 0 where 2^round(log2f|x|) > p_max, and where x < 0 for the unsigned
 * quantizer, else 1; plain pass-through without ste_fine_grained. */
int dwbnq_pow2q_bwd(int dtype, int64_t size, int sign, int with_zero, int n, int m,
                    int ste_fine_grained, int accum, const void *x, const void *dy, void *dx,
                    int device, void *stream);
/* DepthwiseConvolutionCuda<T>::backward_impl
 * (src/nbla/cuda/function/generic/depthwise_convolution.cu:492-650; kernels :114-366).
 * Any of dx [n,c,h,w], dw [c*mult,kh,kw], db [c*mult] may be NULL (propagate_down false).
 * accum_mask bit 0 / 1 / 2: accumulate onto dx / dw / db instead of overwriting (the
 * reference zeroes a gradient that is not accumulated, then adds). The input gradient sums in
 * the reference's order and is bit-identical to the CPU loop; the weight and bias gradients
 * are block reductions finished with atomic adds (order of the fp32 sum not fixed: compare
 * within a tolerance). DWBNQ_F32 only. */
int dwbnq_dwconv_bwd(const dwbnq_conv_desc *desc, const void *x, const void *w, const void *dy,
                     void *dx, void *dw, void *db, int accum_mask, int device, void *stream);

/* ---- 8-bit storage of quantized activations -------------------------------------------- */

/* The outputs of a FixedPointQuantize layer with n <= 8 take 2^n values k * delta: as T
 * values they spend 4 (or 2) bytes on 8 bits of information, on HBM and on every bus the
 * tensor crosses. These entry points keep the activation as its integer code k, one byte per
 * element. The boundary is the reference's QuantizeLinear / DequantizeLinear pair
 * (src/nbla/cuda/function/generic/quantize_linear.cu:22-74: saturate, round half away from
 * zero or half to even; dequantize_linear.cu:22-27): a code tensor is what
 * QuantizeLinear(x, scale = delta, zero_point = 0) yields, stored as int8 / uint8 instead of
 * a float tensor of integers, and FixedPointQuantize(x) == DequantizeLinear(codes). */

typedef enum dwbnq_round_mode {
  DWBNQ_ROUND_HALF_AWAY_FROM_ZERO = 0, /* round(), quantize_linear.cu:33-35            */
  DWBNQ_ROUND_HALF_TO_EVEN = 1         /* quantize_linear.cu:37-47                     */
} dwbnq_round_mode;

/* QuantizeLinear forward with scalar scale and zero point, result stored as 8-bit codes:
 * code = saturate(round(x / scale + zero_point), min_range, max_range), the steps and their
 * order being the reference composite's (division, addition, rounding, saturation). Codes
 * are written as int8 when min_range < 0, else uint8; the range must fit that type.
 * x: `size` elements of `dtype`. */
int dwbnq_quantize_linear_code8_fwd(int dtype, int64_t size, float scale, int zero_point,
                                    int round_mode, int min_range, int max_range, const void *x,
                                    void *codes, int device, void *stream);
/* DequantizeLinear forward from 8-bit codes: y = (code - zero_point) * scale, y of `dtype`. */
int dwbnq_dequantize_linear_code8_fwd(int dtype, int64_t size, float scale, int zero_point,
                                      int codes_signed, const void *codes, void *y, int device,
                                      void *stream);

/* How the fused layer's input codes are to be read: x = code * in_delta (the previous
 * layer's FixedPointQuantize step), codes int8 when in_signed, else uint8. */
typedef struct dwbnq_code8_desc {
  int32_t in_signed;
  float in_delta;
} dwbnq_code8_desc;

/* dwbnq_fused_fwd with x and y as 8-bit codes: y_code = FixedPointQuantize(BN(conv(x_code *
 * in_delta))) / delta. The arithmetic is that of dwbnq_fused_fwd on the dequantized input -
 * same operations, same order, same roundings - so y_code * delta equals its fp32 output
 * value for value (a -0.0 of the signed quantizer is stored as code 0). `q` must be a
 * FixedPointQuantize with n <= 8 and delta a power of two (the code is then exact); codes are
 * int8 when q->sign, else uint8. desc->dtype names the type of w, b and the BN vectors
 * (DWBNQ_F32). Every geometry is accepted; 3x3 convolutions on 7, 14, 28, 56 and 112 wide
 * square planes run on the plane kernels with the code tiles expanded in shared memory, the
 * rest on the generic kernel. A NaN activation has no code and is stored as 0. */
int dwbnq_fused_fwd_code8(const dwbnq_conv_desc *desc, float bn_eps, const dwbnq_quant_desc *q,
                          const dwbnq_code8_desc *io, const void *x_codes, const void *w,
                          const void *b, const void *bn_beta, const void *bn_gamma,
                          const void *bn_mean, const void *bn_var, void *y_codes, int device,
                          void *stream);

/* Which kernel family the fused / dw-conv entry points would use for `desc` given the
 * pointer alignment: 0 = generic direct kernel, 1 = zero-padded shared-memory tile filled
 * by cooperative loads, 2 = zero-padded tile filled by TMA tiled loads, 3 = whole planes
 * copied by the bulk copy engine (planes whose row pitch is not a multiple of 16 bytes),
 * 4 = small planes (7x7, 14x14; 3x3 stride 1): one warp per tile of whole planes, bulk copy
 * in, full-width rows per thread, bulk store out, 5 = the same scheme with the geometry as
 * a run-time argument (3x3 stride 1 on any other plane of even width).
 * *ctas is the number of tiles = CTAs of the launch. Diagnostic only. (The switches that
 * restrict this choice for tests and tuning runs are declared in dwbnq_debug.h.) */
int dwbnq_fused_plan(const dwbnq_conv_desc *desc, const void *x, const void *y,
                     int *path_out, int *planes_per_cta, int *rows_per_tile,
                     int *threads, int64_t *ctas, int *smem_bytes);
/* ---- the pointwise (1x1) convolutions either side of a depthwise layer ------------------ */

/* How an fp32 contraction is evaluated on the tensor cores.
 *  DWBNQ_PW_MATH_FP32: every product is formed from the TF32 halves of both factors in
 *    three tensor-core passes (hi*hi + lo*hi + hi*lo, fp32 accumulation), which keeps the
 *    result within a few units of 1e-6 of sum|w||x| - the accuracy class of the fp32
 *    GEMM the reference runs by default (it disables TF32 unless NNABLA_CUDA_ALLOW_TF32
 *    is set, src/nbla/cuda/init.cpp.tmpl:76-83);
 *  DWBNQ_PW_MATH_TF32: one pass on operands truncated to TF32, what the reference
 *    computes when NNABLA_CUDA_ALLOW_TF32=1. */
typedef enum dwbnq_pw_math { DWBNQ_PW_MATH_FP32 = 0, DWBNQ_PW_MATH_TF32 = 1 } dwbnq_pw_math;
/* Activation between BatchNormalization and the quantizer: ReLU is max(0, x)
 * (src/nbla/cuda/function/generic/relu.cu:31-41), ReLU6 is min(max(x, 0), 6)
 * (src/nbla/cuda/function/generic/relu6.cu:25-26). */
typedef enum dwbnq_act { DWBNQ_ACT_NONE = 0, DWBNQ_ACT_RELU = 1, DWBNQ_ACT_RELU6 = 2 } dwbnq_act;

/* Geometry of Convolution(ctx, base_axis, pad, stride, dilation, group, channel_last)
 * (include/nbla/cuda/function/convolution.hpp:27-33) restricted to the pointwise case the
 * MobileNet blocks use around each depthwise layer: kernel 1x1, pad 0, stride 1,
 * dilation 1, group 1, NCHW. Anything else stays with the reference's own kernels. */
typedef struct dwbnq_pwconv_desc {
  int32_t dtype;      /* dwbnq_dtype                                   */
  int32_t c_in;       /* input channels                                */
  int32_t c_out;      /* output channels                               */
  int32_t h, w;       /* spatial size (input = output)                 */
  int64_t n;          /* product of the axes before base_axis          */
  int32_t math;       /* dwbnq_pw_math (ignored for fp16 tensors)      */
  int32_t act;        /* dwbnq_act, applied after BN, before quantizer */
} dwbnq_pwconv_desc;

/* Bytes of device scratch the pointwise entry points need (per-channel coefficients and
 * the TF32 halves of the weights); 256-byte aligned, contents irrelevant on entry. */
size_t dwbnq_pwconv_workspace_bytes(const dwbnq_pwconv_desc *desc);

/* ConvolutionCuda<T>::forward_impl for the pointwise case: the reference runs one GEMM per
 * image on the im2col buffer and then adds the bias with a rank-1 GEMM
 * (src/nbla/cuda/function/generic/convolution.cu:56-87; the cuDNN class does the same with
 * cudnnConvolutionForward + cudnnAddTensor, src/nbla/cuda/cudnn/function/generic/
 * convolution.cu:135), so y = (sum over input channels of w * x) + b with the order of the
 * sum unspecified. x [n,c_in,h,w]; w [c_out,c_in,1,1]; b [c_out] or NULL; y [n,c_out,h,w]. */
int dwbnq_pwconv_fwd(const dwbnq_pwconv_desc *desc, const void *x, const void *w, const void *b,
                     void *y, void *workspace, int device, void *stream);

/* y = Quantize(act(BN_inference(Convolution_1x1(x)))) in one kernel: BatchNormalization,
 * the activation and FixedPointQuantize / Pow2Quantize run on the accumulators before the
 * only store. Given the convolution result, BN, activation and quantizer are the exact
 * arithmetic of the separate classes (as in dwbnq_fused_fwd); the convolution itself is
 * exact only up to the order of its sum, so a value that lands within rounding distance of
 * a quantization threshold may come out one step away from another implementation's.
 * bn_mean == NULL skips BatchNormalization; q == NULL or kind NONE skips the quantizer;
 * MINMAX is not available here (run dwbnq_minmaxq_fwd on the result). */
int dwbnq_pwconv_fused_fwd(const dwbnq_pwconv_desc *desc, float bn_eps, const dwbnq_quant_desc *q,
                           const void *x, const void *w, const void *b, const void *bn_beta,
                           const void *bn_gamma, const void *bn_mean, const void *bn_var,
                           void *y, void *workspace, int device, void *stream);

/* The two halves of dwbnq_pwconv_fused_fwd for a caller whose parameters do not change between
 * calls (inference): dwbnq_pwconv_prepare writes the workspace - the per-channel coefficients
 * (bias, mean, gamma, sqrt(var + eps), beta) and the fp32 weights or their TF32 halves - once,
 * the way the reference's function objects do their one-time work in setup_impl;
 * dwbnq_pwconv_fused_fwd_prepared then runs the layer on that workspace with one kernel launch
 * and reads neither w nor the vectors. `desc` must be the same in both calls except for n, h
 * and w: the workspace depends on dtype, c_in, c_out, math and act only, so one prepared
 * workspace serves every batch size and plane size. has_bn states
 * whether dwbnq_pwconv_prepare was given bn_mean / bn_var. Results are identical to
 * dwbnq_pwconv_fused_fwd, which is these two calls in sequence. */
int dwbnq_pwconv_prepare(const dwbnq_pwconv_desc *desc, float bn_eps, const void *w, const void *b,
                         const void *bn_beta, const void *bn_gamma, const void *bn_mean,
                         const void *bn_var, void *workspace, int device, void *stream);
int dwbnq_pwconv_fused_fwd_prepared(const dwbnq_pwconv_desc *desc, const dwbnq_quant_desc *q, int has_bn,
                                    const void *x, void *y, void *workspace, int device, void *stream);

/* Which kernel the pointwise entry points would use: 1 = the tcgen05 kernel (c_in a multiple of
 * 4; planes whose size is not a multiple of 4, an x that is not 16-byte aligned and fp16 tensors
 * are gathered with plain loads instead of TMA; fp16 tensors always run ONE TF32 pass, which is
 * exact for binary16 factors, whatever `math` says), 0 = the plain FMA kernel (other c_in).
 * Diagnostic only. */
int dwbnq_pwconv_plan(const dwbnq_pwconv_desc *desc, const void *x, const void *w, int *path_out);

/* ---- communicator: the one exchange the path needs (per-channel min/max) ----------- */

/* NCCL is loaded with dlopen at first use, like the reference does
 * (src/nbla/cuda/communicator/dl_nccl.cpp.tmpl). The reference's communicator offers
 * only sum/avg (multi_process_data_parallel_communicator.cu:790); this one issues a
 * single ncclAllReduce(ncclMax) on the packed vector [max_c..., -min_c...]. */
#define DWBNQ_UNIQUE_ID_BYTES 128
int dwbnq_comm_get_unique_id(void *id128);
int dwbnq_comm_create(const void *id128, int nranks, int rank, int device, void **comm);
int dwbnq_comm_destroy(void *comm);
/* Deadline of the all-reduce the MINMAX entry points issue themselves (dwbnq_minmaxq_fwd,
 * dwbnq_fused_fwd with a `comm`). 0 (the default; the environment variable
 * DWBNQ_COMM_DEADLINE_MS sets another default at dwbnq_comm_create) only enqueues the
 * collective. A positive value makes those calls wait on the host until the collective has
 * completed: after `ms` milliseconds, or on an asynchronous NCCL error, the communicator
 * is aborted and the call returns DWBNQ_ERR_TIMEOUT / DWBNQ_ERR_NCCL - the role of the
 * reference's watch dog (src/nbla/cuda/communicator/watch_dog.cpp:59-108, armed around
 * each collective at multi_process_data_parallel_communicator.cu:718-720). Because the
 * call then synchronises with the host, do not set a deadline on a communicator that is
 * used while a stream capture is in progress. */
int dwbnq_comm_set_deadline_ms(void *comm, int ms);
/* All-reduce(max) of `count` fp32 values in place; waits at most timeout_ms for
 * completion when timeout_ms > 0 (then aborts the communicator and returns
 * DWBNQ_ERR_TIMEOUT), otherwise only enqueues. */
int dwbnq_comm_allreduce_max_f32(void *comm, float *buf, int64_t count, void *stream,
                                 int timeout_ms);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* DWBNQ_H_ */
