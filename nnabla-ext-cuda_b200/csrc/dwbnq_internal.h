// Host-side declarations shared by the translation units of libdwbnq.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/dwbnq.h"
#include "../../include/dwbnq_debug.h"
#include "dwbnq_fused.cuh"
#include "dwbnq_plane.cuh"
#include "dwbnq_plane_gen.cuh"

namespace dwbnq {

// ---- errors (thread-local message behind dwbnq_last_error_string) ----------------------
int fail(int status, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
int fail_cuda(cudaError_t e, const char *what);
void clear_error();

// Makes `device` current (-1 keeps the current one) and returns its ordinal in *out.
int enter_device(int device, int *out);

// Launch with programmatic stream serialization: the grid may become resident while its
// predecessor in the stream drains; the kernels of this library wait for the predecessor's
// completion (griddepcontrol.wait) before their first global access, so stream order holds.
// DWBNQ_PDL=0 in the environment launches plainly.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args &&... args) {
  cudaLaunchConfig_t lc = {};
  lc.gridDim = grid;
  lc.blockDim = block;
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&lc, kern, std::forward<Args>(args)...);
}

// ---- fused / dw-conv family (fused.cu) --------------------------------------------------
enum FusedPath : int { PATH_AUTO = -1, PATH_GENERIC = 0, PATH_COOP = 1, PATH_TMA = 2, PATH_RAW = 3, PATH_PLANE = 4, PATH_PLANE_GEN = 5 };

struct Plan {
  int path;
  TileCfg cfg;
  PlaneGenCfg gen;  // PATH_PLANE_GEN
  long long ctas;
  int threads;
  size_t smem;
};

// Chooses kernel family and tile geometry for a convolution. `x` / `y` are only
// inspected for alignment.
int make_plan(const dwbnq_conv_desc &d, const void *x, const void *y, Plan *plan);
// Launches the fused kernel in mode `qm` (QMode). a.q must already be filled.
int launch_fused(const dwbnq_conv_desc &d, FusedArgs &a, int qm, int device, cudaStream_t stream);
int forced_path();
void set_forced_path(int p);
// Address of the per-device word kernels set when a bounded wait runs out.
int device_flag_ptr(int device, int **ptr);

int validate_conv(const dwbnq_conv_desc *d, int *ho, int *wo);
// Streaming multiprocessors of `device` (-1 = the current device), cached per device.
int sm_count(int device);

// ---- element-wise family (elementwise.cu) -----------------------------------------------
int launch_bn_infer(int dtype, long long size0, long long size1, long long size2, float eps,
                    const void *x, const void *beta, const void *gamma, const void *mean,
                    const void *var, void *y, cudaStream_t stream);
int launch_fpq(int dtype, long long size, const QuantArgs &q, const void *x, void *y,
               cudaStream_t stream);
int launch_pow2q(int dtype, long long size, const QuantArgs &q, const void *x, void *y,
                 cudaStream_t stream);

// QuantizeLinear / DequantizeLinear with 8-bit codes (scalar scale and zero point).
int launch_quantize_linear_code8(int dtype, long long size, float scale, int zero_point, int round_mode,
                                 int min_range, int max_range, const void *x, void *codes, cudaStream_t stream);
int launch_dequantize_linear_code8(int dtype, long long size, float scale, int zero_point, int codes_signed,
                                   const void *codes, void *y, cudaStream_t stream);

// MinMaxQuantize pieces. Workspace layout (4-byte words, C = channels):
//   [0,C) encoded min | [C,2C) encoded max | [2C,3C) scale | [3C,4C) m' | [4C,5C) M' |
//   [5C,7C) packed [max..., -min...] for the all-reduce.
struct MmWorkspace {
  unsigned int *enc_min, *enc_max;
  float *scale, *lo, *hi, *packed;
};
MmWorkspace mm_workspace(void *ws, int channels);
int launch_mm_init(const MmWorkspace &w, int channels, cudaStream_t stream);
int launch_mm_reduce(int dtype, long long size0, int channels, long long size2, const void *x,
                     const MmWorkspace &w, cudaStream_t stream);
int launch_mm_pack(const MmWorkspace &w, int channels, cudaStream_t stream);
// Updates qr_min / qr_max (when x_min_max) and derives scale, m', M'. `from_packed`
// selects the all-reduced packed vector instead of the encoded slots as the source.
int launch_mm_ranges(int dtype, int channels, const dwbnq_quant_desc &q,
                     const dwbnq_minmax_ptrs &mm, const MmWorkspace &w, int from_packed,
                     cudaStream_t stream);
int launch_mm_apply(int dtype, long long size0, int channels, long long size2, const void *x,
                    void *y, const MmWorkspace &w, cudaStream_t stream);

// ---- quantizer parameters (quant_params.cpp, host only) ----------------------------------
void fpq_range(int sign, int n, float delta, float *mx, float *mn);
void pow2q_range(int sign, int with_zero, int n, int m, float *p_max, float *p_min, float *thr);
int fill_fpq(QuantArgs *q, int sign, int n, float delta);
// Host threshold table (277 entries) and the mantissa window around sqrt(2) outside of
// which the decision needs no table.
const uint32_t *pow2_table_host();
int pow2_table_window();
// Fills the Pow2 part of q, uploading the table to `device` on first use.
int fill_pow2(QuantArgs *q, int sign, int with_zero, int n, int m, int device);
// Device copy of the table (pow2_table_dev.cu).
int pow2_table_device(int device, const uint32_t **ptr);

// ---- training side (backward.cu) ---------------------------------------------------------------
// Straight-through backward of a quantizer. mode 0 = pass-through, 1 = FixedPointQuantize mask
// (fpq_max / fpq_min), 2 = Pow2Quantize mask (pow2_first_above: the smallest magnitude pattern
// whose rounded power of two exceeds p_max; pow2_sign).
int launch_ste_backward(int dtype, int mode, int accum, long long size, float fpq_max, float fpq_min,
                        unsigned int pow2_first_above, int pow2_sign, const void *x, const void *dy, void *dx,
                        cudaStream_t stream);
// Gradients of DepthwiseConvolution (fp32); any of dx, dw, db may be null. accum_mask: bit 0
// dx, bit 1 dw, bit 2 db are accumulated onto instead of overwritten.
int launch_dwconv_backward(const dwbnq_conv_desc &d, int ho, int wo, const void *x, const void *w, const void *dy,
                           void *dx, void *dw, void *db, int accum_mask, cudaStream_t stream);
// Smallest float bit pattern a > 0 with 2^round(log2f(a)) >= v (host libm, bisection).
uint32_t pow2_first_pattern_reaching(float v);

// ---- pointwise convolution (pointwise.cu) ------------------------------------------------------
int pwconv_validate(const dwbnq_pwconv_desc *d);
size_t pwconv_workspace_bytes(const dwbnq_pwconv_desc &d);
// 1 = the tcgen05 kernel, 0 = the plain FMA kernel (thread's forced choice included).
int pwconv_path(const dwbnq_pwconv_desc &d, const void *x, const void *w);
// Launch shape of the tcgen05 kernel for a descriptor on a device of `sms` SMs (diagnostic):
// columns per channel tile, channel tiles, activation path (0 TMA, 1 one-element gather, 2
// four-position gather), tiles, CTAs, pipeline stages, accumulator buffers, shared-column epilogue.
int pwconv_tiling(const dwbnq_pwconv_desc &d, const void *x, int sms, int out[8]);
void set_forced_pw_path(int p);
void set_pw_max_ctas(int n);
// The two halves of launch_pwconv: fill the workspace from the parameters; run on a filled one.
int pwconv_prepare(const dwbnq_pwconv_desc &d, float bn_eps, const void *w, const void *b, const void *beta,
                   const void *gamma, const void *mean, const void *var, void *workspace, cudaStream_t stream);
int pwconv_run(const dwbnq_pwconv_desc &d, const dwbnq_quant_desc *q, int has_bn, const void *x, void *y,
               void *workspace, int dev, cudaStream_t stream);
// Prepares the per-channel coefficients (and the TF32 halves of w) in `workspace`, then runs
// the convolution with the fused epilogue. BN is skipped when mean is null; q may be null.
int launch_pwconv(const dwbnq_pwconv_desc &d, float bn_eps, const dwbnq_quant_desc *q, const void *x, const void *w,
                  const void *b, const void *beta, const void *gamma, const void *mean, const void *var, void *y,
                  void *workspace, int dev, cudaStream_t stream);

// ---- communicator (comm.cpp) --------------------------------------------------------------
int comm_allreduce_max(void *comm, float *buf, long long count, cudaStream_t stream,
                       int timeout_ms);
// Deadline (ms, 0 = none) the communicator carries for the collectives the MINMAX entry
// points issue on the caller's behalf.
int comm_deadline_ms(void *comm);

}  // namespace dwbnq
