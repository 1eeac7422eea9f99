// extern "C" surface of libdwbnq (include/dwbnq.h): argument validation, error strings
// and the operator-level sequencing. No kernel lives here.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <cstdlib>

#include <nvtx3/nvToolsExt.h>

#include "dwbnq_internal.h"

namespace dwbnq {

// A named NVTX range around each operator call, so that a timeline shows which library call
// a kernel belongs to (the reference wraps its own regions the same way,
// src/nbla/cuda/nvtx.cpp:35-59). Header-only NVTX: without a profiler attached the push and
// the pop are a pointer test each.
struct NvtxRange {
  explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange &) = delete;
  NvtxRange &operator=(const NvtxRange &) = delete;
};

bool pdl_enabled() {
  static const bool enabled = [] {
    const char *e = std::getenv("DWBNQ_PDL");
    return !(e && e[0] == '0');
  }();
  return enabled;
}


namespace {
thread_local char g_err[512] = "";
}

void clear_error() { g_err[0] = '\0'; }

int fail(int status, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

int fail_cuda(cudaError_t e, const char *what) {
  (void)cudaGetLastError();  // clear the sticky-less error state
  return fail(DWBNQ_ERR_CUDA, "%s failed: (%s) %s", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

int enter_device(int device, int *out) {
  cudaError_t e;
  if (device >= 0) {
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
    *out = device;
    return DWBNQ_OK;
  }
  int cur = 0;
  e = cudaGetDevice(&cur);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  *out = cur;
  return DWBNQ_OK;
}

namespace {

int check_dtype(int dtype) {
  if (dtype != DWBNQ_F32 && dtype != DWBNQ_F16)
    return fail(DWBNQ_ERR_INVALID_ARG, "dtype %d is neither DWBNQ_F32 nor DWBNQ_F16", dtype);
  return DWBNQ_OK;
}

int check_mm(const dwbnq_quant_desc *q, const dwbnq_minmax_ptrs *mm, const void *workspace) {
  if (!mm || !mm->qr_min || !mm->qr_max || !mm->ql_min || !mm->ql_max)
    return fail(DWBNQ_ERR_INVALID_ARG, "MinMaxQuantize needs qr_min, qr_max, ql_min and ql_max");
  if (!workspace) return fail(DWBNQ_ERR_INVALID_ARG, "MinMaxQuantize needs a workspace");
  if (reinterpret_cast<uintptr_t>(workspace) % 256)
    return fail(DWBNQ_ERR_INVALID_ARG, "workspace must be 256-byte aligned");
  if (q->ema && !(q->decay >= 0.0f && q->decay <= 1.0f))
    return fail(DWBNQ_ERR_INVALID_ARG, "decay %g is not in [0, 1]", q->decay);
  return DWBNQ_OK;
}

// The range part of MinMaxQuantize once the encoded per-channel min/max are in the
// workspace: optional all-reduce across shards, then the range derivation. The collective
// runs under the deadline the communicator carries (dwbnq_comm_set_deadline_ms): with one
// set, a peer that never joins ends this call with DWBNQ_ERR_TIMEOUT and an aborted
// communicator instead of a stream that never drains.
int mm_finish_ranges(int dtype, int channels, const dwbnq_quant_desc &q, const dwbnq_minmax_ptrs &mm,
                     const MmWorkspace &w, void *comm, cudaStream_t stream) {
  int st;
  int from_packed = 0;
  if (q.x_min_max && comm) {
    st = launch_mm_pack(w, channels, stream);
    if (st != DWBNQ_OK) return st;
    st = comm_allreduce_max(comm, w.packed, 2LL * channels, stream, comm_deadline_ms(comm));
    if (st != DWBNQ_OK) return st;
    from_packed = 1;
  }
  return launch_mm_ranges(dtype, channels, q, mm, w, from_packed, stream);
}

void fill_args(FusedArgs *a, const dwbnq_conv_desc &d, int ho, int wo, float eps, const void *x,
               const void *w, const void *b, const void *beta, const void *gamma, const void *mean,
               const void *var, void *y) {
  std::memset(a, 0, sizeof(*a));
  a->x = x;
  a->w = w;
  a->b = b;
  a->beta = beta;
  a->gamma = gamma;
  a->mean = mean;
  a->var = var;
  a->y = y;
  a->eps = eps;
  a->has_bn = mean != nullptr;
  a->n = d.n;
  a->C = d.c;
  a->H = d.h;
  a->W = d.w;
  a->OC = d.c * d.multiplier;
  a->Ho = ho;
  a->Wo = wo;
  a->kh = d.kh;
  a->kw = d.kw;
  a->sh = d.stride_h;
  a->sw = d.stride_w;
  a->ph = d.pad_h;
  a->pw = d.pad_w;
  a->dh = d.dil_h;
  a->dw = d.dil_w;
  a->mult = d.multiplier;
}

}  // namespace
}  // namespace dwbnq

using namespace dwbnq;

extern "C" {

int dwbnq_version(void) { return DWBNQ_ABI_VERSION; }

const char *dwbnq_last_error_string(void) { return g_err; }

int dwbnq_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

int dwbnq_check_device_flag(int device) {
  clear_error();
  int dev;
  int st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  int *p = nullptr;
  st = device_flag_ptr(dev, &p);
  if (st != DWBNQ_OK) return st;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceSynchronize");
  int v = 0;
  e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpy(device flag)");
  if (v) {
    const int zero = 0;
    cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
    return fail(DWBNQ_ERR_DEVICE_FLAG,
                "a kernel recorded an error on device %d (flag %d: 1 = a bounded wait ran out, 2 = an index left its "
                "tensor in the bounds-checked build)",
                dev, v);
  }
  return DWBNQ_OK;
}

int dwbnq_conv_out_shape(const dwbnq_conv_desc *desc, int32_t *ho, int32_t *wo) {
  clear_error();
  int h, w;
  int st = validate_conv(desc, &h, &w);
  if (st != DWBNQ_OK) return st;
  if (ho) *ho = h;
  if (wo) *wo = w;
  return DWBNQ_OK;
}

int dwbnq_fpq_range(int sign, int n, float delta, float *max_out, float *min_out) {
  clear_error();
  if (!max_out || !min_out) return fail(DWBNQ_ERR_INVALID_ARG, "output pointer is null");
  QuantArgs q;
  int st = fill_fpq(&q, sign, n, delta);
  if (st != DWBNQ_OK) return st;
  *max_out = q.fpq_max;
  *min_out = q.fpq_min;
  return DWBNQ_OK;
}

int dwbnq_pow2q_range(int sign, int with_zero, int n, int m, float *p_max, float *p_min,
                      float *pruning_threshold) {
  clear_error();
  if (!p_max || !p_min || !pruning_threshold) return fail(DWBNQ_ERR_INVALID_ARG, "output pointer is null");
  if (n < 1 || n > 31) return fail(DWBNQ_ERR_INVALID_ARG, "Pow2Quantize: bit width n=%d out of range", n);
  pow2q_range(sign, with_zero, n, m, p_max, p_min, pruning_threshold);
  return DWBNQ_OK;
}

int dwbnq_pow2q_threshold_table(uint32_t *table277) {
  clear_error();
  if (!table277) return fail(DWBNQ_ERR_INVALID_ARG, "table pointer is null");
  std::memcpy(table277, pow2_table_host(), 277 * sizeof(uint32_t));
  return DWBNQ_OK;
}

size_t dwbnq_workspace_bytes(int32_t channels) {
  if (channels <= 0) return 0;
  const size_t b = (size_t)channels * 7 * 4;
  return (b + 255) / 256 * 256;
}

size_t dwbnq_pwconv_workspace_bytes(const dwbnq_pwconv_desc *desc) {
  clear_error();
  if (pwconv_validate(desc) != DWBNQ_OK) return 0;
  return pwconv_workspace_bytes(*desc);
}

int dwbnq_pwconv_fused_fwd(const dwbnq_pwconv_desc *desc, float bn_eps, const dwbnq_quant_desc *q, const void *x,
                           const void *w, const void *b, const void *bn_beta, const void *bn_gamma,
                           const void *bn_mean, const void *bn_var, void *y, void *workspace, int device,
                           void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_pwconv_fused_fwd");
  int st = pwconv_validate(desc);
  if (st != DWBNQ_OK) return st;
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  return launch_pwconv(*desc, bn_eps, q, x, w, b, bn_beta, bn_gamma, bn_mean, bn_var, y, workspace, dev,
                       static_cast<cudaStream_t>(stream));
}

int dwbnq_pwconv_fwd(const dwbnq_pwconv_desc *desc, const void *x, const void *w, const void *b, void *y,
                     void *workspace, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_pwconv_fwd");
  int st = pwconv_validate(desc);
  if (st != DWBNQ_OK) return st;
  if (desc->act != DWBNQ_ACT_NONE) return fail(DWBNQ_ERR_INVALID_ARG, "dwbnq_pwconv_fwd takes no activation (act = %d)", desc->act);
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  return launch_pwconv(*desc, 0.0f, nullptr, x, w, b, nullptr, nullptr, nullptr, nullptr, y, workspace, dev,
                       static_cast<cudaStream_t>(stream));
}

int dwbnq_pwconv_prepare(const dwbnq_pwconv_desc *desc, float bn_eps, const void *w, const void *b, const void *bn_beta,
                         const void *bn_gamma, const void *bn_mean, const void *bn_var, void *workspace, int device,
                         void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_pwconv_prepare");
  int st = pwconv_validate(desc);
  if (st != DWBNQ_OK) return st;
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  return pwconv_prepare(*desc, bn_eps, w, b, bn_beta, bn_gamma, bn_mean, bn_var, workspace, static_cast<cudaStream_t>(stream));
}

int dwbnq_pwconv_fused_fwd_prepared(const dwbnq_pwconv_desc *desc, const dwbnq_quant_desc *q, int has_bn, const void *x,
                                    void *y, void *workspace, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_pwconv_fused_fwd_prepared");
  int st = pwconv_validate(desc);
  if (st != DWBNQ_OK) return st;
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  return pwconv_run(*desc, q, has_bn, x, y, workspace, dev, static_cast<cudaStream_t>(stream));
}

int dwbnq_pwconv_plan(const dwbnq_pwconv_desc *desc, const void *x, const void *w, int *path_out) {
  clear_error();
  int st = pwconv_validate(desc);
  if (st != DWBNQ_OK) return st;
  if (!path_out) return fail(DWBNQ_ERR_INVALID_ARG, "path_out is null");
  *path_out = pwconv_path(*desc, x, w);
  return DWBNQ_OK;
}

int dwbnq_debug_pwconv_tiling(const dwbnq_pwconv_desc *desc, const void *x, int sms, int *out8) {
  clear_error();
  int st = pwconv_validate(desc);
  if (st != DWBNQ_OK) return st;
  if (!out8) return fail(DWBNQ_ERR_INVALID_ARG, "out8 is null");
  if (sms <= 0) return fail(DWBNQ_ERR_INVALID_ARG, "sms %d is not positive", sms);
  return pwconv_tiling(*desc, x, sms, out8);
}

int dwbnq_set_forced_pw_path(int path) {
  clear_error();
  if (path < -1 || path > 1) return fail(DWBNQ_ERR_INVALID_ARG, "pointwise path %d is not -1, 0 or 1", path);
  set_forced_pw_path(path);
  return DWBNQ_OK;
}

int dwbnq_set_pw_max_ctas(int ctas) {
  clear_error();
  if (ctas < 0) return fail(DWBNQ_ERR_INVALID_ARG, "ctas %d is negative", ctas);
  set_pw_max_ctas(ctas);
  return DWBNQ_OK;
}

int dwbnq_set_forced_path(int path) {
  clear_error();
  if (path < PATH_AUTO || path > PATH_PLANE_GEN) return fail(DWBNQ_ERR_INVALID_ARG, "path %d is not -1..5", path);
  set_forced_path(path);
  return DWBNQ_OK;
}

int dwbnq_fused_plan(const dwbnq_conv_desc *desc, const void *x, const void *y, int *path_out,
                     int *planes_per_cta, int *rows_per_tile, int *threads, int64_t *ctas,
                     int *smem_bytes) {
  clear_error();
  if (!desc) return fail(DWBNQ_ERR_INVALID_ARG, "conv desc is null");
  Plan p;
  int st = make_plan(*desc, x, y, &p);
  if (st != DWBNQ_OK) return st;
  if (path_out) *path_out = p.path;
  if (planes_per_cta) *planes_per_cta = p.cfg.P;
  if (rows_per_tile) *rows_per_tile = p.cfg.TH;
  if (threads) *threads = p.threads;
  if (ctas) *ctas = p.ctas;
  if (smem_bytes) *smem_bytes = (int)p.smem;
  return DWBNQ_OK;
}

int dwbnq_fused_fwd(const dwbnq_conv_desc *desc, float bn_eps, const dwbnq_quant_desc *q,
                    const void *x, const void *w, const void *b, const void *bn_beta,
                    const void *bn_gamma, const void *bn_mean, const void *bn_var,
                    const dwbnq_minmax_ptrs *mm, void *y, void *workspace, void *comm, int device,
                    void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_fused_fwd");
  int ho, wo;
  int st = validate_conv(desc, &ho, &wo);
  if (st != DWBNQ_OK) return st;
  const int kind = q ? q->kind : DWBNQ_Q_NONE;
  if (kind < DWBNQ_Q_NONE || kind > DWBNQ_Q_MINMAX)
    return fail(DWBNQ_ERR_INVALID_ARG, "quantizer kind %d unknown", kind);
  // An empty batch has nothing to read or write - unless this rank's (empty) shard belongs
  // to a batch whose per-channel min/max are all-reduced: then the rank must still take
  // part in the collective (its identities +inf / -inf are neutral under max), or its peers
  // would wait for it forever, and it must derive the same ranges as they do.
  const bool empty = desc->n == 0;
  const bool empty_joins = empty && kind == DWBNQ_Q_MINMAX && q->x_min_max && comm != nullptr;
  if (empty && !empty_joins) return DWBNQ_OK;
  if (!empty && (!x || !w || !y)) return fail(DWBNQ_ERR_INVALID_ARG, "x, w and y must not be null");
  if ((bn_mean == nullptr) != (bn_var == nullptr))
    return fail(DWBNQ_ERR_INVALID_ARG, "bn_mean and bn_var must be given together");
  if (kind == DWBNQ_Q_MINMAX) {
    st = check_mm(q, mm, workspace);
    if (st != DWBNQ_OK) return st;
  }
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  FusedArgs a;
  fill_args(&a, *desc, ho, wo, bn_eps, x, w, b, bn_beta, bn_gamma, bn_mean, bn_var, y);
  switch (kind) {
    case DWBNQ_Q_NONE:
      return launch_fused(*desc, a, QM_NONE, dev, s);
    case DWBNQ_Q_FPQ:
      st = fill_fpq(&a.q, q->sign, q->n, q->delta);
      if (st != DWBNQ_OK) return st;
      return launch_fused(*desc, a, QM_FPQ, dev, s);
    case DWBNQ_Q_POW2:
      st = fill_pow2(&a.q, q->sign, q->with_zero, q->n, q->m, dev);
      if (st != DWBNQ_OK) return st;
      return launch_fused(*desc, a, QM_POW2, dev, s);
    default:
      break;
  }
  // MinMaxQuantize: a first pass reduces the activation to per-channel min / max (encoded
  // slots of the workspace), the ranges are derived (after the all-reduce, for a sharded
  // batch), and a second pass quantizes. Which form the two passes take is chosen below.
  const int channels = a.OC;
  const MmWorkspace ws = mm_workspace(workspace, channels);
  a.q.mm_enc_min = ws.enc_min;
  a.q.mm_enc_max = ws.enc_max;
  a.q.mm_scale = ws.scale;
  a.q.mm_lo = ws.lo;
  a.q.mm_hi = ws.hi;
  if (empty_joins) {
    st = launch_mm_init(ws, channels, s);
    if (st != DWBNQ_OK) return st;
    return mm_finish_ranges(desc->dtype, channels, *q, *mm, ws, comm, s);
  }
  if (q->x_min_max) {
    st = launch_mm_init(ws, channels, s);
    if (st != DWBNQ_OK) return st;
    // fp32 on the plane family: the first pass also stores the activation in y (exact in
    // fp32) and the second pass quantizes y in place, 1.3x less traffic than recomputing.
    // fp16 must recompute: its contract is one rounding, of the quantized value.
    Plan plan;
    st = make_plan(*desc, a.x, a.y, &plan);
    if (st != DWBNQ_OK) return st;
    const bool store_first = desc->dtype == DWBNQ_F32 && (plan.path == PATH_PLANE || plan.path == PATH_PLANE_GEN);
    st = launch_fused(*desc, a, store_first ? QM_MM_REDUCE_STORE : QM_MM_REDUCE, dev, s);
    if (st != DWBNQ_OK) return st;
    if (store_first) {
      st = mm_finish_ranges(desc->dtype, channels, *q, *mm, ws, comm, s);
      if (st != DWBNQ_OK) return st;
      return launch_mm_apply(desc->dtype, desc->n, channels, (long long)ho * wo, y, y, ws, s);
    }
  }
  st = mm_finish_ranges(desc->dtype, channels, *q, *mm, ws, comm, s);
  if (st != DWBNQ_OK) return st;
  return launch_fused(*desc, a, QM_MM_APPLY, dev, s);
}

int dwbnq_fused_fwd_code8(const dwbnq_conv_desc *desc, float bn_eps, const dwbnq_quant_desc *q,
                          const dwbnq_code8_desc *io, const void *x_codes, const void *w, const void *b,
                          const void *bn_beta, const void *bn_gamma, const void *bn_mean, const void *bn_var,
                          void *y_codes, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_fused_fwd_code8");
  int ho, wo;
  int st = validate_conv(desc, &ho, &wo);
  if (st != DWBNQ_OK) return st;
  if (desc->dtype != DWBNQ_F32)
    return fail(DWBNQ_ERR_UNSUPPORTED, "8-bit storage: weights and BN vectors must be DWBNQ_F32");
  if (!q || q->kind != DWBNQ_Q_FPQ)
    return fail(DWBNQ_ERR_INVALID_ARG, "8-bit storage needs a FixedPointQuantize quantizer (its codes are what is stored)");
  if (!io) return fail(DWBNQ_ERR_INVALID_ARG, "code8 desc is null");
  if (!(io->in_delta > 0.0f) || io->in_delta > 3.0e38f)
    return fail(DWBNQ_ERR_INVALID_ARG, "in_delta must be positive and finite");
  if (desc->n == 0) return DWBNQ_OK;
  if (!x_codes || !w || !y_codes) return fail(DWBNQ_ERR_INVALID_ARG, "x, w and y must not be null");
  if ((bn_mean == nullptr) != (bn_var == nullptr))
    return fail(DWBNQ_ERR_INVALID_ARG, "bn_mean and bn_var must be given together");
  FusedArgs a;
  fill_args(&a, *desc, ho, wo, bn_eps, x_codes, w, b, bn_beta, bn_gamma, bn_mean, bn_var, y_codes);
  st = fill_fpq(&a.q, q->sign, q->n, q->delta);
  if (st != DWBNQ_OK) return st;
  if (q->n > 8) return fail(DWBNQ_ERR_UNSUPPORTED, "8-bit storage: FixedPointQuantize with n = %d does not fit a byte", q->n);
  if (!a.q.fpq_fast)
    return fail(DWBNQ_ERR_UNSUPPORTED, "8-bit storage needs delta to be a power of two (the code y / delta is then exact)");
  a.code8 = 1;
  a.code_in_signed = io->in_signed ? 1 : 0;
  a.code_in_delta = io->in_delta;
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  return launch_fused(*desc, a, QM_FPQ, dev, static_cast<cudaStream_t>(stream));
}

int dwbnq_quantize_linear_code8_fwd(int dtype, int64_t size, float scale, int zero_point, int round_mode,
                                    int min_range, int max_range, const void *x, void *codes, int device,
                                    void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_quantize_linear_code8_fwd");
  int st = check_dtype(dtype);
  if (st != DWBNQ_OK) return st;
  if (size < 0) return fail(DWBNQ_ERR_INVALID_ARG, "negative size");
  if (!(scale > 0.0f) || scale > 3.0e38f) return fail(DWBNQ_ERR_INVALID_ARG, "scale must be positive and finite");
  if (round_mode != DWBNQ_ROUND_HALF_AWAY_FROM_ZERO && round_mode != DWBNQ_ROUND_HALF_TO_EVEN)
    return fail(DWBNQ_ERR_INVALID_ARG, "round mode %d unknown", round_mode);
  if (min_range > max_range) return fail(DWBNQ_ERR_INVALID_ARG, "min_range %d > max_range %d", min_range, max_range);
  if (min_range < 0 ? (min_range < -128 || max_range > 127) : max_range > 255)
    return fail(DWBNQ_ERR_UNSUPPORTED, "range [%d, %d] does not fit %s", min_range, max_range,
                min_range < 0 ? "int8" : "uint8");
  if (size > 0 && (!x || !codes)) return fail(DWBNQ_ERR_INVALID_ARG, "x and codes must not be null");
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  if (size == 0) return DWBNQ_OK;
  return launch_quantize_linear_code8(dtype, size, scale, zero_point, round_mode, min_range, max_range, x, codes,
                                      static_cast<cudaStream_t>(stream));
}

int dwbnq_dequantize_linear_code8_fwd(int dtype, int64_t size, float scale, int zero_point, int codes_signed,
                                      const void *codes, void *y, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_dequantize_linear_code8_fwd");
  int st = check_dtype(dtype);
  if (st != DWBNQ_OK) return st;
  if (size < 0) return fail(DWBNQ_ERR_INVALID_ARG, "negative size");
  if (size > 0 && (!codes || !y)) return fail(DWBNQ_ERR_INVALID_ARG, "codes and y must not be null");
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  if (size == 0) return DWBNQ_OK;
  return launch_dequantize_linear_code8(dtype, size, scale, zero_point, codes_signed, codes, y,
                                        static_cast<cudaStream_t>(stream));
}

int dwbnq_fpq_bwd(int dtype, int64_t size, int sign, int n, float delta, int ste_fine_grained, int accum,
                  const void *x, const void *dy, void *dx, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_fpq_bwd");
  int st = check_dtype(dtype);
  if (st != DWBNQ_OK) return st;
  if (size < 0) return fail(DWBNQ_ERR_INVALID_ARG, "negative size");
  QuantArgs q;
  std::memset(&q, 0, sizeof(q));
  st = fill_fpq(&q, sign, n, delta);
  if (st != DWBNQ_OK) return st;
  if (size > 0 && (!dy || !dx || (ste_fine_grained && !x)))
    return fail(DWBNQ_ERR_INVALID_ARG, "dy and dx (and x for the fine-grained form) must not be null");
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  if (size == 0) return DWBNQ_OK;
  return launch_ste_backward(dtype, ste_fine_grained ? 1 : 0, accum, size, q.fpq_max, q.fpq_min, 0u, 0, x, dy, dx,
                             static_cast<cudaStream_t>(stream));
}

int dwbnq_pow2q_bwd(int dtype, int64_t size, int sign, int with_zero, int n, int m, int ste_fine_grained, int accum,
                    const void *x, const void *dy, void *dx, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_pow2q_bwd");
  int st = check_dtype(dtype);
  if (st != DWBNQ_OK) return st;
  if (size < 0) return fail(DWBNQ_ERR_INVALID_ARG, "negative size");
  if (n < 1 || n > 31) return fail(DWBNQ_ERR_INVALID_ARG, "Pow2Quantize: bit width n=%d out of range", n);
  if (size > 0 && (!dy || !dx || (ste_fine_grained && !x)))
    return fail(DWBNQ_ERR_INVALID_ARG, "dy and dx (and x for the fine-grained form) must not be null");
  float p_max, p_min, thr;
  pow2q_range(sign, with_zero, n, m, &p_max, &p_min, &thr);
  // q > p_max for powers of two q: q >= 2 * p_max (an overflow to inf leaves only |x| = inf)
  const uint32_t first_above = pow2_first_pattern_reaching(p_max * 2.0f);
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  if (size == 0) return DWBNQ_OK;
  return launch_ste_backward(dtype, ste_fine_grained ? 2 : 0, accum, size, 0.0f, 0.0f, first_above, sign ? 1 : 0, x, dy,
                             dx, static_cast<cudaStream_t>(stream));
}

int dwbnq_dwconv_bwd(const dwbnq_conv_desc *desc, const void *x, const void *w, const void *dy, void *dx, void *dw,
                     void *db, int accum_mask, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_dwconv_bwd");
  int ho, wo;
  int st = validate_conv(desc, &ho, &wo);
  if (st != DWBNQ_OK) return st;
  if (desc->dtype != DWBNQ_F32)
    return fail(DWBNQ_ERR_UNSUPPORTED, "DepthwiseConvolution backward is implemented for DWBNQ_F32");
  if (!dx && !dw && !db) return DWBNQ_OK;  // nothing to propagate (the reference returns early too)
  if (!dy) return fail(DWBNQ_ERR_INVALID_ARG, "dy must not be null");
  if (dx && !w) return fail(DWBNQ_ERR_INVALID_ARG, "the input gradient needs w");
  if (dw && !x) return fail(DWBNQ_ERR_INVALID_ARG, "the weight gradient needs x");
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  if (desc->n == 0 && !dw && !db) return DWBNQ_OK;
  return launch_dwconv_backward(*desc, ho, wo, x, w, dy, dx, dw, db, accum_mask, static_cast<cudaStream_t>(stream));
}

int dwbnq_dwconv_fwd(const dwbnq_conv_desc *desc, const void *x, const void *w, const void *b,
                     void *y, int device, void *stream) {
  return dwbnq_fused_fwd(desc, 0.0f, nullptr, x, w, b, nullptr, nullptr, nullptr, nullptr, nullptr, y,
                         nullptr, nullptr, device, stream);
}

int dwbnq_bn_infer_fwd(int dtype, int64_t size0, int64_t size1, int64_t size2, float eps,
                       const void *x, const void *beta, const void *gamma, const void *mean,
                       const void *var, void *y, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_bn_infer_fwd");
  int st = check_dtype(dtype);
  if (st != DWBNQ_OK) return st;
  if (size0 < 0 || size1 <= 0 || size2 < 0)
    return fail(DWBNQ_ERR_INVALID_ARG, "view [%lld,%lld,%lld] is not a valid shape", (long long)size0,
                (long long)size1, (long long)size2);
  if (!x || !y || !mean || !var) return fail(DWBNQ_ERR_INVALID_ARG, "x, y, mean and var must not be null");
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  return launch_bn_infer(dtype, size0, size1, size2, eps, x, beta, gamma, mean, var, y,
                         static_cast<cudaStream_t>(stream));
}

int dwbnq_fpq_fwd(int dtype, int64_t size, int sign, int n, float delta, const void *x, void *y,
                  int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_fpq_fwd");
  int st = check_dtype(dtype);
  if (st != DWBNQ_OK) return st;
  if (size < 0) return fail(DWBNQ_ERR_INVALID_ARG, "negative size");
  if (size > 0 && (!x || !y)) return fail(DWBNQ_ERR_INVALID_ARG, "x and y must not be null");
  QuantArgs q;
  std::memset(&q, 0, sizeof(q));
  st = fill_fpq(&q, sign, n, delta);
  if (st != DWBNQ_OK) return st;
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  if (size == 0) return DWBNQ_OK;
  return launch_fpq(dtype, size, q, x, y, static_cast<cudaStream_t>(stream));
}

int dwbnq_pow2q_fwd(int dtype, int64_t size, int sign, int with_zero, int n, int m, const void *x,
                    void *y, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_pow2q_fwd");
  int st = check_dtype(dtype);
  if (st != DWBNQ_OK) return st;
  if (size < 0) return fail(DWBNQ_ERR_INVALID_ARG, "negative size");
  if (size > 0 && (!x || !y)) return fail(DWBNQ_ERR_INVALID_ARG, "x and y must not be null");
  if (n < 1 || n > 31) return fail(DWBNQ_ERR_INVALID_ARG, "Pow2Quantize: bit width n=%d out of range", n);
  if (size == 0) return DWBNQ_OK;
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  QuantArgs q;
  std::memset(&q, 0, sizeof(q));
  st = fill_pow2(&q, sign, with_zero, n, m, dev);
  if (st != DWBNQ_OK) return st;
  return launch_pow2q(dtype, size, q, x, y, static_cast<cudaStream_t>(stream));
}

int dwbnq_minmaxq_fwd(int dtype, int64_t size0, int32_t channels, int64_t size2,
                      const dwbnq_quant_desc *q, const void *x, const dwbnq_minmax_ptrs *mm, void *y,
                      void *workspace, void *comm, int device, void *stream) {
  clear_error();
  NvtxRange nvtx_range("dwbnq_minmaxq_fwd");
  int st = check_dtype(dtype);
  if (st != DWBNQ_OK) return st;
  if (size0 < 0 || channels <= 0 || size2 < 0)
    return fail(DWBNQ_ERR_INVALID_ARG, "view [%lld,%d,%lld] is not a valid shape", (long long)size0, channels,
                (long long)size2);
  if (!q) return fail(DWBNQ_ERR_INVALID_ARG, "quantizer desc is null");
  if (!x || !y) return fail(DWBNQ_ERR_INVALID_ARG, "x and y must not be null");
  st = check_mm(q, mm, workspace);
  if (st != DWBNQ_OK) return st;
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const MmWorkspace ws = mm_workspace(workspace, channels);
  if (q->x_min_max) {
    st = launch_mm_init(ws, channels, s);
    if (st != DWBNQ_OK) return st;
    st = launch_mm_reduce(dtype, size0, channels, size2, x, ws, s);
    if (st != DWBNQ_OK) return st;
  }
  st = mm_finish_ranges(dtype, channels, *q, *mm, ws, comm, s);
  if (st != DWBNQ_OK) return st;
  return launch_mm_apply(dtype, size0, channels, size2, x, y, ws, s);
}

}  // extern "C"
