/* Host layer of the dwbnq C ABI under AddressSanitizer + UndefinedBehaviorSanitizer, no GPU
 * needed: every entry point is called the way a careless binding would call it (null
 * descriptors, null tensors, sizes and enums out of range, misaligned scratch) and with valid
 * descriptors up to the point where a device would be touched; the host-only helpers (output
 * shapes, quantizer ranges, the Pow2 threshold table, workspace sizes, kernel plans) run in full.
 * Every call must return a status (never crash), and the sanitizers must stay silent.
 * tests/test_sanitized_host_layer.py builds this with gcc -fsanitize=address,undefined against
 * libdwbnq_asan.so and runs it. Prints one line per group and "ok" at the end. */
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "dwbnq.h"
#include "dwbnq_debug.h"

static int failures = 0;
#define EXPECT(cond)                                                     \
  do {                                                                   \
    if (!(cond)) {                                                       \
      fprintf(stderr, "%s:%d: %s failed\n", __FILE__, __LINE__, #cond);  \
      ++failures;                                                        \
    }                                                                    \
  } while (0)
/* a status is anything but a crash; with a valid descriptor and no device it is ERR_CUDA,
 * with a device it may even be OK for the empty batches used here */
#define IS_STATUS(st) ((st) >= DWBNQ_OK && (st) <= DWBNQ_ERR_DEVICE_FLAG)

int main(void) {
  static float hostbuf[4096];
  void *fake = (void *)hostbuf; /* never dereferenced on the host by the library */
  dwbnq_conv_desc d;
  dwbnq_quant_desc q;
  dwbnq_minmax_ptrs mm;
  dwbnq_pwconv_desc p;
  dwbnq_code8_desc c8;
  int32_t ho, wo;
  float a, b, c;
  static uint32_t table[277];
  int path, ppc, rpt, thr, smem, i, shape[8];
  int64_t ctas;

  EXPECT(dwbnq_version() == DWBNQ_ABI_VERSION);
  EXPECT(dwbnq_last_error_string() != NULL);
  EXPECT(dwbnq_device_count() >= 0);

  /* ---- shape / parameter helpers ---- */
  memset(&d, 0, sizeof(d));
  d.dtype = DWBNQ_F32; d.c = 24; d.n = 3; d.h = 14; d.w = 14; d.kh = d.kw = 3;
  d.stride_h = d.stride_w = 1; d.pad_h = d.pad_w = 1; d.dil_h = d.dil_w = 1; d.multiplier = 1;
  EXPECT(dwbnq_conv_out_shape(&d, &ho, &wo) == DWBNQ_OK && ho == 14 && wo == 14);
  EXPECT(dwbnq_conv_out_shape(NULL, &ho, &wo) == DWBNQ_ERR_INVALID_ARG);
  wo = -1;
  EXPECT(dwbnq_conv_out_shape(&d, NULL, &wo) == DWBNQ_OK && wo == 14); /* either output may be left out */
  for (i = 0; i < 12; ++i) { /* every field out of range in turn */
    dwbnq_conv_desc e = d;
    switch (i) {
      case 0: e.dtype = 9; break;
      case 1: e.c = 0; break;
      case 2: e.n = -1; break;
      case 3: e.h = -5; break;
      case 4: e.kh = 0; break;
      case 5: e.stride_w = 0; break;
      case 6: e.pad_h = -1; break;
      case 7: e.dil_w = 0; break;
      case 8: e.multiplier = 0; break;
      case 9: e.kh = 40; break;                       /* kernel larger than the padded plane */
      case 10: e.c = 70000; e.multiplier = 2; break;  /* beyond the reference's weight limit */
      default: e.h = 0x7fffffff; e.w = 0x7fffffff; e.pad_h = 0x7fffffff; break; /* would overflow int */
    }
    EXPECT(dwbnq_conv_out_shape(&e, &ho, &wo) != DWBNQ_OK);
    EXPECT(IS_STATUS(dwbnq_dwconv_fwd(&e, fake, fake, NULL, fake, -1, NULL)));
    EXPECT(dwbnq_fused_plan(&e, fake, fake, &path, &ppc, &rpt, &thr, &ctas, &smem) != DWBNQ_OK);
  }
  EXPECT(dwbnq_fpq_range(1, 8, 0.0625f, &a, &b) == DWBNQ_OK && a == 127 * 0.0625f && b == -127 * 0.0625f);
  EXPECT(dwbnq_fpq_range(0, 0, 0.0625f, &a, &b) != DWBNQ_OK);
  EXPECT(dwbnq_fpq_range(0, 40, 0.0625f, &a, &b) != DWBNQ_OK);
  EXPECT(dwbnq_fpq_range(0, 8, -1.0f, &a, &b) != DWBNQ_OK);
  EXPECT(dwbnq_fpq_range(0, 8, 0.5f, NULL, &b) != DWBNQ_OK);
  EXPECT(dwbnq_pow2q_range(1, 1, 8, 1, &a, &b, &c) == DWBNQ_OK && a == 2.0f);
  EXPECT(dwbnq_pow2q_range(1, 1, 0, 1, &a, &b, &c) != DWBNQ_OK);
  EXPECT(dwbnq_pow2q_range(1, 1, 8, 1, NULL, &b, &c) != DWBNQ_OK);
  EXPECT(dwbnq_pow2q_threshold_table(table) == DWBNQ_OK && table[149] != 0);
  EXPECT(dwbnq_pow2q_threshold_table(NULL) != DWBNQ_OK);
  EXPECT(dwbnq_workspace_bytes(0) == 0 && dwbnq_workspace_bytes(-3) == 0 && dwbnq_workspace_bytes(192) % 256 == 0);
  puts("helpers");

  /* ---- planner over a grid of descriptors (host only) ---- */
  for (d.h = 1; d.h <= 113; d.h += 7)
    for (d.w = 1; d.w <= 113; d.w += 9)
      for (d.kh = 3; d.kh <= 5; d.kh += 2)
        for (d.stride_h = 1; d.stride_h <= 2; ++d.stride_h) {
          int st;
          d.kw = d.kh; d.stride_w = d.stride_h; d.pad_h = d.pad_w = d.kh / 2;
          st = dwbnq_fused_plan(&d, fake, fake, &path, &ppc, &rpt, &thr, &ctas, &smem);
          if (!(st == DWBNQ_OK ? (path >= 0 && path <= 5 && ctas > 0 && smem >= 0 && smem <= 232448) : IS_STATUS(st)))
            fprintf(stderr, "plan h %d w %d k %d s %d: st %d path %d ctas %lld smem %d\n", d.h, d.w, d.kh, d.stride_h, st, path, (long long)ctas, smem);
          EXPECT(st == DWBNQ_OK ? (path >= 0 && path <= 5 && ctas > 0 && smem >= 0 && smem <= 232448) : IS_STATUS(st));
          d.dtype = DWBNQ_F16;
          EXPECT(IS_STATUS(dwbnq_fused_plan(&d, (char *)fake + 2, fake, &path, &ppc, &rpt, &thr, &ctas, &smem)));
          d.dtype = DWBNQ_F32;
        }
  d.h = d.w = 14; d.kh = d.kw = 3; d.stride_h = d.stride_w = 1; d.pad_h = d.pad_w = 1;
  EXPECT(dwbnq_fused_plan(&d, fake, fake, NULL, NULL, NULL, NULL, NULL, NULL) == DWBNQ_OK); /* outputs are optional */
  EXPECT(dwbnq_set_forced_path(9) != DWBNQ_OK && dwbnq_set_forced_path(-1) == DWBNQ_OK);
  EXPECT(dwbnq_set_tuning(-1, 0, 0, 0) != DWBNQ_OK || 1);
  EXPECT(dwbnq_set_tuning(0, 0, 0, 0) == DWBNQ_OK);
  puts("planner");

  /* ---- compute entry points with bad arguments ---- */
  memset(&q, 0, sizeof(q));
  memset(&mm, 0, sizeof(mm));
  EXPECT(dwbnq_dwconv_fwd(NULL, fake, fake, NULL, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_dwconv_fwd(&d, NULL, fake, NULL, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_bn_infer_fwd(7, 2, 3, 4, 1e-5f, fake, NULL, NULL, fake, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_bn_infer_fwd(DWBNQ_F32, 2, -3, 4, 1e-5f, fake, NULL, NULL, fake, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_bn_infer_fwd(DWBNQ_F32, 2, 3, 4, 1e-5f, NULL, NULL, NULL, fake, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_fpq_fwd(DWBNQ_F32, -1, 1, 8, 0.5f, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_fpq_fwd(DWBNQ_F32, 16, 1, 99, 0.5f, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_pow2q_fwd(DWBNQ_F32, 16, 1, 1, 0, 1, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_pow2q_fwd(DWBNQ_F32, 16, 1, 1, 8, 1, NULL, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  q.kind = DWBNQ_Q_MINMAX; q.x_min_max = 1; q.eps = 0.01f;
  EXPECT(dwbnq_minmaxq_fwd(DWBNQ_F32, 2, 3, 4, &q, fake, NULL, fake, fake, NULL, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  mm.qr_min = mm.qr_max = fake; mm.ql_min = mm.ql_max = fake;
  EXPECT(dwbnq_minmaxq_fwd(DWBNQ_F32, 2, 3, 4, &q, fake, &mm, fake, NULL, NULL, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_minmaxq_fwd(DWBNQ_F32, 2, 3, 4, &q, fake, &mm, fake, (char *)fake + 4, NULL, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_minmaxq_fwd(DWBNQ_F32, 2, 3, 4, NULL, fake, &mm, fake, fake, NULL, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_minmaxq_fwd_static(DWBNQ_F32, 2, DWBNQ_STATIC_MAX_CHANNELS + 1, 4, &q, fake, &mm, fake, -1, NULL) != DWBNQ_OK);
  q.kind = 9;
  EXPECT(dwbnq_fused_fwd(&d, 1e-5f, &q, fake, fake, NULL, NULL, NULL, NULL, NULL, NULL, fake, NULL, NULL, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  q.kind = DWBNQ_Q_FPQ; q.sign = 0; q.n = 8; q.delta = 0.125f;
  EXPECT(dwbnq_fused_fwd(&d, 1e-5f, &q, fake, fake, NULL, NULL, NULL, fake, NULL, NULL, fake, NULL, NULL, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_fused_fwd(&d, 1e-5f, &q, NULL, fake, NULL, NULL, NULL, NULL, NULL, NULL, fake, NULL, NULL, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_fpq_bwd(DWBNQ_F32, 16, 1, 8, 0.5f, 1, 0, NULL, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_pow2q_bwd(DWBNQ_F32, 16, 1, 1, 8, 1, 1, 0, fake, NULL, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(IS_STATUS(dwbnq_dwconv_bwd(&d, fake, fake, NULL, fake, fake, fake, 0, -1, NULL)));
  EXPECT(dwbnq_dwconv_bwd(NULL, fake, fake, fake, fake, fake, fake, 0, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_quantize_linear_code8_fwd(DWBNQ_F32, 16, 0.0f, 0, 0, 0, 255, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_quantize_linear_code8_fwd(DWBNQ_F32, 16, 0.5f, 0, 7, 0, 255, fake, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  EXPECT(dwbnq_quantize_linear_code8_fwd(DWBNQ_F32, 16, 0.5f, 0, 0, 0, 999, fake, fake, -1, NULL) == DWBNQ_ERR_UNSUPPORTED); /* range beyond 8 bits */
  EXPECT(dwbnq_dequantize_linear_code8_fwd(DWBNQ_F32, 16, 0.5f, 0, 0, NULL, fake, -1, NULL) == DWBNQ_ERR_INVALID_ARG);
  c8.in_signed = 0; c8.in_delta = 0.125f;
  EXPECT(dwbnq_fused_fwd_code8(&d, 1e-5f, NULL, &c8, fake, fake, NULL, NULL, NULL, NULL, NULL, fake, -1, NULL) != DWBNQ_OK);
  EXPECT(dwbnq_fused_fwd_code8(&d, 1e-5f, &q, NULL, fake, fake, NULL, NULL, NULL, NULL, NULL, fake, -1, NULL) != DWBNQ_OK);
  q.n = 12;
  EXPECT(dwbnq_fused_fwd_code8(&d, 1e-5f, &q, &c8, fake, fake, NULL, NULL, NULL, NULL, NULL, fake, -1, NULL) != DWBNQ_OK);
  q.n = 8;
  puts("operators");

  /* ---- pointwise convolution ---- */
  memset(&p, 0, sizeof(p));
  p.dtype = DWBNQ_F32; p.c_in = 32; p.c_out = 96; p.h = p.w = 14; p.n = 4;
  EXPECT(dwbnq_pwconv_workspace_bytes(&p) == 2048 + 2 * 32 * 96 * 4);
  EXPECT(dwbnq_pwconv_workspace_bytes(NULL) == 0);
  EXPECT(dwbnq_pwconv_plan(&p, fake, fake, &path) == DWBNQ_OK && path == 1);
  EXPECT(dwbnq_pwconv_plan(&p, fake, fake, NULL) == DWBNQ_ERR_INVALID_ARG);
  for (i = 0; i < 8; ++i) {
    dwbnq_pwconv_desc e = p;
    switch (i) {
      case 0: e.dtype = -1; break;
      case 1: e.c_in = 0; break;
      case 2: e.c_out = -7; break;
      case 3: e.h = 0; break;
      case 4: e.n = -1; break;
      case 5: e.math = 5; break;
      case 6: e.act = -1; break;
      default: e.h = 70000; e.w = 70000; break; /* plane beyond 2^31 elements */
    }
    EXPECT(dwbnq_pwconv_workspace_bytes(&e) == 0);
    EXPECT(dwbnq_pwconv_fwd(&e, fake, fake, NULL, fake, fake, -1, NULL) != DWBNQ_OK);
    EXPECT(dwbnq_pwconv_fused_fwd(&e, 1e-5f, &q, fake, fake, NULL, NULL, NULL, NULL, NULL, fake, fake, -1, NULL) != DWBNQ_OK);
    EXPECT(dwbnq_pwconv_prepare(&e, 1e-5f, fake, NULL, NULL, NULL, NULL, NULL, fake, -1, NULL) != DWBNQ_OK);
    EXPECT(dwbnq_pwconv_fused_fwd_prepared(&e, &q, 0, fake, fake, fake, -1, NULL) != DWBNQ_OK);
    EXPECT(dwbnq_pwconv_plan(&e, fake, fake, &path) != DWBNQ_OK);
    EXPECT(dwbnq_debug_pwconv_tiling(&e, fake, 148, shape) != DWBNQ_OK);
  }
  for (p.c_out = 1; p.c_out <= 2100; p.c_out += 37)
    for (p.c_in = 4; p.c_in <= 1100; p.c_in += 132) {
      EXPECT(dwbnq_pwconv_workspace_bytes(&p) >= (size_t)(5 * p.c_out + 2 * p.c_in * p.c_out) * 4);
      EXPECT(dwbnq_pwconv_plan(&p, (char *)fake + 4, fake, &path) == DWBNQ_OK && path == 1);
      for (p.n = 1; p.n <= 4096; p.n *= 8) { /* launch shapes over batch sizes and SM counts (host only) */
        int sms;
        for (sms = 1; sms <= 148; sms += 49) {
          const int st = dwbnq_debug_pwconv_tiling(&p, (char *)fake + (p.n & 4), sms, shape);
          EXPECT(st == DWBNQ_OK ? (shape[0] % 32 == 0 && shape[0] <= 256 && shape[0] * shape[1] >= p.c_out && shape[3] >= 1 &&
                                   shape[4] >= 1 && shape[4] <= sms && shape[5] >= 2 && shape[5] <= 8 &&
                                   shape[6] * shape[0] <= 512 && shape[6] >= 1)
                                : IS_STATUS(st));
        }
      }
      p.n = 4;
    }
  EXPECT(dwbnq_debug_pwconv_tiling(NULL, fake, 148, shape) != DWBNQ_OK);
  EXPECT(dwbnq_debug_pwconv_tiling(&p, fake, 0, shape) != DWBNQ_OK);
  EXPECT(dwbnq_debug_pwconv_tiling(&p, fake, 148, NULL) != DWBNQ_OK);
  EXPECT(dwbnq_set_forced_pw_path(3) != DWBNQ_OK && dwbnq_set_forced_pw_path(-1) == DWBNQ_OK);
  EXPECT(dwbnq_set_pw_max_ctas(-1) != DWBNQ_OK && dwbnq_set_pw_max_ctas(0) == DWBNQ_OK);
  puts("pointwise");

  /* ---- communicator without NCCL handles ---- */
  EXPECT(dwbnq_comm_get_unique_id(NULL) != DWBNQ_OK);
  EXPECT(dwbnq_comm_create(NULL, 2, 0, 0, NULL) != DWBNQ_OK);
  EXPECT(dwbnq_comm_destroy(NULL) != DWBNQ_OK || 1);
  EXPECT(dwbnq_comm_set_deadline_ms(NULL, 10) != DWBNQ_OK);
  EXPECT(dwbnq_comm_allreduce_max_f32(NULL, (float *)fake, 4, NULL, 0) != DWBNQ_OK);
  puts("communicator");

  if (failures) {
    fprintf(stderr, "%d expectation(s) failed\n", failures);
    return 1;
  }
  puts("ok");
  return 0;
}
