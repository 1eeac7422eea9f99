/* A plain C99 client of the dwbnq C ABI (no Python, no torch): reads a small layer from a
 * binary file, runs dw-conv -> BN -> FixedPointQuantize through dwbnq_fused_fwd on device
 * memory it allocates with the CUDA runtime, and writes the result to another file.
 * tests/test_cabi_client.py builds it with gcc, runs it on the GPU and compares the output
 * with the CPU oracle bit for bit.
 *
 * Input file: int32 header {n, c, h, w, k, stride, pad, sign, bits} then float32 delta, eps,
 * then x[n*c*h*w], w[c*k*k], b[c], beta[c], gamma[c], mean[c], var[c] as float32. */
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>

#include "dwbnq.h"

static void *to_device(const float *host, size_t count) {
  void *d = NULL;
  if (cudaMalloc(&d, count * sizeof(float)) != cudaSuccess) return NULL;
  if (cudaMemcpy(d, host, count * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) return NULL;
  return d;
}

int main(int argc, char **argv) {
  int hdr[9];
  float fl[2];
  FILE *f;
  size_t nx, nw, nc, ny;
  float *buf, *y;
  void *dx, *dw, *db, *dbeta, *dgamma, *dmean, *dvar, *dy;
  dwbnq_conv_desc d;
  dwbnq_quant_desc q;
  int ho, wo, st;
  if (argc != 3) {
    fprintf(stderr, "usage: %s <layer.bin> <out.bin>\n", argv[0]);
    return 2;
  }
  f = fopen(argv[1], "rb");
  if (!f || fread(hdr, sizeof(int), 9, f) != 9 || fread(fl, sizeof(float), 2, f) != 2) return 3;
  nx = (size_t)hdr[0] * hdr[1] * hdr[2] * hdr[3];
  nw = (size_t)hdr[1] * hdr[4] * hdr[4];
  nc = (size_t)hdr[1];
  buf = (float *)malloc((nx + nw + 5 * nc) * sizeof(float));
  if (!buf || fread(buf, sizeof(float), nx + nw + 5 * nc, f) != nx + nw + 5 * nc) return 4;
  fclose(f);

  d.dtype = DWBNQ_F32;
  d.c = hdr[1];
  d.n = hdr[0];
  d.h = hdr[2];
  d.w = hdr[3];
  d.kh = d.kw = hdr[4];
  d.stride_h = d.stride_w = hdr[5];
  d.pad_h = d.pad_w = hdr[6];
  d.dil_h = d.dil_w = 1;
  d.multiplier = 1;
  if (dwbnq_conv_out_shape(&d, &ho, &wo) != DWBNQ_OK) {
    fprintf(stderr, "%s\n", dwbnq_last_error_string());
    return 5;
  }
  ny = (size_t)d.n * d.c * ho * wo;

  dx = to_device(buf, nx);
  dw = to_device(buf + nx, nw);
  db = to_device(buf + nx + nw, nc);
  dbeta = to_device(buf + nx + nw + nc, nc);
  dgamma = to_device(buf + nx + nw + 2 * nc, nc);
  dmean = to_device(buf + nx + nw + 3 * nc, nc);
  dvar = to_device(buf + nx + nw + 4 * nc, nc);
  if (!dx || !dw || !db || !dbeta || !dgamma || !dmean || !dvar || cudaMalloc(&dy, ny * sizeof(float)) != cudaSuccess)
    return 6;

  q.kind = DWBNQ_Q_FPQ;
  q.sign = hdr[7];
  q.n = hdr[8];
  q.delta = fl[0];
  q.with_zero = 0;
  q.m = 0;
  q.decay = 0.0f;
  q.eps = 0.0f;
  q.x_min_max = 0;
  q.ema = 0;
  st = dwbnq_fused_fwd(&d, fl[1], &q, dx, dw, db, dbeta, dgamma, dmean, dvar, NULL, dy, NULL, NULL, 0, NULL);
  if (st != DWBNQ_OK) {
    fprintf(stderr, "dwbnq_fused_fwd: %d %s\n", st, dwbnq_last_error_string());
    return 7;
  }
  if (cudaDeviceSynchronize() != cudaSuccess || dwbnq_check_device_flag(0) != DWBNQ_OK) return 8;
  y = (float *)malloc(ny * sizeof(float));
  if (!y || cudaMemcpy(y, dy, ny * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) return 9;
  f = fopen(argv[2], "wb");
  if (!f || fwrite(y, sizeof(float), ny, f) != ny) return 10;
  fclose(f);
  printf("%d %d %d %d\n", (int)d.n, d.c, ho, wo);
  return 0;
}
