// Host side of the fused dw-conv -> BN -> quantizer family: validation, the tile planner,
// TMA descriptor construction and kernel dispatch; plus the generic kernel instantiations.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "dwbnq_internal.h"

namespace dwbnq {

__device__ int g_device_flag = 0;

namespace {

// Test / tuning switches (include/dwbnq_debug.h) belong to the calling host thread: a thread
// that forces a family or overrides the planner never changes another thread's kernels.
constexpr int kPathUnset = -2;
thread_local int t_forced_path = kPathUnset;
// Planner overrides for tuning runs: planes per CTA, row blocks per tile (0 = auto).
thread_local int t_tune_p = 0, t_tune_rb = 0;

constexpr int kMaxDevices = 64;
int *g_flag_ptr[kMaxDevices] = {nullptr};
std::mutex g_flag_mutex;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      p = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int round_up(int a, int b) { return ceil_div(a, b) * b; }

constexpr int kGenericThreads = 256;
// Grid of the generic kernel: one thread per output, grid-stride beyond 64 CTAs per SM.
long long generic_blocks(long long total, int sms) {
  long long blocks = (total + kGenericThreads - 1) / kGenericThreads;
  const long long cap = (long long)sms * 64;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : blocks;
}

template <typename T>
cudaError_t launch_generic_t(int qm, const FusedArgs &a, long long total, int sms, cudaStream_t stream) {
  const int threads = kGenericThreads;
  const long long blocks = generic_blocks(total, sms);
  switch (qm) {
    case QM_NONE: fused_generic_kernel<T, QM_NONE><<<(unsigned)blocks, threads, 0, stream>>>(a, total); break;
    case QM_FPQ: fused_generic_kernel<T, QM_FPQ><<<(unsigned)blocks, threads, 0, stream>>>(a, total); break;
    case QM_POW2: fused_generic_kernel<T, QM_POW2><<<(unsigned)blocks, threads, 0, stream>>>(a, total); break;
    case QM_MM_APPLY: fused_generic_kernel<T, QM_MM_APPLY><<<(unsigned)blocks, threads, 0, stream>>>(a, total); break;
    case QM_MM_REDUCE: fused_generic_kernel<T, QM_MM_REDUCE><<<(unsigned)blocks, threads, 0, stream>>>(a, total); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace

int forced_path() {
  // the environment's default is read once (init-once state); a thread's own setting wins
  static const int env_default = [] {
    const char *e = std::getenv("DWBNQ_FORCE_PATH");
    if (e && *e) {
      if (!std::strcmp(e, "generic")) return (int)PATH_GENERIC;
      if (!std::strcmp(e, "coop")) return (int)PATH_COOP;
      if (!std::strcmp(e, "tma")) return (int)PATH_TMA;
      if (!std::strcmp(e, "raw")) return (int)PATH_RAW;
      if (!std::strcmp(e, "plane")) return (int)PATH_PLANE;
      if (!std::strcmp(e, "planegen")) return (int)PATH_PLANE_GEN;
    }
    return (int)PATH_AUTO;
  }();
  return t_forced_path == kPathUnset ? env_default : t_forced_path;
}
void set_forced_path(int p) { t_forced_path = p; }

int device_flag_ptr(int device, int **ptr) {
  if (device < 0 || device >= kMaxDevices) return fail(DWBNQ_ERR_INVALID_ARG, "device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_flag_mutex);
  if (!g_flag_ptr[device]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_device_flag);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(device flag)");
    g_flag_ptr[device] = static_cast<int *>(p);
  }
  *ptr = g_flag_ptr[device];
  return DWBNQ_OK;
}

int validate_conv(const dwbnq_conv_desc *d, int *ho, int *wo) {
  if (!d) return fail(DWBNQ_ERR_INVALID_ARG, "conv desc is null");
  if (d->dtype != DWBNQ_F32 && d->dtype != DWBNQ_F16)
    return fail(DWBNQ_ERR_INVALID_ARG, "dtype %d is neither DWBNQ_F32 nor DWBNQ_F16", d->dtype);
  if (d->n < 0 || d->c <= 0 || d->h <= 0 || d->w <= 0)
    return fail(DWBNQ_ERR_INVALID_ARG, "input shape [%lld,%d,%d,%d] is not positive", (long long)d->n, d->c, d->h, d->w);
  if (d->kh <= 0 || d->kw <= 0 || d->stride_h <= 0 || d->stride_w <= 0 || d->dil_h <= 0 || d->dil_w <= 0)
    return fail(DWBNQ_ERR_INVALID_ARG, "kernel / stride / dilation must be positive");
  if (d->pad_h < 0 || d->pad_w < 0) return fail(DWBNQ_ERR_INVALID_ARG, "negative padding");
  if (d->multiplier <= 0) return fail(DWBNQ_ERR_INVALID_ARG, "multiplier must be positive");
  const long long eh = (long long)d->h + 2LL * d->pad_h - (long long)d->dil_h * (d->kh - 1) - 1;
  const long long ew = (long long)d->w + 2LL * d->pad_w - (long long)d->dil_w * (d->kw - 1) - 1;
  if (eh < 0 || ew < 0)
    return fail(DWBNQ_ERR_INVALID_ARG, "kernel %dx%d (dilation %d,%d) does not fit input %dx%d with pad %d,%d",
                d->kh, d->kw, d->dil_h, d->dil_w, d->h, d->w, d->pad_h, d->pad_w);
  // Limit of the reference implementation: output-channels x filter-size <= 65536.
  if ((long long)d->c * d->multiplier * d->kh * d->kw > 65536)
    return fail(DWBNQ_ERR_UNSUPPORTED,
                "GPU implementation limit reached: output-channels x filter-size can not be more than 65536");
  // The kernels index one plane (and one padded plane) with 32-bit integers.
  const long long oh = eh / d->stride_h + 1, ow = ew / d->stride_w + 1;
  const long long ph = (long long)d->h + 2LL * d->pad_h, pw = (long long)d->w + 2LL * d->pad_w;
  if (ph > INT32_MAX || pw > INT32_MAX || ph * pw > INT32_MAX || oh * ow > INT32_MAX)
    return fail(DWBNQ_ERR_UNSUPPORTED, "padded plane %lldx%lld / output plane %lldx%lld exceeds 2^31-1 elements", ph, pw,
                oh, ow);
  if (ho) *ho = (int)oh;
  if (wo) *wo = (int)ow;
  return DWBNQ_OK;
}

// Streaming multiprocessors of `device` (-1: the current device), asked of the driver once
// per device; grids that are capped "per SM" are sized from this, not from a literal.
int sm_count(int device) {
  static std::atomic<int> cached[kMaxDevices];
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) {
    (void)cudaGetLastError();
    device = 0;
  }
  const bool slot = device >= 0 && device < kMaxDevices;
  int n = slot ? cached[device].load(std::memory_order_relaxed) : 0;
  if (n <= 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      return 148;  // no usable device: the launch that follows reports the real error
    }
    if (slot) cached[device].store(n, std::memory_order_relaxed);
  }
  return n;
}

namespace {

long long gcd_ll(long long a, long long b) { return b ? gcd_ll(b, a % b) : a; }

}  // namespace

namespace {
int make_plan_tiled(const dwbnq_conv_desc &d, const void *x, const void *y, Plan *plan);
}

int make_plan(const dwbnq_conv_desc &d, const void *x, const void *y, Plan *plan) {
  int st = make_plan_tiled(d, x, y, plan);
  if (st != DWBNQ_OK || plan->path != PATH_GENERIC) return st;
  int Ho = 0, Wo = 0;
  validate_conv(&d, &Ho, &Wo);
  plan->threads = kGenericThreads;
  plan->ctas = generic_blocks(d.n * d.c * d.multiplier * Ho * Wo, sm_count(-1));
  plan->smem = 0;
  return DWBNQ_OK;
}

namespace {

int make_plan_tiled(const dwbnq_conv_desc &d, const void *x, const void *y, Plan *plan) {
  int Ho, Wo;
  int st = validate_conv(&d, &Ho, &Wo);
  if (st != DWBNQ_OK) return st;
  std::memset(plan, 0, sizeof(*plan));
  plan->path = PATH_GENERIC;
  const int forced = forced_path();
  const int B = d.dtype == DWBNQ_F32 ? 4 : 2;
  const int S = 16 / B;  // elements per 16-byte vector = outputs per thread and patch row
  const int K = d.kh;
  const int s = d.stride_h;
  const bool tileable = d.kh == d.kw && (K == 3 || K == 5) && d.stride_h == d.stride_w &&
                        (s == 1 || s == 2) && d.pad_h == K / 2 && d.pad_w == K / 2 &&
                        d.dil_h == 1 && d.dil_w == 1 && d.multiplier == 1 && d.n > 0;
  if (!tileable || forced == PATH_GENERIC) return DWBNQ_OK;

  const int R = kRowsPerPatch;
  const int pad = K / 2;
  const long long n_planes = d.n * d.c;
  if (n_planes > 0x7fffffffLL) return DWBNQ_OK;

  // ---- small planes (7x7, 14x14, 28x28): one warp per CTA, whole planes -------------------
  const PlaneGeom pg = plane_geom(K, d.h, d.w, s);
  if (pg.tpp > 0 && (forced == PATH_AUTO || forced == PATH_PLANE)) {
    TileCfg &c = plan->cfg;
    c.P = (K == 3 && s == 1 && d.w == 7) ? 64 : 32 / pg.tpp;  // 7x7: two planes per thread
    c.R = kPlaneRows;
    c.n_rb = pg.nrb;
    c.n_strips = pg.ncb;
    c.n_row_tiles = pg.bands;
    c.TH = Ho / pg.bands;
    c.TR = d.h;
    c.WS = d.w;
    c.tile_elems = d.h * d.w;
    const bool al = (reinterpret_cast<uintptr_t>(x) % 16) == 0 && (reinterpret_cast<uintptr_t>(y) % 16) == 0;
    c.vec_fill = al ? 1 : 0;
    c.vec_store = al ? 1 : 0;
    const long long nt = (n_planes + c.P - 1) / c.P * pg.bands;
    if (nt > 0x7fffffffLL) return DWBNQ_OK;
    c.n_tiles = (int)nt;
    plan->path = PATH_PLANE;
    plan->threads = 32;
    plan->smem = plane_launch_smem(K, d.w, s, d.dtype == DWBNQ_F32 ? 4 : 2);
    plan->ctas = c.n_tiles;
    return DWBNQ_OK;
  }
  if (forced == PATH_PLANE) return DWBNQ_OK;  // no instantiation for this shape: generic kernel

  // ---- any other plane of even width, 3x3 stride 1: the general-geometry plane kernel -------
  if (K == 3 && s == 1 && (forced == PATH_AUTO || forced == PATH_PLANE_GEN)) {
    const bool al = (reinterpret_cast<uintptr_t>(x) % 16) == 0 && (reinterpret_cast<uintptr_t>(y) % 16) == 0;
    float util = 0.0f;
    const PlaneGenCfg g = plane_gen_geometry(d.h, d.w, n_planes, d.dtype == DWBNQ_F32 ? 4 : 2, al, &util);
    // Measured on B200 against the TMA tile family (planes 6..96 wide): the plane scheme wins on
    // small planes (up to 32 x 32), whenever the row pitch rules out the TMA tile, and with the
    // 7 x 14 blocks when they tile the plane well; on mid-size planes that only the 8 x 8
    // blocks tile, the TMA tile is 10-20 % faster.
    const bool tma_possible = (reinterpret_cast<uintptr_t>(x) % 16) == 0 &&
                              ((long long)d.w * (d.dtype == DWBNQ_F32 ? 4 : 2)) % 16 == 0 && encode_tiled_fn() != nullptr;
    const bool take = forced == PATH_PLANE_GEN || !tma_possible || (long long)d.h * d.w <= 1024 ||
                      (util >= 0.8f && g.wb == 14);
    if (g.n_tiles > 0 && take) {
      TileCfg &c = plan->cfg;
      c.P = g.P;
      c.R = g.r;
      c.n_rb = g.brb;
      c.n_strips = g.ncb;
      c.n_row_tiles = g.bands;
      c.TH = g.brb * g.r;
      c.TR = d.h;
      c.WS = d.w;
      c.tile_elems = d.h * d.w;
      c.vec_fill = c.vec_store = al ? 1 : 0;
      c.n_tiles = g.n_tiles;
      plan->gen = g;
      plan->path = PATH_PLANE_GEN;
      plan->threads = 32;
      plan->smem = plane_gen_smem_bytes(g, d.dtype == DWBNQ_F32 ? 4 : 2);
      plan->ctas = g.n_tiles;
      return DWBNQ_OK;
    }
  }
  if (forced == PATH_PLANE_GEN) return DWBNQ_OK;
  const int n_strips = ceil_div(Wo, S);
  const int n_rb_total = ceil_div(Ho, R);
  // One tile per CTA and several CTAs per SM: the budget keeps four tiles (plus records)
  // inside the 227 KB of shared memory of an SM.
  const long long stage_budget = 48 * 1024;
  const int max_threads = 256;
  const bool x_al = (reinterpret_cast<uintptr_t>(x) % 16) == 0;
  const bool y_al = (reinterpret_cast<uintptr_t>(y) % 16) == 0;
  const long long plane_bytes = (long long)d.h * d.w * B;

  // ---- which family -----------------------------------------------------------------------
  const bool tma_ok = x_al && ((long long)d.w * B) % 16 == 0 && encode_tiled_fn() != nullptr;
  const int raw_lead = round_up(pad * d.w + pad + 1, S);
  const int raw_trail = round_up(n_strips * S * s + K, S) + S;
  const bool raw_ok = (raw_lead + raw_trail) * (long long)B + plane_bytes <= stage_budget &&
                      plane_bytes * 2 < 0x7fffffffLL;
  int path;
  if (forced == PATH_COOP) path = PATH_COOP;
  else if (forced == PATH_RAW) path = raw_ok ? PATH_RAW : PATH_COOP;
  else path = tma_ok ? PATH_TMA : (raw_ok ? PATH_RAW : PATH_COOP);

  TileCfg &c = plan->cfg;
  c.n_strips = n_strips;
  c.R = R;
  c.vec_store = (y_al && Wo % S == 0) ? 1 : 0;
  int P = 1;
  if (path == PATH_RAW) {
    // Whole planes, verbatim. P is a multiple of `pal` so every full tile starts on a
    // 16-byte boundary and spans a multiple of 16 bytes (what the bulk copy engine needs).
    const int ipp = n_strips * n_rb_total;
    const long long pal = 16 / gcd_ll(plane_bytes, 16);
    const long long fit = (stage_budget - (raw_lead + raw_trail) * (long long)B) / plane_bytes;
    // small planes: many small CTAs hide the per-CTA copy / record latency better than few
    // large ones (measured on B200): about 64 threads each
    long long want = std::max(1, (ipp <= 64 ? 64 : max_threads) / ipp);
    if (t_tune_p > 0) want = t_tune_p;
    want = std::min(want, fit);
    long long Pl = want / pal * pal;
    if (Pl < pal) Pl = pal <= fit ? pal : want;  // cannot align: the copies fall back to threads
    if (Pl > n_planes) Pl = n_planes;
    if (Pl < 1) Pl = 1;
    P = (int)Pl;
    c.n_row_tiles = 1;
    c.n_rb = n_rb_total;
    c.TH = n_rb_total * R;
    c.WS = d.w;
    c.TR = d.h;
    c.box_rows = d.h;
    c.n_boxes = 1;
    c.tile_elems = d.h * d.w;
    c.raw_lead = raw_lead;
    c.stage_elems = round_up((raw_lead + P * c.tile_elems + raw_trail) * B, 128) / B;
    c.vec_fill = (x_al && (P * plane_bytes) % 16 == 0) ? 1 : 0;
  } else {
    const int WS = round_up(S + (n_strips * S - 1) * s + K - pad, S);
    if (WS > 256) return DWBNQ_OK;  // wider than one TMA box: generic kernel
    // Row blocks per tile: aim at one patch per thread, split the plane evenly, and keep one
    // plane's tile inside the budget.
    int rb_per_tile = std::max(1, std::min(n_rb_total, max_threads / n_strips));
    if (t_tune_rb > 0) rb_per_tile = std::min(t_tune_rb, n_rb_total);
    int n_row_tiles, TH, TR, n_boxes, box_rows, tile_elems;
    for (;;) {
      n_row_tiles = ceil_div(n_rb_total, rb_per_tile);
      rb_per_tile = ceil_div(n_rb_total, n_row_tiles);
      TH = rb_per_tile * R;
      TR = (TH - 1) * s + K;
      // A TMA box has at most 256 rows and its shared-memory destination must be 128-byte
      // aligned: with several boxes per plane the rows per box are a multiple of 8.
      n_boxes = ceil_div(TR, 256);
      box_rows = n_boxes == 1 ? TR : round_up(ceil_div(TR, n_boxes), 8);
      tile_elems = round_up(box_rows * n_boxes * WS * B, 128) / B;
      if ((long long)tile_elems * B <= stage_budget || rb_per_tile == 1) break;
      rb_per_tile = std::max(1, rb_per_tile - 1);
    }
    const long long tile_bytes = (long long)tile_elems * B;
    if (tile_bytes > 96 * 1024) return DWBNQ_OK;
    const int ipp = n_strips * rb_per_tile;
    // whole small planes: about 64 threads per CTA (see above); otherwise fill the CTA
    P = std::max(1, ((n_row_tiles == 1 && ipp <= 64) ? 64 : max_threads) / ipp);
    while (P > 1 && (long long)P * tile_bytes > stage_budget) --P;
    if (t_tune_p > 0) P = t_tune_p;
    if (P > n_planes) P = (int)n_planes;
    c.n_row_tiles = n_row_tiles;
    c.n_rb = rb_per_tile;
    c.TH = TH;
    c.WS = WS;
    c.TR = TR;
    c.box_rows = box_rows;
    c.n_boxes = n_boxes;
    c.tile_elems = tile_elems;
    c.raw_lead = 0;
    c.stage_elems = P * tile_elems;
    c.vec_fill = (x_al && d.w % S == 0) ? 1 : 0;
  }
  // one patch per thread: block = (strips, planes, row blocks)
  if (n_strips * c.n_rb > max_threads || c.n_rb > 64) return DWBNQ_OK;
  while (P > 1 && P * n_strips * c.n_rb > max_threads) {
    --P;
    if (path == PATH_RAW) {
      c.stage_elems = round_up((raw_lead + P * c.tile_elems + raw_trail) * B, 128) / B;
      c.vec_fill = (x_al && (P * plane_bytes) % 16 == 0) ? 1 : 0;
    } else {
      c.stage_elems = P * c.tile_elems;
    }
  }
  c.P = P;
  const long long n_tiles = ((n_planes + P - 1) / P) * c.n_row_tiles;
  if (n_tiles > 0x7fffffffLL) return DWBNQ_OK;
  c.n_tiles = (int)n_tiles;
  const size_t smem = tiled_smem_bytes(P, c.stage_elems, B, K);
  if (smem > 200 * 1024) return DWBNQ_OK;
  const int threads = P * n_strips * c.n_rb;  // one patch per thread
  plan->threads = threads;
  plan->smem = smem;
  plan->path = path;
  plan->ctas = c.n_tiles;
  return DWBNQ_OK;
}

}  // namespace

int launch_fused(const dwbnq_conv_desc &d, FusedArgs &a, int qm, int device, cudaStream_t stream) {
  Plan plan;
  int st = make_plan(d, a.x, a.y, &plan);
  if (st != DWBNQ_OK) return st;
  if (d.n == 0) return DWBNQ_OK;
  st = device_flag_ptr(device, &a.flag);
  if (st != DWBNQ_OK) return st;
  const long long total = d.n * (long long)a.OC * a.Ho * a.Wo;
  cudaError_t e;
  if (a.code8) {
    // 8-bit storage: the plane kernels that carry a code path, else the generic kernel
    int pq = qm;
    if (pq == QM_FPQ && a.has_bn && a.q.fpq_fast && !(a.q.fpq_min < 0.0f)) pq = QM_FPQ_LEAN;
    if (!(plan.path == PATH_PLANE && plane_has_code8(d.dtype, d.kh, d.w, d.stride_h, pq))) plan.path = PATH_GENERIC;
  }
  if (plan.path == PATH_GENERIC) {
    const int sms = sm_count(device);
    e = d.dtype == DWBNQ_F32 ? launch_generic_t<float>(qm, a, total, sms, stream)
                             : launch_generic_t<__half>(qm, a, total, sms, stream);
    if (e != cudaSuccess) return fail_cuda(e, "fused_generic_kernel launch");
    return DWBNQ_OK;
  }
  if (plan.path == PATH_PLANE_GEN) {
    if (qm == QM_FPQ && a.has_bn && a.q.fpq_fast && !(a.q.fpq_min < 0.0f)) qm = QM_FPQ_LEAN;
    e = launch_plane_gen(d.dtype, qm, a, plan.gen, stream);
    if (e != cudaSuccess) return fail_cuda(e, "fused_plane_gen_kernel launch");
    return DWBNQ_OK;
  }
  if (plan.path == PATH_PLANE) {
    // BN + unsigned power-of-two FixedPointQuantize: the instantiation without mode tests
    if (qm == QM_FPQ && a.has_bn && a.q.fpq_fast && !(a.q.fpq_min < 0.0f)) qm = QM_FPQ_LEAN;
    PlaneCfg pc;
    pc.P = plan.cfg.P;
    pc.n_tiles = plan.cfg.n_tiles;
    pc.bulk = plan.cfg.vec_fill;
    e = launch_plane(d.dtype, d.kh, d.w, d.stride_h, qm, a, pc, stream);
    if (e != cudaSuccess) return fail_cuda(e, "fused_plane_kernel launch");
    return DWBNQ_OK;
  }
  const int mode = plan.path == PATH_TMA ? TM_TMA : plan.path == PATH_RAW ? TM_RAW : TM_COOP;
  // The common FixedPointQuantize case gets the kernel compiled without per-row tests.
  // (every patch row of every tile must lie inside the image: the tiles cover Ho exactly)
  if (qm == QM_FPQ && a.has_bn && a.q.fpq_fast && !(a.q.fpq_min < 0.0f) && plan.cfg.vec_store &&
      plan.cfg.n_row_tiles * plan.cfg.n_rb * kRowsPerPatch == a.Ho)
    qm = QM_FPQ_LEAN;
  CUtensorMap tmap;
  std::memset(&tmap, 0, sizeof(tmap));
  if (mode == TM_TMA) {
    const int B = d.dtype == DWBNQ_F32 ? 4 : 2;
    const cuuint64_t gdim[3] = {(cuuint64_t)d.w, (cuuint64_t)d.h, (cuuint64_t)(d.n * d.c)};
    const cuuint64_t gstride[2] = {(cuuint64_t)d.w * B, (cuuint64_t)d.w * d.h * B};
    const cuuint32_t box[3] = {(cuuint32_t)plan.cfg.WS, (cuuint32_t)plan.cfg.box_rows, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult r = encode_tiled_fn()(
        &tmap, d.dtype == DWBNQ_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
        3, const_cast<void *>(a.x), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DWBNQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  }
  const bool f32 = d.dtype == DWBNQ_F32;
  const int ctas = plan.cfg.n_tiles;  // one CTA per tile
  if (f32) e = d.kh == 3 ? launch_tiled<float, 3>(d.stride_h, qm, mode, tmap, a, plan.cfg, ctas, plan.threads, plan.smem, stream)
                         : launch_tiled<float, 5>(d.stride_h, qm, mode, tmap, a, plan.cfg, ctas, plan.threads, plan.smem, stream);
  else e = d.kh == 3 ? launch_tiled<__half, 3>(d.stride_h, qm, mode, tmap, a, plan.cfg, ctas, plan.threads, plan.smem, stream)
                     : launch_tiled<__half, 5>(d.stride_h, qm, mode, tmap, a, plan.cfg, ctas, plan.threads, plan.smem, stream);
  if (e != cudaSuccess) return fail_cuda(e, "fused_tiled_kernel launch");
  return DWBNQ_OK;
}

}  // namespace dwbnq

// One warp, one barrier nobody completes: the bounded wait runs out after `limit_ns` and the
// kernel records it, exactly like a copy-engine kernel whose transfer never landed.
namespace dwbnq {
__global__ void expire_wait_kernel(int *flag, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  if (!mbar_wait_bounded(&bar, 0, limit_ns)) {
    if (flag) atomicExch(flag, 1);
    return;
  }
}
}  // namespace dwbnq

extern "C" int dwbnq_set_tuning(int planes_per_cta, int row_blocks_per_tile, int threads, int rows_per_patch) {
  (void)threads;
  (void)rows_per_patch;
  dwbnq::t_tune_p = planes_per_cta;
  dwbnq::t_tune_rb = row_blocks_per_tile;
  return DWBNQ_OK;
}

extern "C" int dwbnq_debug_expire_wait(unsigned int limit_us, int device, void *stream) {
  using namespace dwbnq;
  clear_error();
  int dev;
  int st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  int *flag = nullptr;
  st = device_flag_ptr(dev, &flag);
  if (st != DWBNQ_OK) return st;
  expire_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flag, 1000ull * limit_us);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "expire_wait_kernel launch");
  return DWBNQ_OK;
}
