// MinMaxQuantize forward for callers that cannot hand over scratch memory.
//
// dwbnq_minmaxq_fwd needs a small device workspace (per-channel min / max slots and the
// derived ranges) and expects the caller to provide it. Some callers have no way to do that
// from where they call: a function object that only receives its input and output tensors
// from a framework whose allocator has already claimed the whole device, an inference loop
// that must not touch the allocator once it is running, a plugin entry that is handed raw
// pointers and nothing else. For them this file keeps the workspace in a fixed, file-scope
// device array that exists on every GPU the library is loaded on, from load until exit.
#include <mutex>

#include "dwbnq_internal.h"

namespace dwbnq {

// 7 words per channel (see MmWorkspace), DWBNQ_STATIC_MAX_CHANNELS channels: 112 KiB per GPU.
static __device__ __align__(256) unsigned int g_mm_static_ws[7 * DWBNQ_STATIC_MAX_CHANNELS];

namespace {

constexpr int kMaxDevices = 64;
void *g_ws_ptr[kMaxDevices] = {nullptr};
std::mutex g_ws_mutex;

// In host code `g_mm_static_ws` is only a handle for the symbol, not an address a kernel
// could use: the device address is looked up once per device, with that device current.
int static_workspace(int device, void **ptr) {
  if (device < 0 || device >= kMaxDevices) return fail(DWBNQ_ERR_INVALID_ARG, "device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  if (!g_ws_ptr[device]) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_mm_static_ws);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(static MinMaxQuantize workspace)");
    g_ws_ptr[device] = p;
  }
  *ptr = g_ws_ptr[device];
  return DWBNQ_OK;
}

}  // namespace
}  // namespace dwbnq

using namespace dwbnq;

extern "C" int dwbnq_minmaxq_fwd_static(int dtype, int64_t size0, int32_t channels, int64_t size2,
                                        const dwbnq_quant_desc *q, const void *x,
                                        const dwbnq_minmax_ptrs *mm, void *y, int device, void *stream) {
  clear_error();
  if (dtype != DWBNQ_F32 && dtype != DWBNQ_F16)
    return fail(DWBNQ_ERR_INVALID_ARG, "dtype %d is neither DWBNQ_F32 nor DWBNQ_F16", dtype);
  if (size0 < 0 || channels <= 0 || size2 < 0)
    return fail(DWBNQ_ERR_INVALID_ARG, "view [%lld,%d,%lld] is not a valid shape", (long long)size0, channels,
                (long long)size2);
  if (channels > DWBNQ_STATIC_MAX_CHANNELS)
    return fail(DWBNQ_ERR_UNSUPPORTED,
                "dwbnq_minmaxq_fwd_static handles at most %d channels (got %d): use dwbnq_minmaxq_fwd with a "
                "caller-provided workspace",
                DWBNQ_STATIC_MAX_CHANNELS, channels);
  if (!q) return fail(DWBNQ_ERR_INVALID_ARG, "quantizer desc is null");
  if (!x || !y) return fail(DWBNQ_ERR_INVALID_ARG, "x and y must not be null");
  if (!mm || !mm->qr_min || !mm->qr_max || !mm->ql_min || !mm->ql_max)
    return fail(DWBNQ_ERR_INVALID_ARG, "MinMaxQuantize needs qr_min, qr_max, ql_min and ql_max");
  if (q->ema && !(q->decay >= 0.0f && q->decay <= 1.0f))
    return fail(DWBNQ_ERR_INVALID_ARG, "decay %g is not in [0, 1]", q->decay);
  int dev;
  int st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  void *wsp = nullptr;
  st = static_workspace(dev, &wsp);
  if (st != DWBNQ_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const MmWorkspace ws = mm_workspace(wsp, channels);
  // The array keeps whatever the previous call left: the min / max slots are re-armed here,
  // every other word is written before it is read.
  if (q->x_min_max) {
    st = launch_mm_init(ws, channels, s);
    if (st != DWBNQ_OK) return st;
    st = launch_mm_reduce(dtype, size0, channels, size2, x, ws, s);
    if (st != DWBNQ_OK) return st;
  }
  st = launch_mm_ranges(dtype, channels, *q, *mm, ws, /*from_packed=*/0, s);
  if (st != DWBNQ_OK) return st;
  return launch_mm_apply(dtype, size0, channels, size2, x, y, ws, s);
}
