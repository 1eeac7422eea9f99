// Device copy of the Pow2Quantize threshold table: a file-scope array per device, filled
// once per device from the host table (no allocation).
#include <mutex>

#include "dwbnq_internal.h"

namespace dwbnq {

__device__ uint32_t g_pow2_table_dev[277];

namespace {
constexpr int kMaxDevices = 64;
const uint32_t *g_ptr[kMaxDevices] = {nullptr};
std::mutex g_mutex;
}  // namespace

int pow2_table_device(int device, const uint32_t **ptr) {
  if (device < 0 || device >= kMaxDevices) return fail(DWBNQ_ERR_INVALID_ARG, "device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_ptr[device]) {
    // Synchronous copy: complete before any kernel launched after this call can start.
    cudaError_t e = cudaMemcpyToSymbol(g_pow2_table_dev, pow2_table_host(), 277 * sizeof(uint32_t));
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemcpyToSymbol(pow2 threshold table)");
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_pow2_table_dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(pow2 threshold table)");
    g_ptr[device] = static_cast<const uint32_t *>(p);
  }
  *ptr = g_ptr[device];
  return DWBNQ_OK;
}

}  // namespace dwbnq
