// The one collective of the path: an all-reduce(max) of the packed per-channel vector
// [max_c..., -min_c...] when MinMaxQuantize reduces over a batch that is sharded across
// GPUs. NCCL is resolved with dlopen at first use so the library loads (and every other
// entry point works) where NCCL is absent.
#include <dlfcn.h>

#include <cstdlib>

#include <chrono>
#include <cstring>
#include <mutex>
#include <thread>

#include "dwbnq_internal.h"

namespace dwbnq {

namespace {

// Minimal mirror of the stable NCCL C ABI (nccl.h): opaque communicator, 128-byte id,
// result code 0 = success, 7 = in progress; ncclFloat32 = 7; ncclMax = 2.
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
constexpr int kNcclSuccess = 0;
constexpr int kNcclInProgress = 7;
constexpr int kNcclFloat32 = 7;
constexpr int kNcclMax = 2;

struct NcclApi {
  void *handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId *) = nullptr;
  int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int *) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  bool ok = false;
};

NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
  // DWBNQ_NCCL_LIB names the library to load instead of the default sonames (a site build
  // of NCCL, or the stand-in the tests use to exercise the error and deadline paths).
  const char *override_path = std::getenv("DWBNQ_NCCL_LIB");
  const char *names[] = {override_path && *override_path ? override_path : "libnccl.so.2", "libnccl.so.2",
                         "libnccl.so"};
  for (const char *n : names) {
    g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.handle) break;
  }
  if (!g_nccl.handle) return;
  void *h = g_nccl.handle;
  g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
  g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
  g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
  g_nccl.CommAbort = reinterpret_cast<decltype(g_nccl.CommAbort)>(dlsym(h, "ncclCommAbort"));
  g_nccl.CommGetAsyncError = reinterpret_cast<decltype(g_nccl.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
  g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(dlsym(h, "ncclAllReduce"));
  g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
  g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.CommAbort &&
              g_nccl.CommGetAsyncError && g_nccl.AllReduce && g_nccl.GetErrorString;
}

int need_nccl() {
  std::call_once(g_nccl_once, load_nccl);
  if (!g_nccl.ok) return fail(DWBNQ_ERR_NCCL, "NCCL could not be loaded (dlopen libnccl.so.2): %s",
                              g_nccl.handle ? "missing symbols" : "library not found");
  return DWBNQ_OK;
}

int fail_nccl(int r, const char *what) {
  return fail(DWBNQ_ERR_NCCL, "%s failed: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?");
}

struct Comm {
  ncclComm_t nccl = nullptr;
  int nranks = 0, rank = 0, device = 0;
  int deadline_ms = 0;  // for the collectives the MINMAX entry points issue (0 = enqueue only)
  bool aborted = false;
};

int env_deadline_ms() {
  const char *e = std::getenv("DWBNQ_COMM_DEADLINE_MS");
  if (!e || !*e) return 0;
  const long v = std::strtol(e, nullptr, 10);
  return v > 0 && v < 0x7fffffffL ? (int)v : 0;
}

}  // namespace

int comm_deadline_ms(void *comm) { return comm ? static_cast<Comm *>(comm)->deadline_ms : 0; }

int comm_allreduce_max(void *comm, float *buf, long long count, cudaStream_t stream, int timeout_ms) {
  if (!comm) return fail(DWBNQ_ERR_INVALID_ARG, "communicator is null");
  Comm *c = static_cast<Comm *>(comm);
  if (c->aborted) return fail(DWBNQ_ERR_NCCL, "communicator was aborted after a time-out");
  if (!buf || count <= 0) return fail(DWBNQ_ERR_INVALID_ARG, "all-reduce buffer is null or empty");
  int st = need_nccl();
  if (st != DWBNQ_OK) return st;
  int r = g_nccl.AllReduce(buf, buf, (size_t)count, kNcclFloat32, kNcclMax, c->nccl, stream);
  if (r != kNcclSuccess) return fail_nccl(r, "ncclAllReduce(max)");
  if (timeout_ms <= 0) return DWBNQ_OK;
  // Deadline: poll an event recorded behind the collective and the communicator's
  // asynchronous error state; abort the communicator when the deadline passes.
  cudaEvent_t ev;
  cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  if (e != cudaSuccess) return fail_cuda(e, "cudaEventCreate");
  e = cudaEventRecord(ev, stream);
  if (e != cudaSuccess) {
    cudaEventDestroy(ev);
    return fail_cuda(e, "cudaEventRecord");
  }
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  int result = DWBNQ_OK;
  for (;;) {
    e = cudaEventQuery(ev);
    if (e == cudaSuccess) break;
    if (e != cudaErrorNotReady) {
      result = fail_cuda(e, "cudaEventQuery behind ncclAllReduce");
      break;
    }
    int async = kNcclSuccess;
    r = g_nccl.CommGetAsyncError(c->nccl, &async);
    if (r != kNcclSuccess || (async != kNcclSuccess && async != kNcclInProgress)) {
      result = fail_nccl(r != kNcclSuccess ? r : async, "ncclAllReduce(max) (asynchronous error)");
      break;
    }
    if (std::chrono::steady_clock::now() > deadline) {
      g_nccl.CommAbort(c->nccl);
      c->aborted = true;
      c->nccl = nullptr;
      result = fail(DWBNQ_ERR_TIMEOUT, "min/max all-reduce did not complete within %d ms; communicator aborted", timeout_ms);
      break;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  cudaEventDestroy(ev);
  return result;
}

}  // namespace dwbnq

using namespace dwbnq;

extern "C" int dwbnq_comm_get_unique_id(void *id128) {
  clear_error();
  if (!id128) return fail(DWBNQ_ERR_INVALID_ARG, "id buffer is null");
  int st = need_nccl();
  if (st != DWBNQ_OK) return st;
  ncclUniqueId id;
  int r = g_nccl.GetUniqueId(&id);
  if (r != kNcclSuccess) return fail_nccl(r, "ncclGetUniqueId");
  std::memcpy(id128, &id, sizeof(id));
  return DWBNQ_OK;
}

extern "C" int dwbnq_comm_create(const void *id128, int nranks, int rank, int device, void **comm) {
  clear_error();
  if (!id128 || !comm) return fail(DWBNQ_ERR_INVALID_ARG, "id or output pointer is null");
  if (nranks <= 0 || rank < 0 || rank >= nranks)
    return fail(DWBNQ_ERR_INVALID_ARG, "rank %d is not in [0, %d)", rank, nranks);
  int st = need_nccl();
  if (st != DWBNQ_OK) return st;
  int dev;
  st = enter_device(device, &dev);
  if (st != DWBNQ_OK) return st;
  ncclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  Comm *c = new Comm();
  c->nranks = nranks;
  c->rank = rank;
  c->device = dev;
  c->deadline_ms = env_deadline_ms();
  int r = g_nccl.CommInitRank(&c->nccl, nranks, id, rank);
  if (r != kNcclSuccess) {
    delete c;
    return fail_nccl(r, "ncclCommInitRank");
  }
  *comm = c;
  return DWBNQ_OK;
}

extern "C" int dwbnq_comm_set_deadline_ms(void *comm, int ms) {
  clear_error();
  if (!comm) return fail(DWBNQ_ERR_INVALID_ARG, "communicator is null");
  if (ms < 0) return fail(DWBNQ_ERR_INVALID_ARG, "deadline %d ms is negative", ms);
  static_cast<Comm *>(comm)->deadline_ms = ms;
  return DWBNQ_OK;
}

extern "C" int dwbnq_comm_destroy(void *comm) {
  clear_error();
  if (!comm) return DWBNQ_OK;
  Comm *c = static_cast<Comm *>(comm);
  int result = DWBNQ_OK;
  if (c->nccl && g_nccl.ok) {
    int r = g_nccl.CommDestroy(c->nccl);
    if (r != kNcclSuccess) result = fail_nccl(r, "ncclCommDestroy");
  }
  delete c;
  return result;
}

extern "C" int dwbnq_comm_allreduce_max_f32(void *comm, float *buf, int64_t count, void *stream,
                                            int timeout_ms) {
  clear_error();
  return comm_allreduce_max(comm, buf, count, static_cast<cudaStream_t>(stream), timeout_ms);
}
