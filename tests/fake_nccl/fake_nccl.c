/* TEST INFRASTRUCTURE: a stand-in for libnccl with the seven entry points libdwbnq binds,
 * used (through DWBNQ_NCCL_LIB) to make the communicator's failure paths happen on the
 * HOST: no GPU kernel ever waits for a peer here.
 *   FAKE_NCCL_MODE=ok     all-reduce of one rank: nothing to do
 *   FAKE_NCCL_MODE=error  ncclAllReduce returns an error code
 *   FAKE_NCCL_MODE=stall  ncclAllReduce enqueues a host function that sleeps
 *                         FAKE_NCCL_STALL_MS on the stream: work recorded behind it does not
 *                         complete until then, as if a peer had not joined
 *   FAKE_NCCL_MODE=async  like stall, and ncclCommGetAsyncError reports an error */
#include <cuda_runtime_api.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

typedef struct { int aborted; } fake_comm;
typedef struct { char internal[128]; } ncclUniqueId;

static int g_aborts = 0, g_allreduces = 0;

static const char *mode(void) {
  const char *m = getenv("FAKE_NCCL_MODE");
  return m ? m : "ok";
}
static void CUDART_CB stall_cb(void *ms) { usleep((useconds_t)(size_t)ms * 1000); }

int fake_nccl_aborts(void) { return g_aborts; }
int fake_nccl_allreduces(void) { return g_allreduces; }

int ncclGetUniqueId(ncclUniqueId *id) {
  memset(id->internal, 0x5a, sizeof(id->internal));
  return 0;
}
int ncclCommInitRank(fake_comm **comm, int nranks, ncclUniqueId id, int rank) {
  (void)nranks;
  (void)rank;
  if (id.internal[0] != 0x5a) return 4; /* ncclInvalidArgument */
  *comm = (fake_comm *)calloc(1, sizeof(fake_comm));
  return *comm ? 0 : 2;
}
int ncclCommDestroy(fake_comm *c) {
  free(c);
  return 0;
}
int ncclCommAbort(fake_comm *c) {
  ++g_aborts;
  free(c);
  return 0;
}
int ncclCommGetAsyncError(fake_comm *c, int *err) {
  (void)c;
  *err = strcmp(mode(), "async") == 0 ? 6 /* ncclRemoteError */ : 0;
  return 0;
}
int ncclAllReduce(const void *s, void *r, size_t count, int dtype, int op, fake_comm *c, cudaStream_t stream) {
  (void)s;
  (void)r;
  (void)count;
  (void)dtype;
  (void)op;
  (void)c;
  ++g_allreduces;
  if (strcmp(mode(), "error") == 0) return 3; /* ncclInternalError */
  if (strcmp(mode(), "stall") == 0 || strcmp(mode(), "async") == 0) {
    const char *ms = getenv("FAKE_NCCL_STALL_MS");
    if (cudaLaunchHostFunc(stream, stall_cb, (void *)(size_t)(ms ? atoi(ms) : 1500)) != cudaSuccess) return 1;
  }
  return 0;
}
const char *ncclGetErrorString(int e) {
  (void)e;
  return "fake nccl error";
}
