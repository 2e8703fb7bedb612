/* Stand-in for libnccl used by tests/test_comm_cpu.py: the failure is made on the host, no GPU and no
 * real NCCL involved.  Behaviour is chosen with the environment variable FAKE_NCCL_MODE when the first
 * communicator is created:
 *   never_joins   ncclCommInitRankConfig returns ncclInProgress and the communicator's state stays
 *                 ncclInProgress for ever (a peer that never called init)
 *   async_error   init completes, the communicator then reports ncclRemoteError
 *   ok            every call succeeds at once; ncclAllReduce only counts its calls
 * Result codes and the entry points' signatures are those of the public nccl.h. */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

typedef enum { ncclSuccess = 0, ncclUnhandledCudaError = 1, ncclSystemError = 2, ncclInternalError = 3, ncclInvalidArgument = 4,
               ncclInvalidUsage = 5, ncclRemoteError = 6, ncclInProgress = 7 } ncclResult_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef struct fake_comm { int mode; int aborted; } *ncclComm_t;

static int g_aborts = 0, g_allreduces = 0, g_destroys = 0;
int fake_nccl_abort_count(void) { return g_aborts; }
int fake_nccl_allreduce_count(void) { return g_allreduces; }
int fake_nccl_destroy_count(void) { return g_destroys; }

static int mode_from_env(void) {
  const char* m = getenv("FAKE_NCCL_MODE");
  if (m && strcmp(m, "never_joins") == 0) return 1;
  if (m && strcmp(m, "async_error") == 0) return 2;
  return 0;
}

ncclResult_t ncclGetVersion(int* v) { *v = 22703; return ncclSuccess; }
ncclResult_t ncclGetUniqueId(ncclUniqueId* id) { memset(id, 0x5a, sizeof *id); return ncclSuccess; }
ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* config) {
  (void)nranks; (void)id; (void)rank; (void)config;
  *comm = (ncclComm_t)calloc(1, sizeof(struct fake_comm));
  (*comm)->mode = mode_from_env();
  return (*comm)->mode == 1 ? ncclInProgress : ncclSuccess;
}
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* state) {
  *state = comm->mode == 1 ? ncclInProgress : comm->mode == 2 ? ncclRemoteError : ncclSuccess;
  return ncclSuccess;
}
ncclResult_t ncclCommAbort(ncclComm_t comm) { comm->aborted = 1; ++g_aborts; return ncclSuccess; }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { (void)comm; ++g_destroys; return ncclSuccess; }
ncclResult_t ncclAllReduce(const void* s, void* r, size_t count, int dt, int op, ncclComm_t comm, void* stream) {
  (void)s; (void)r; (void)count; (void)dt; (void)op; (void)comm; (void)stream;
  ++g_allreduces;
  return ncclSuccess;
}
ncclResult_t ncclGroupStart(void) { return ncclSuccess; }
ncclResult_t ncclGroupEnd(void) { return ncclSuccess; }
const char* ncclGetErrorString(ncclResult_t r) { return r == ncclRemoteError ? "remote process exited or there was a network error" : r == ncclInProgress ? "in progress" : "fake nccl"; }
