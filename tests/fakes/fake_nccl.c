/* A stand-in for libnccl.so.2 for CPU tests of the bounded waits in sca_mgpu_*: no GPU, no network.
 * Behaviour is chosen through the environment variable FAKE_NCCL_MODE when the communicator is created:
 *   "ok"        every call succeeds at once
 *   "never"     the communicator stays "in progress" for ever (a peer that never joins)
 *   "fail"      the communicator reports an asynchronous system error
 * Every ncclCommAbort is counted; fake_nccl_aborts() returns the count. */
#include <stdlib.h>
#include <string.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef struct FakeComm { int mode; } *ncclComm_t;
typedef int ncclResult_t;
enum { ncclSuccess = 0, ncclSystemError = 2, ncclInProgress = 7 };

static int g_aborts = 0;
int fake_nccl_aborts(void) { return g_aborts; }

ncclResult_t ncclGetUniqueId(ncclUniqueId* id) {
    memset(id, 0x5a, sizeof(*id));
    return ncclSuccess;
}
ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, void* config) {
    (void)nranks; (void)id; (void)rank; (void)config;
    const char* mode = getenv("FAKE_NCCL_MODE");
    *comm = (ncclComm_t)malloc(sizeof(struct FakeComm));
    (*comm)->mode = (mode && !strcmp(mode, "never")) ? 1 : (mode && !strcmp(mode, "fail")) ? 2 : 0;
    return (*comm)->mode == 0 ? ncclSuccess : ncclInProgress;
}
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* state) {
    *state = comm->mode == 1 ? ncclInProgress : comm->mode == 2 ? ncclSystemError : ncclSuccess;
    return ncclSuccess;
}
ncclResult_t ncclCommAbort(ncclComm_t comm) {
    ++g_aborts;
    free(comm);
    return ncclSuccess;
}
ncclResult_t ncclCommDestroy(ncclComm_t comm) {
    free(comm);
    return ncclSuccess;
}
ncclResult_t ncclAllGather(const void* send, void* recv, size_t count, int dtype, ncclComm_t comm, void* stream) {
    (void)send; (void)recv; (void)count; (void)dtype; (void)comm; (void)stream;
    return ncclSuccess;
}
const char* ncclGetErrorString(ncclResult_t rc) { return rc == ncclSystemError ? "unhandled system error" : "fake"; }
