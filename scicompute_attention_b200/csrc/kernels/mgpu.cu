// Multi-GPU plumbing behind the C ABI: a NCCL communicator with bounded waits, for the one collective of the
// design - the all-gather of the (m, l, O) triples of a KV-sequence-split decode. No counterpart in the reference,
// which is single-GPU.
//
// NCCL is loaded at run time (dlopen of libnccl.so.2, or of the file SCA_NCCL_LIBRARY names), so the library has no
// link-time dependency on it and a process that already carries a NCCL (e.g. through its ML framework) shares that
// copy. The communicator is created NON-BLOCKING: every NCCL call returns at once and progress is observed through
// ncclCommGetAsyncError. Both places where a rank can wait for its peers - communicator set-up and the completion of
// an all-gather - are wall-clock bounded; when the limit passes the communicator is aborted (ncclCommAbort, which
// also makes a waiting NCCL kernel leave) and the call returns SCA_TIMEOUT instead of hanging.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include "common.cuh"

namespace sca_b200 {
namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    std::string error;
};

NcclApi& Api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* named = std::getenv("SCA_NCCL_LIBRARY");
        const char* file = (named != nullptr && named[0] != '\0') ? named : "libnccl.so.2";
        api.handle = dlopen(file, RTLD_NOW | RTLD_GLOBAL);
        if (api.handle == nullptr) {
            api.error = std::string("cannot load ") + file + ": " + dlerror();
            return;
        }
        auto need = [&](const char* name) -> void* {
            void* sym = dlsym(api.handle, name);
            if (sym == nullptr && api.error.empty()) api.error = std::string(file) + " lacks " + name;
            return sym;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(need("ncclGetUniqueId"));
        api.CommInitRankConfig = reinterpret_cast<decltype(api.CommInitRankConfig)>(need("ncclCommInitRankConfig"));
        api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(need("ncclCommGetAsyncError"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(need("ncclCommAbort"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(need("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(need("ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(need("ncclGetErrorString"));
    });
    return api;
}

int FailNccl(const NcclApi& api, ncclResult_t rc, const char* what) {
    const char* text = api.GetErrorString != nullptr ? api.GetErrorString(rc) : "?";
    return Fail(SCA_CUDA_ERROR, std::string(what) + ": NCCL error " + std::to_string(static_cast<int>(rc)) + " (" + text + ")");
}

struct Communicator {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    bool aborted = false;
};

using Clock = std::chrono::steady_clock;

// Polls the communicator until its pending operation has finished. 0 = done, SCA_TIMEOUT after `timeout_ms`
// (the communicator is aborted first), another code on a NCCL error.
int WaitForCommunicator(NcclApi& api, Communicator* c, int32_t timeout_ms, const char* what) {
    const Clock::time_point start = Clock::now();
    while (true) {
        ncclResult_t state = ncclSuccess;
        const ncclResult_t rc = api.CommGetAsyncError(c->comm, &state);
        if (rc != ncclSuccess) return FailNccl(api, rc, what);
        if (state == ncclSuccess) return SCA_OK;
        if (state != ncclInProgress) {
            api.CommAbort(c->comm);
            c->aborted = true;
            return FailNccl(api, state, what);
        }
        if (timeout_ms > 0 && Clock::now() - start > std::chrono::milliseconds(timeout_ms)) {
            api.CommAbort(c->comm);
            c->aborted = true;
            return Fail(SCA_TIMEOUT, std::string(what) + ": no answer from the other ranks within " + std::to_string(timeout_ms) +
                                         " ms; the communicator was aborted");
        }
        // an enqueue on a non-blocking communicator finishes within microseconds: probe without sleeping first, so
        // that a decode step does not pay a timer tick, and back off only when the wait is a real one
        if (Clock::now() - start < std::chrono::microseconds(500)) std::this_thread::yield();
        else std::this_thread::sleep_for(std::chrono::microseconds(100));
    }
}

}  // namespace
}  // namespace sca_b200

using namespace sca_b200;

extern "C" int sca_mgpu_unique_id(unsigned char* id_out) {
    ClearError();
    static_assert(sizeof(ncclUniqueId) == SCA_MGPU_ID_BYTES, "SCA_MGPU_ID_BYTES must be the size of ncclUniqueId");
    if (id_out == nullptr) return Fail(SCA_INVALID_ARGUMENT, "mgpu: null id buffer");
    NcclApi& api = Api();
    if (!api.error.empty()) return Fail(SCA_NOT_IMPLEMENTED, "mgpu: " + api.error);
    ncclUniqueId id;
    if (const ncclResult_t rc = api.GetUniqueId(&id); rc != ncclSuccess) return FailNccl(api, rc, "ncclGetUniqueId");
    std::memcpy(id_out, &id, sizeof(id));
    return SCA_OK;
}

extern "C" int sca_mgpu_init(const unsigned char* id, int32_t rank, int32_t world, int32_t timeout_ms, void** comm_out) {
    ClearError();
    if (id == nullptr || comm_out == nullptr) return Fail(SCA_INVALID_ARGUMENT, "mgpu init: null argument");
    *comm_out = nullptr;
    if (world < 1 || rank < 0 || rank >= world) {
        return Fail(SCA_INVALID_ARGUMENT, "mgpu init: rank=" + std::to_string(rank) + " world=" + std::to_string(world));
    }
    NcclApi& api = Api();
    if (!api.error.empty()) return Fail(SCA_NOT_IMPLEMENTED, "mgpu: " + api.error);
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 0;  // every call returns at once; waits happen here, with a limit
    Communicator* c = new Communicator();
    c->rank = rank;
    c->world = world;
    const ncclResult_t rc = api.CommInitRankConfig(&c->comm, world, uid, rank, &config);
    if (rc != ncclSuccess && rc != ncclInProgress) {
        delete c;
        return FailNccl(api, rc, "ncclCommInitRankConfig");
    }
    // a non-positive limit means the default of one minute: set-up never waits without a bound
    if (int wait = WaitForCommunicator(api, c, timeout_ms > 0 ? timeout_ms : 60000, "mgpu init")) {
        delete c;  // aborted above when it timed out or failed
        return wait;
    }
    *comm_out = c;
    return SCA_OK;
}

extern "C" int sca_mgpu_allgather_triples(void* comm, const float* mine, float* gathered, int64_t floats_per_rank,
                                          void* stream, int32_t timeout_ms) {
    ClearError();
    Communicator* c = static_cast<Communicator*>(comm);
    if (c == nullptr || mine == nullptr || gathered == nullptr || floats_per_rank < 1) {
        return Fail(SCA_INVALID_ARGUMENT, "mgpu all-gather: null argument or empty payload");
    }
    if (c->aborted) return Fail(SCA_INVALID_ARGUMENT, "mgpu all-gather: the communicator was aborted");
    NcclApi& api = Api();
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const ncclResult_t rc = api.AllGather(mine, gathered, static_cast<size_t>(floats_per_rank), ncclFloat, c->comm, s);
    if (rc != ncclSuccess && rc != ncclInProgress) return FailNccl(api, rc, "ncclAllGather");
    // the enqueue itself may still be in progress on a non-blocking communicator (bounded even for asynchronous use)
    if (int wait = WaitForCommunicator(api, c, timeout_ms > 0 ? timeout_ms : 30000, "mgpu all-gather (enqueue)")) return wait;
    if (timeout_ms <= 0) return SCA_OK;  // asynchronous use: the caller orders later work on the stream
    // bounded completion: an event behind the collective, polled together with the communicator's state
    cudaEvent_t done = nullptr;
    if (cudaError_t e = cudaEventCreateWithFlags(&done, cudaEventDisableTiming); e != cudaSuccess) {
        return FailCuda(e, "mgpu all-gather: cudaEventCreate");
    }
    int result = SCA_OK;
    if (cudaError_t e = cudaEventRecord(done, s); e != cudaSuccess) {
        result = FailCuda(e, "mgpu all-gather: cudaEventRecord");
    } else {
        const Clock::time_point start = Clock::now();
        while (true) {
            const cudaError_t q = cudaEventQuery(done);
            if (q == cudaSuccess) break;
            if (q != cudaErrorNotReady) {
                cudaGetLastError();
                result = FailCuda(q, "mgpu all-gather: cudaEventQuery");
                break;
            }
            ncclResult_t state = ncclSuccess;
            api.CommGetAsyncError(c->comm, &state);
            if (state != ncclSuccess && state != ncclInProgress) {
                api.CommAbort(c->comm);
                c->aborted = true;
                result = FailNccl(api, state, "mgpu all-gather");
                break;
            }
            if (Clock::now() - start > std::chrono::milliseconds(timeout_ms)) {
                api.CommAbort(c->comm);  // makes the waiting collective kernel leave
                c->aborted = true;
                result = Fail(SCA_TIMEOUT, "mgpu all-gather: a rank did not deliver its triples within " +
                                               std::to_string(timeout_ms) + " ms; the communicator was aborted");
                break;
            }
            std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
    }
    cudaEventDestroy(done);
    return result;
}

extern "C" int sca_mgpu_abort(void* comm) {
    ClearError();
    Communicator* c = static_cast<Communicator*>(comm);
    if (c == nullptr) return Fail(SCA_INVALID_ARGUMENT, "mgpu abort: null communicator");
    if (!c->aborted) {
        Api().CommAbort(c->comm);
        c->aborted = true;
    }
    return SCA_OK;
}

extern "C" int sca_mgpu_destroy(void* comm) {
    ClearError();
    Communicator* c = static_cast<Communicator*>(comm);
    if (c == nullptr) return SCA_OK;
    if (!c->aborted) Api().CommDestroy(c->comm);  // an aborted communicator is already gone
    delete c;
    return SCA_OK;
}
