// Host-side plumbing shared by every entry point of the C ABI: thread-local error text, launch
// checks, the dynamic shared-memory opt-in cache and the device probe.
//
// Stands in for src/runtime/launcher.cu:26-111 (smem attribute cache, immediate launch check,
// SCI_ATTENTION_DEBUG_SYNC) and src/runtime/device_probe.cu:35-84 (the reference's own C ABI).
#include <cstdlib>
#include <chrono>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace sca_b200 {
namespace {

thread_local std::string g_last_error;

bool DebugSync() {
    static const bool on = [] {
        const char* v = std::getenv("SCI_ATTENTION_DEBUG_SYNC");
        return v != nullptr && v[0] == '1';
    }();
    return on;
}

}  // namespace

bool DebugSyncEnabled() { return DebugSync(); }

int Fail(int code, const std::string& message) {
    g_last_error = message;
    return code;
}

void ClearError() { g_last_error.clear(); }

int FailCuda(cudaError_t err, const char* what) {
    const int code = (err == cudaErrorMemoryAllocation) ? SCA_CUDA_OOM
                     : (err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver)
                         ? SCA_CUDA_NOT_AVAILABLE
                         : SCA_CUDA_ERROR;
    return Fail(code, std::string(what) + ": " + cudaGetErrorName(err) + ": " + cudaGetErrorString(err));
}

int CheckLaunch(const char* kernel_name, cudaStream_t stream) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return FailCuda(err, kernel_name);
    if (DebugSync()) {
        err = cudaStreamSynchronize(stream);
        if (err != cudaSuccess) return FailCuda(err, kernel_name);
    }
    return SCA_OK;
}

int EnsureDynamicSmem(const void* kernel, size_t bytes, const char* kernel_name) {
    // the 48 KiB default covers static + dynamic shared memory together: opt in early enough to leave room for a
    // kernel's static variables
    if (bytes <= 40 * 1024) return SCA_OK;
    static std::mutex mu;
    static std::unordered_map<const void*, size_t> granted;  // per (device, kernel) would be stricter;
    int device = 0;                                           // the key below folds the device in
    cudaGetDevice(&device);
    const void* key = reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(kernel) ^
                                                    (static_cast<uintptr_t>(device) << 56));
    std::lock_guard<std::mutex> lock(mu);
    auto it = granted.find(key);
    if (it != granted.end() && it->second >= bytes) return SCA_OK;
    const cudaError_t err =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (err != cudaSuccess) {
        cudaGetLastError();
        return FailCuda(err, (std::string("cudaFuncSetAttribute(") + kernel_name + ", dynamic shared memory " +
                              std::to_string(bytes) + " B)").c_str());
    }
    granted[key] = bytes;
    return SCA_OK;
}

int SmCount() {
    static thread_local int cached_device = -1;
    static thread_local int cached = 0;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 148;
    if (device != cached_device) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_device = device;
    }
    return cached;
}

}  // namespace sca_b200

using namespace sca_b200;

extern "C" const char* sca_last_error(void) { return g_last_error.c_str(); }

namespace {
// The reference's host layer asks the probe on every attention call (DeviceCapability::CudaAvailable,
// src/runtime/capability.cpp:86-89, called from every backend's Supports / Forward), and cudaGetDeviceProperties
// alone takes milliseconds. The static part of the answer is therefore kept per device after the first successful
// probe; the free-memory figure is refreshed when it is older than 50 ms.
constexpr int kMaxProbedDevices = 64;
struct CachedProbe {
    bool valid = false;
    ScaDeviceProbe probe{};
    std::chrono::steady_clock::time_point memory_read{};
};
std::mutex g_probe_mutex;
CachedProbe g_probe_cache[kMaxProbedDevices];
}  // namespace

extern "C" int sca_probe_device(int device_id, ScaDeviceProbe* out) {
    if (out == nullptr) return 1;
    std::memset(out, 0, sizeof(*out));
    out->binary_has_sm80 = 1;
    out->binary_has_sm90 = 1;
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count <= 0 || device_id < 0 || device_id >= count) {
        cudaGetLastError();
        std::strncpy(out->name, "cuda-unavailable", SCA_DEVICE_NAME_MAX - 1);
        return err != cudaSuccess ? static_cast<int>(err) : 1;
    }
    const bool cacheable = device_id < kMaxProbedDevices;
    std::unique_lock<std::mutex> lock(g_probe_mutex, std::defer_lock);
    if (cacheable) lock.lock();
    CachedProbe local;
    CachedProbe& slot = cacheable ? g_probe_cache[device_id] : local;
    if (!slot.valid) {
        cudaDeviceProp prop{};
        err = cudaGetDeviceProperties(&prop, device_id);
        if (err != cudaSuccess) {
            cudaGetLastError();
            return static_cast<int>(err);
        }
        ScaDeviceProbe& p = slot.probe;
        std::memset(&p, 0, sizeof(p));
        p.binary_has_sm80 = 1;
        p.binary_has_sm90 = 1;
        std::strncpy(p.name, prop.name, SCA_DEVICE_NAME_MAX - 1);
        p.major = prop.major;
        p.minor = prop.minor;
        p.sm_count = prop.multiProcessorCount;
        p.smem_per_sm = prop.sharedMemPerMultiprocessor;
        p.smem_per_block_default = prop.sharedMemPerBlock;
        p.smem_per_block_optin = prop.sharedMemPerBlockOptin;
        p.regs_per_sm = static_cast<unsigned long long>(prop.regsPerMultiprocessor);
        p.max_threads_per_sm = static_cast<unsigned long long>(prop.maxThreadsPerMultiProcessor);
        p.l2_bytes = static_cast<unsigned long long>(prop.l2CacheSize);
        p.total_mem_bytes = prop.totalGlobalMem;
        p.cuda_available = 1;
        slot.valid = true;
        slot.memory_read = {};
    }
    const auto now = std::chrono::steady_clock::now();
    int current = 0;
    if (now - slot.memory_read > std::chrono::milliseconds(50) && cudaGetDevice(&current) == cudaSuccess &&
        current == device_id) {
        size_t free_b = 0, total_b = 0;
        if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) {
            slot.probe.free_mem_bytes = free_b;
            slot.memory_read = now;
        } else {
            cudaGetLastError();
        }
    }
    *out = slot.probe;
    return 0;
}

extern "C" int sca_probe_device_b200(int device_id, ScaDeviceProbeB200* out) {
    if (out == nullptr) return 1;
    std::memset(out, 0, sizeof(*out));
    out->binary_has_sm100a = 1;
    const int rc = sca_probe_device(device_id, &out->base);
    if (rc != 0) return rc;
    out->tmem_columns = (out->base.major == 10) ? 512 : 0;
    out->max_cluster_size = out->base.major >= 9 ? 8 : 1;
    return 0;
}

extern "C" int sca_mem_get_info(unsigned long long* free_bytes, unsigned long long* total_bytes) {
    size_t free_b = 0, total_b = 0;
    const cudaError_t err = cudaMemGetInfo(&free_b, &total_b);
    if (err != cudaSuccess) {
        cudaGetLastError();
        if (free_bytes != nullptr) *free_bytes = 0;
        if (total_bytes != nullptr) *total_bytes = 0;
        return static_cast<int>(err);
    }
    if (free_bytes != nullptr) *free_bytes = free_b;
    if (total_bytes != nullptr) *total_bytes = total_b;
    return 0;
}
