// sci:: infrastructure layer: host device, CUDA device, device manager, stream, cross-device tensor
// copies. The only host translation unit that talks to the CUDA runtime directly.
#include <cuda_runtime_api.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

#include "device/cuda_device.hpp"
#include "device/device.hpp"
#include "device/stream.hpp"
#include "tensor/tensor.hpp"

#define SCI_EXPORT __attribute__((visibility("default")))

namespace sci {

// ---- Device default -----------------------------------------------------------------------------
SCI_EXPORT void Device::copy_async(void* dst, const void* src, size_t bytes, Stream&) { copy_to_device(dst, src, bytes); }

// ---- host device -----------------------------------------------------------------------------------
namespace {

class HostDeviceImpl final : public Device {
public:
    DeviceType type() const override { return DeviceType::kCPU; }
    std::string name() const override { return "host"; }
    void* allocate(size_t bytes) override { return std::calloc(1, bytes == 0 ? 1 : bytes); }
    void deallocate(void* ptr) override { std::free(ptr); }
    void copy_to_device(void* dst, const void* src, size_t bytes) override { std::memcpy(dst, src, bytes); }
    void copy_to_host(void* dst, const void* src, size_t bytes) override { std::memcpy(dst, src, bytes); }
    void memset(void* ptr, int value, size_t bytes) override { std::memset(ptr, value, bytes); }
    void synchronize() override {}
};

}  // namespace

SCI_EXPORT Device& HostDevice() {
    static HostDeviceImpl* device = new HostDeviceImpl();  // never destroyed: tensors may outlive statics
    return *device;
}

// ---- CUDA device -----------------------------------------------------------------------------------
namespace {

// Runs `fn` with `device` current and restores the previous device afterwards.
template <typename Fn>
void WithDevice(int device, Fn&& fn) {
    int previous = -1;
    cudaGetDevice(&previous);
    if (previous != device) cudaSetDevice(device);
    fn();
    if (previous != device && previous >= 0) cudaSetDevice(previous);
}

}  // namespace

// One CudaDevice object per GPU for the life of the process: library-internal tensors that outlive a call (the
// scratch pool) keep a plain Device pointer, and callers are free to drop their handle at any time - the
// reference's own tests create a fresh handle per case (tests/kernel/test_naive_correctness.cu:24-27).
SCI_EXPORT std::shared_ptr<CudaDevice> CudaDevice::Create(int device_id) {
    static std::mutex mu;
    static auto* devices = new std::map<int, std::shared_ptr<CudaDevice>>();  // never destroyed
    std::lock_guard<std::mutex> lock(mu);
    auto it = devices->find(device_id);
    if (it != devices->end()) return it->second;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device_id < 0 || device_id >= count) {
        cudaGetLastError();
        return nullptr;
    }
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, device_id) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    std::shared_ptr<CudaDevice> created(new CudaDevice(device_id, prop.name));
    (*devices)[device_id] = created;
    return created;
}

// Tensors come from the device's stream-ordered memory pool (cudaMallocAsync) with the pool told to keep what
// is freed: a call that returns a newly allocated output every time, as the attention entry points do, then
// costs neither a cudaMalloc nor the device-wide synchronisation of a cudaFree. Outside a StreamOrderedScope
// allocation and release are ordered on the legacy default stream, inside one on the scope's stream.
// Memory the pool holds counts as used in cudaMemGetInfo until cudaDeviceReset or process exit.
namespace {
bool PoolReady(int id) {
    static std::mutex mu;
    static std::map<int, bool>* ready = new std::map<int, bool>();
    std::lock_guard<std::mutex> lock(mu);
    auto it = ready->find(id);
    if (it != ready->end()) return it->second;
    bool ok = false;
    int supported = 0;
    cudaMemPool_t pool = nullptr;
    if (cudaDeviceGetAttribute(&supported, cudaDevAttrMemoryPoolsSupported, id) == cudaSuccess && supported != 0 &&
        cudaDeviceGetDefaultMemPool(&pool, id) == cudaSuccess) {
        unsigned long long keep = ~0ull;
        ok = cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) == cudaSuccess;
    }
    if (!ok) cudaGetLastError();
    (*ready)[id] = ok;
    return ok;
}
}  // namespace

// ---- stream-ordered scope (see cuda_device.hpp) -------------------------------------------------------
namespace {
thread_local void* g_scope_stream = nullptr;
thread_local bool g_scope_active = false;

struct LastWork {
    cudaEvent_t event = nullptr;
    bool recorded = false;
};
std::mutex& LastWorkMutex() {
    static std::mutex mu;
    return mu;
}
// Per device: marker after the last library work queued on a non-blocking stream. Leaked on purpose (events must
// not be destroyed from a static destructor, after the CUDA runtime is gone).
std::map<int, LastWork>& LastWorkMap() {
    static auto* map = new std::map<int, LastWork>();
    return *map;
}

bool IsNonBlocking(cudaStream_t stream) {
    if (stream == nullptr || stream == cudaStreamLegacy || stream == cudaStreamPerThread) return false;
    unsigned int flags = 0;
    if (cudaStreamGetFlags(stream, &flags) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return (flags & cudaStreamNonBlocking) != 0;
}
bool IsCapturing(cudaStream_t stream) {
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &status) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return status != cudaStreamCaptureStatusNone;
}
}  // namespace

SCI_EXPORT StreamOrderedScope::StreamOrderedScope(void* cuda_stream)
    : previous_(g_scope_stream), previous_active_(g_scope_active) {
    g_scope_stream = cuda_stream;
    g_scope_active = true;
}

SCI_EXPORT StreamOrderedScope::~StreamOrderedScope() {
    cudaStream_t stream = static_cast<cudaStream_t>(g_scope_stream);
    g_scope_stream = previous_;
    g_scope_active = previous_active_;
    if (!IsNonBlocking(stream) || IsCapturing(stream)) return;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    std::lock_guard<std::mutex> lock(LastWorkMutex());
    LastWork& last = LastWorkMap()[device];
    if (last.event == nullptr && cudaEventCreateWithFlags(&last.event, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        last.event = nullptr;
        return;
    }
    if (cudaEventRecord(last.event, stream) == cudaSuccess) last.recorded = true;
    else cudaGetLastError();
}

SCI_EXPORT void* CudaDevice::allocate(size_t bytes) {
    void* ptr = nullptr;
    const size_t n = bytes == 0 ? 1 : bytes;
    WithDevice(id_, [&] {
        const bool pooled = PoolReady(id_);
        cudaStream_t stream = g_scope_active ? static_cast<cudaStream_t>(g_scope_stream) : cudaStreamLegacy;
        const cudaError_t got = pooled ? cudaMallocAsync(&ptr, n, stream) : cudaMalloc(&ptr, n);
        if (got != cudaSuccess) {
            cudaGetLastError();
            ptr = nullptr;
            return;
        }
        // fresh tensors read as zero, like the host device's calloc
        if (cudaMemsetAsync(ptr, 0, n, stream) != cudaSuccess) cudaGetLastError();
    });
    return ptr;
}
SCI_EXPORT void CudaDevice::deallocate(void* ptr) {
    if (ptr == nullptr) return;
    WithDevice(id_, [&] {
        if (!PoolReady(id_)) {
            if (cudaFree(ptr) != cudaSuccess) cudaGetLastError();  // synchronises the device: nothing can be in flight
            return;
        }
        cudaStream_t stream = cudaStreamLegacy;
        if (g_scope_active) {
            stream = static_cast<cudaStream_t>(g_scope_stream);  // a temporary of the running call: same stream
        } else {
            // released by the caller at some later time: after earlier work of every blocking stream (legacy-stream
            // semantics) and after the last library work on a non-blocking stream of this device
            std::lock_guard<std::mutex> lock(LastWorkMutex());
            auto it = LastWorkMap().find(id_);
            if (it != LastWorkMap().end() && it->second.recorded &&
                cudaStreamWaitEvent(cudaStreamLegacy, it->second.event, 0) != cudaSuccess) {
                cudaGetLastError();
            }
        }
        if (cudaFreeAsync(ptr, stream) != cudaSuccess) cudaGetLastError();
    });
}
SCI_EXPORT void CudaDevice::copy_to_device(void* dst, const void* src, size_t bytes) {
    WithDevice(id_, [&] { cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice); });
}
SCI_EXPORT void CudaDevice::copy_to_host(void* dst, const void* src, size_t bytes) {
    WithDevice(id_, [&] { cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost); });
}
SCI_EXPORT void CudaDevice::copy_within(void* dst, const void* src, size_t bytes) {
    WithDevice(id_, [&] { cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice); });
}
SCI_EXPORT void CudaDevice::memset(void* ptr, int value, size_t bytes) {
    WithDevice(id_, [&] { cudaMemset(ptr, value, bytes); });
}
SCI_EXPORT void CudaDevice::synchronize() {
    WithDevice(id_, [&] { cudaDeviceSynchronize(); });
}
SCI_EXPORT void CudaDevice::copy_async(void* dst, const void* src, size_t bytes, Stream& stream) {
    WithDevice(id_, [&] {
        cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream.handle()));
    });
}
SCI_EXPORT size_t CudaDevice::total_memory() const {
    size_t free_b = 0, total_b = 0;
    WithDevice(id_, [&] { cudaMemGetInfo(&free_b, &total_b); });
    return total_b;
}
SCI_EXPORT size_t CudaDevice::free_memory() const {
    size_t free_b = 0, total_b = 0;
    WithDevice(id_, [&] {
        cudaMemGetInfo(&free_b, &total_b);
        // what the tensor pool holds but does not use is available to the next tensor
        if (PoolReady(id_)) {
            cudaMemPool_t pool = nullptr;
            unsigned long long reserved = 0, used = 0;
            if (cudaDeviceGetDefaultMemPool(&pool, id_) == cudaSuccess &&
                cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &reserved) == cudaSuccess &&
                cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &used) == cudaSuccess && reserved > used) {
                free_b += static_cast<size_t>(reserved - used);
            } else {
                cudaGetLastError();
            }
        }
    });
    return free_b;
}

// ---- device manager --------------------------------------------------------------------------------
SCI_EXPORT DeviceManager& DeviceManager::Instance() {
    static DeviceManager* manager = new DeviceManager();
    return *manager;
}

SCI_EXPORT std::shared_ptr<Device> DeviceManager::get_device(DeviceType type, int index) {
    if (type != DeviceType::kCUDA) return std::shared_ptr<Device>(&HostDevice(), [](Device*) {});
    return CudaDevice::Create(index);  // the per-GPU object is shared and immortal
}

// ---- stream ------------------------------------------------------------------------------------------
namespace {
thread_local Stream g_current_stream;
}

SCI_EXPORT Stream& Stream::GetCurrent() { return g_current_stream; }
SCI_EXPORT void Stream::SetCurrent(const Stream& stream) { g_current_stream = stream; }
SCI_EXPORT void Stream::synchronize() {
    if (type_ == DeviceType::kCUDA) cudaStreamSynchronize(static_cast<cudaStream_t>(handle_));
}

// ---- tensor copies ------------------------------------------------------------------------------------
SCI_EXPORT void Tensor::copy_from(const Tensor& other) {
    if (data_ == nullptr || other.data_ == nullptr || device_ == nullptr || other.device_ == nullptr) return;
    const size_t bytes = std::min(bytes_, other.bytes_);
    const bool dst_gpu = device_->type() == DeviceType::kCUDA;
    const bool src_gpu = other.device_->type() == DeviceType::kCUDA;
    if (!dst_gpu && !src_gpu) {
        std::memcpy(data_, other.data_, bytes);
    } else if (dst_gpu && !src_gpu) {
        device_->copy_to_device(data_, other.data_, bytes);
    } else if (!dst_gpu && src_gpu) {
        other.device_->copy_to_host(data_, other.data_, bytes);
    } else if (device_->id() == other.device_->id()) {
        device_->copy_within(data_, other.data_, bytes);
    } else {
        cudaMemcpyPeer(data_, device_->id(), other.data_, other.device_->id(), bytes);
    }
}

}  // namespace sci
