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

SCI_EXPORT std::shared_ptr<CudaDevice> CudaDevice::Create(int device_id) {
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
    return std::shared_ptr<CudaDevice>(new CudaDevice(device_id, prop.name));
}

// Tensors come from the device's stream-ordered memory pool (cudaMallocAsync on the legacy default stream)
// with the pool told to keep what is freed: a call that returns a newly allocated output every time, as the
// attention entry points do, then costs neither a cudaMalloc nor the device-wide synchronisation of a
// cudaFree. Frees are ordered on the legacy stream, i.e. after earlier work of every blocking stream.
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

SCI_EXPORT void* CudaDevice::allocate(size_t bytes) {
    void* ptr = nullptr;
    const size_t n = bytes == 0 ? 1 : bytes;
    WithDevice(id_, [&] {
        const bool pooled = PoolReady(id_);
        const cudaError_t got = pooled ? cudaMallocAsync(&ptr, n, cudaStreamLegacy) : cudaMalloc(&ptr, n);
        if (got != cudaSuccess) {
            cudaGetLastError();
            ptr = nullptr;
            return;
        }
        // fresh tensors read as zero, like the host device's calloc
        if (cudaMemsetAsync(ptr, 0, n, cudaStreamLegacy) != cudaSuccess) cudaGetLastError();
    });
    return ptr;
}
SCI_EXPORT void CudaDevice::deallocate(void* ptr) {
    if (ptr == nullptr) return;
    WithDevice(id_, [&] {
        const cudaError_t freed = PoolReady(id_) ? cudaFreeAsync(ptr, cudaStreamLegacy) : cudaFree(ptr);
        if (freed != cudaSuccess) cudaGetLastError();
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
    static std::mutex mu;
    static std::map<int, std::shared_ptr<CudaDevice>>* devices = new std::map<int, std::shared_ptr<CudaDevice>>();
    std::lock_guard<std::mutex> lock(mu);
    auto it = devices->find(index);
    if (it != devices->end()) return it->second;
    std::shared_ptr<CudaDevice> created = CudaDevice::Create(index);
    if (created) (*devices)[index] = created;
    return created;
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
