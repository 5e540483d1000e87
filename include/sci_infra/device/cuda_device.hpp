// sci::CudaDevice (one GPU: cudaMalloc / cudaMemcpy / cudaMemset behind the Device interface) and
// sci::DeviceManager (shared handles by (type, index)).
#pragma once

#include <memory>

#include "device/device.hpp"

namespace sci {

class CudaDevice final : public Device {
public:
    // nullptr when no such GPU is visible.
    static std::shared_ptr<CudaDevice> Create(int device_id);

    DeviceType type() const override { return DeviceType::kCUDA; }
    int id() const override { return id_; }
    std::string name() const override { return name_; }
    void* allocate(size_t bytes) override;
    void deallocate(void* ptr) override;
    void copy_to_device(void* dst, const void* src, size_t bytes) override;
    void copy_to_host(void* dst, const void* src, size_t bytes) override;
    void copy_within(void* dst, const void* src, size_t bytes) override;
    void memset(void* ptr, int value, size_t bytes) override;
    void synchronize() override;
    void copy_async(void* dst, const void* src, size_t bytes, Stream& stream) override;
    size_t total_memory() const override;
    size_t free_memory() const override;

private:
    CudaDevice(int id, std::string name) : id_(id), name_(std::move(name)) {}
    int id_;
    std::string name_;
};

// While one of these is alive on a thread, CudaDevice::allocate / deallocate on that thread are ordered on
// `cuda_stream` (cudaMallocAsync, the zero fill and cudaFreeAsync all go to that stream) instead of the legacy
// default stream. The attention entry points open one for the stream of the call, so that a freshly allocated,
// zero-filled output is ordered before the kernel that writes it on ANY kind of stream - a cudaStreamNonBlocking
// stream does not synchronise with the legacy stream. When the scope closes on such a stream it leaves a marker
// behind; memory that is released later, outside any scope, is freed only after that marker, i.e. after the last
// work the library queued on a non-blocking stream of that device.
class StreamOrderedScope {
public:
    explicit StreamOrderedScope(void* cuda_stream);
    ~StreamOrderedScope();
    StreamOrderedScope(const StreamOrderedScope&) = delete;
    StreamOrderedScope& operator=(const StreamOrderedScope&) = delete;

private:
    void* previous_;
    bool previous_active_;
};

class DeviceManager {
public:
    static DeviceManager& Instance();
    // CPU / pinned: the host device. CUDA: the GPU with that index, or nullptr when absent.
    std::shared_ptr<Device> get_device(DeviceType type, int index);
};

}  // namespace sci
