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

class DeviceManager {
public:
    static DeviceManager& Instance();
    // CPU / pinned: the host device. CUDA: the GPU with that index, or nullptr when absent.
    std::shared_ptr<Device> get_device(DeviceType type, int index);
};

}  // namespace sci
