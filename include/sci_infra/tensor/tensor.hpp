// sci::Tensor: move-only, contiguous, bound to a Device. Owning tensors free their memory through
// the device; the external-pointer constructor wraps caller memory.
#pragma once

#include <algorithm>
#include <cstddef>

#include "core/status.hpp"
#include "core/types.hpp"
#include "device/device.hpp"

namespace sci {

class Tensor {
public:
    Tensor() = default;
    Tensor(const TensorShape& shape, DType dtype, Device& device)
        : shape_(shape), dtype_(dtype), device_(&device),
          bytes_(static_cast<size_t>(shape.num_elements()) * kDTypeSize(dtype)) {
        data_ = device.allocate(bytes_);
        owns_ = data_ != nullptr;
    }
    Tensor(const TensorShape& shape, DType dtype, Device& device, void* external_data, bool owns_data = false)
        : shape_(shape), dtype_(dtype), device_(&device), data_(external_data), owns_(owns_data),
          bytes_(static_cast<size_t>(shape.num_elements()) * kDTypeSize(dtype)) {}
    ~Tensor() { Release(); }

    Tensor(Tensor&& other) noexcept { Steal(other); }
    Tensor& operator=(Tensor&& other) noexcept {
        if (this != &other) {
            Release();
            Steal(other);
        }
        return *this;
    }
    Tensor(const Tensor&) = delete;
    Tensor& operator=(const Tensor&) = delete;

    const TensorShape& shape() const { return shape_; }
    index_t ndims() const { return shape_.ndims(); }
    index_t dim(size_t i) const { return shape_.dim(i); }
    index_t num_elements() const { return shape_.num_elements(); }
    DType dtype() const { return dtype_; }
    Device& device() const { return *device_; }
    DeviceType device_type() const { return device_ != nullptr ? device_->type() : DeviceType::kCPU; }
    void* data() { return data_; }
    const void* data() const { return data_; }
    size_t num_bytes() const { return bytes_; }
    bool is_contiguous() const { return true; }

    // Copies `bytes` from HOST memory into this tensor (blocking).
    void copy_from(const void* host_source, size_t bytes) {
        if (data_ == nullptr || host_source == nullptr || device_ == nullptr) return;
        device_->copy_to_device(data_, host_source, std::min(bytes, bytes_));
    }
    // Copies another tensor's bytes into this one across any pair of devices (blocking).
    void copy_from(const Tensor& other);

private:
    void Release() {
        if (owns_ && data_ != nullptr && device_ != nullptr) device_->deallocate(data_);
        data_ = nullptr;
        owns_ = false;
    }
    void Steal(Tensor& other) {
        shape_ = other.shape_;
        dtype_ = other.dtype_;
        device_ = other.device_;
        data_ = other.data_;
        owns_ = other.owns_;
        bytes_ = other.bytes_;
        other.data_ = nullptr;
        other.owns_ = false;
    }

    TensorShape shape_{};
    DType dtype_{DType::kFloat32};
    Device* device_{nullptr};
    void* data_{nullptr};
    bool owns_{false};
    size_t bytes_{0};
};

}  // namespace sci
