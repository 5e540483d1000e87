// sci:: scalar and shape vocabulary (DType, DeviceType, TensorShape) - source-compatible subset of the
// infrastructure types the attention API mentions.
#pragma once

#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <vector>

namespace sci {

using index_t = int64_t;

enum class DType : uint8_t {
    kFloat32 = 0, kFloat16 = 1, kBFloat16 = 2, kInt8 = 3, kInt32 = 4, kInt64 = 5, kBool = 6, kFloat64 = 7, kUInt8 = 8,
};

constexpr size_t kDTypeSize(DType dtype) {
    switch (dtype) {
        case DType::kFloat32: case DType::kInt32: return 4;
        case DType::kFloat16: case DType::kBFloat16: return 2;
        case DType::kInt8: case DType::kBool: case DType::kUInt8: return 1;
        case DType::kInt64: case DType::kFloat64: return 8;
    }
    return 0;
}

constexpr const char* kDTypeName(DType dtype) {
    switch (dtype) {
        case DType::kFloat32: return "float32";
        case DType::kFloat16: return "float16";
        case DType::kBFloat16: return "bfloat16";
        case DType::kInt8: return "int8";
        case DType::kInt32: return "int32";
        case DType::kInt64: return "int64";
        case DType::kBool: return "bool";
        case DType::kFloat64: return "float64";
        case DType::kUInt8: return "uint8";
    }
    return "unknown";
}

enum class DeviceType : uint8_t { kCPU = 0, kCUDA = 1, kCPUPinned = 2 };

constexpr const char* kDeviceTypeName(DeviceType type) {
    switch (type) {
        case DeviceType::kCPU: return "cpu";
        case DeviceType::kCUDA: return "cuda";
        case DeviceType::kCPUPinned: return "cpu_pinned";
    }
    return "unknown";
}

enum class Layout : uint8_t { kContiguous = 0, kStrided = 1 };

// Up to 8 extents; extra initialisers are ignored.
class TensorShape {
public:
    static constexpr int kMaxDims = 8;
    TensorShape() = default;
    TensorShape(std::initializer_list<index_t> dims) { for (index_t d : dims) Push(d); }
    explicit TensorShape(const std::vector<index_t>& dims) { for (index_t d : dims) Push(d); }

    index_t ndims() const { return count_; }
    index_t dim(size_t i) const { return extents_[i]; }
    index_t& dim(size_t i) { return extents_[i]; }
    index_t num_elements() const {
        if (count_ == 0) return 0;
        index_t n = 1;
        for (index_t i = 0; i < count_; ++i) n *= extents_[i];
        return n;
    }

private:
    void Push(index_t d) { if (count_ < kMaxDims) extents_[count_++] = d; }
    index_t extents_[kMaxDims]{};
    index_t count_{0};
};

}  // namespace sci
