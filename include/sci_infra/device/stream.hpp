// sci::Stream: a non-owning view of a CUDA stream (handle() is the cudaStream_t as void*; nullptr is
// the default stream). GetCurrent() is the per-thread "current" stream that public entry points use
// when the caller passes no stream.
#pragma once

#include "core/types.hpp"

namespace sci {

class Stream {
public:
    Stream() = default;
    explicit Stream(void* cuda_stream, DeviceType type = DeviceType::kCUDA) : handle_(cuda_stream), type_(type) {}

    void* handle() const { return handle_; }
    DeviceType device_type() const { return type_; }
    void synchronize();  // no-op for a CPU stream

    static Stream& GetCurrent();
    static void SetCurrent(const Stream& stream);

private:
    void* handle_{nullptr};
    DeviceType type_{DeviceType::kCPU};
};

}  // namespace sci
