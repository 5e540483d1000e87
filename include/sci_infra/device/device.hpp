// sci::Device: allocation and copy interface a Tensor is bound to. HostDevice serves host memory;
// CudaDevice (device/cuda_device.hpp) serves one GPU.
#pragma once

#include <cstddef>
#include <cstring>
#include <string>

#include "core/types.hpp"

namespace sci {

class Stream;

class Device {
public:
    virtual ~Device() = default;
    virtual DeviceType type() const = 0;
    virtual int id() const { return 0; }
    virtual std::string name() const = 0;
    virtual void* allocate(size_t bytes) = 0;   // nullptr on failure; fresh memory is zero-filled
    virtual void deallocate(void* ptr) = 0;
    virtual void copy_to_device(void* dst, const void* src, size_t bytes) = 0;  // host -> this device, blocking
    virtual void copy_to_host(void* dst, const void* src, size_t bytes) = 0;    // this device -> host, blocking
    virtual void copy_within(void* dst, const void* src, size_t bytes) { std::memcpy(dst, src, bytes); }
    virtual void memset(void* ptr, int value, size_t bytes) = 0;
    virtual void synchronize() = 0;
    virtual void copy_async(void* dst, const void* src, size_t bytes, Stream& stream);  // host -> device on `stream`
    virtual size_t total_memory() const { return 0; }
    virtual size_t free_memory() const { return 0; }
};

// Process-wide host-memory device.
Device& HostDevice();
// Name kept for sources written against the reference's CPU-only shim.
inline Device& StubHostDevice() { return HostDevice(); }

}  // namespace sci
