// sci:: status vocabulary used by the attention API. The reference takes these types from an
// infrastructure library that is not part of its repository; this is an independent, source-compatible
// implementation of the subset its public headers and tests use (Status, StatusCode, Result<T>,
// MakeUnexpected, Ok).
#pragma once

#include <cstdint>
#include <optional>
#include <string>
#include <utility>

namespace sci {

enum class StatusCode : int32_t {
    kOk = 0,
    kError = 1,
    kNotFound = 2,
    kInvalidArgument = 4,
    kNotImplemented = 5,
    kOutOfMemory = 6,
    kResourceExhausted = 7,
    kInvalidOperation = 10,
    kInternal = 12,
    kCudaError = 100,
    kCudaNotAvailable = 101,
    kCudaOutOfMemory = 102,
    kDeviceError = 500,
};

constexpr const char* StatusCodeToString(StatusCode code) {
    switch (code) {
        case StatusCode::kOk: return "OK";
        case StatusCode::kError: return "Error";
        case StatusCode::kNotFound: return "Not Found";
        case StatusCode::kInvalidArgument: return "Invalid Argument";
        case StatusCode::kNotImplemented: return "Not Implemented";
        case StatusCode::kOutOfMemory: return "Out of Memory";
        case StatusCode::kResourceExhausted: return "Resource Exhausted";
        case StatusCode::kInvalidOperation: return "Invalid Operation";
        case StatusCode::kInternal: return "Internal Error";
        case StatusCode::kCudaError: return "CUDA Error";
        case StatusCode::kCudaNotAvailable: return "CUDA Not Available";
        case StatusCode::kCudaOutOfMemory: return "CUDA Out of Memory";
        case StatusCode::kDeviceError: return "Device Error";
    }
    return "Unknown";
}

class Status {
public:
    Status() = default;
    Status(StatusCode code, std::string message = {}) : code_(code), message_(std::move(message)) {}

    static Status Ok() { return {}; }
    static Status Error(const std::string& m = "Unknown error") { return {StatusCode::kError, m}; }
    static Status InvalidArgument(const std::string& m = "Invalid argument") { return {StatusCode::kInvalidArgument, m}; }
    static Status NotImplemented(const std::string& m = "Not implemented") { return {StatusCode::kNotImplemented, m}; }
    static Status InvalidOperation(const std::string& m = "Invalid operation") { return {StatusCode::kInvalidOperation, m}; }
    static Status OutOfMemory(const std::string& m = "Out of memory") { return {StatusCode::kOutOfMemory, m}; }
    static Status CudaError(const std::string& m = "CUDA error") { return {StatusCode::kCudaError, m}; }
    static Status CudaNotAvailable(const std::string& m = "CUDA not available") { return {StatusCode::kCudaNotAvailable, m}; }
    static Status CudaOutOfMemory(const std::string& m = "CUDA out of memory") { return {StatusCode::kCudaOutOfMemory, m}; }

    bool ok() const { return code_ == StatusCode::kOk; }
    explicit operator bool() const { return ok(); }
    StatusCode code() const { return code_; }
    const std::string& message() const { return message_; }
    bool operator==(const Status& other) const { return code_ == other.code_; }
    bool operator!=(const Status& other) const { return code_ != other.code_; }
    std::string ToString() const { return ok() ? "OK" : std::string(StatusCodeToString(code_)) + ": " + message_; }

private:
    StatusCode code_{StatusCode::kOk};
    std::string message_;
};

struct Unexpected {
    explicit Unexpected(Status s) : error_(std::move(s)) {}
    const Status& error() const { return error_; }
    Status error_;
};

// Value-or-Status. A default-constructed Expected holds a default-constructed T.
template <typename T>
class Expected {
public:
    Expected() : value_(std::in_place) {}
    explicit Expected(T value) : value_(std::move(value)) {}
    explicit Expected(Unexpected u) : error_(std::move(u.error_)) {}

    bool ok() const noexcept { return value_.has_value(); }
    explicit operator bool() const noexcept { return ok(); }
    T& value() & { return *value_; }
    const T& value() const& { return *value_; }
    T* operator->() { return &*value_; }
    const T* operator->() const { return &*value_; }
    T& operator*() { return *value_; }
    const T& operator*() const { return *value_; }
    Status error() const { return ok() ? Status::Ok() : error_; }
    const std::string& message() const {
        static const std::string kEmpty;
        return ok() ? kEmpty : error_.message();
    }

private:
    std::optional<T> value_;
    Status error_;
};

template <typename T>
using Result = Expected<T>;

template <typename T>
Expected<T> MakeUnexpected(Status s) {
    return Expected<T>(Unexpected(std::move(s)));
}

template <typename T>
Result<T> Ok(T value) {
    return Result<T>(std::move(value));
}

}  // namespace sci
