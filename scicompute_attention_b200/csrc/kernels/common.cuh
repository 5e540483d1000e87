// Shared device/host helpers for the sm_100a kernels: error reporting behind the C ABI, 16-byte
// async copies, warp-level tensor-core wrappers used by the bandwidth kernels, and softmax math.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstdint>
#include <string>

#include "sca_b200.h"

namespace sca_b200 {

// ---- error plumbing (host) --------------------------------------------------------------------
// Stores the message for sca_last_error() and returns `code` so call sites can `return Fail(...)`.
int Fail(int code, const std::string& message);
void ClearError();
// Maps a cudaError_t to SCA_CUDA_ERROR / SCA_CUDA_OOM with "<what>: <cudaGetErrorName>: <string>".
int FailCuda(cudaError_t err, const char* what);
// cudaGetLastError() right after a launch (reference behaviour: src/runtime/launcher.cu:94-100);
// honours SCI_ATTENTION_DEBUG_SYNC=1 by synchronising the stream and reporting the async error.
int CheckLaunch(const char* kernel_name, cudaStream_t stream);
// True when SCI_ATTENTION_DEBUG_SYNC=1 (CheckLaunch then synchronises the stream after every launch).
bool DebugSyncEnabled();
// Opt-in to > 48 KiB of dynamic shared memory once per kernel symbol.
int EnsureDynamicSmem(const void* kernel, size_t bytes, const char* kernel_name);
// Cached SM count of the current device.
int SmCount();

inline bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- device helpers -----------------------------------------------------------------------------
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t SmemAddr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte global->shared async copy; src_bytes == 0 zero-fills the destination without reading.
__device__ __forceinline__ void CpAsync16(uint32_t smem_dst, const void* gmem_src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_dst), "l"(gmem_src),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void CpAsyncWait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint4 LdsV4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// D(16x8, f32) += A(16x16) * B(16x8); A row-major, B column-major fragments, 16-bit inputs.
template <typename T>
__device__ __forceinline__ void MmaM16N8K16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void MmaM16N8K16<__half>(float (&c)[4], uint32_t a0, uint32_t a1,
                                                    uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void MmaM16N8K16<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1,
                                                           uint32_t a2, uint32_t a3, uint32_t b0,
                                                           uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Packs two floats into one 32-bit register of 16-bit values (lo in bits 0..15), round-to-nearest.
template <typename T>
__device__ __forceinline__ uint32_t Pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t Pack2<__half>(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t Pack2<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ float Exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float ToFloat(float v) { return v; }
__device__ __forceinline__ float ToFloat(__half v) { return __half2float(v); }
__device__ __forceinline__ float ToFloat(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T FromFloat(float v);
template <>
__device__ __forceinline__ float FromFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half FromFloat<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 FromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

}  // namespace sca_b200
