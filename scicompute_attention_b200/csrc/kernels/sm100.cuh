// Thin inline-PTX layer for the Blackwell (sm_100a) async machinery used by the prefill kernel:
// mbarriers with bounded waits, TMA tensor loads, tensor-memory (TMEM) allocation and access, and
// tcgen05.mma with shared-memory / tensor-memory operands. Replaces the reference's sm_80 wrappers
// (src/cuda_common/mma_policy.cuh, ldmatrix.cuh, cp_async.cuh).
#pragma once

#include <cuda.h>

#include <cstdint>

namespace sca_b200 {
namespace sm100 {

// ---- mbarrier ------------------------------------------------------------------------------------
__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void FenceBarrierInit() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA / tcgen05 operands).
__device__ __forceinline__ void FenceProxyAsync() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void MbarArrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One probe of the barrier. The hint lets the hardware park the thread for up to that many nanoseconds
// instead of returning at once, so that a waiting warp does not take issue slots from the warps that work.
constexpr uint32_t kTryWaitHintNs = 20000;
__device__ __forceinline__ bool MbarTryWait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(kTryWaitHintNs)
        : "memory");
    return done != 0;
}

// About two seconds at 2 GHz: far beyond any legitimate wait inside one attention tile.
constexpr long long kWaitLimitCycles = 4000000000LL;

// Waits for the phase with the given parity. Never spins forever: gives up when the CTA-wide abort
// flag is raised by another role or when the cycle budget is spent (and raises the flag itself).
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
        if (MbarTryWait(bar, parity)) return true;
    }
    const long long start = clock64();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (MbarTryWait(bar, parity)) return true;
        }
        if (*abort_flag != 0) return false;
        if (clock64() - start > kWaitLimitCycles) {
            *abort_flag = 1;
            return false;
        }
    }
}

// ---- TMA -------------------------------------------------------------------------------------------
__device__ __forceinline__ void PrefetchTensorMap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// 4-D tiled load global -> shared of this CTA; completion is counted in bytes on `bar`.
__device__ __forceinline__ void TmaLoad4D(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int c0,
                                          int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// ---- tensor memory -----------------------------------------------------------------------------------
__device__ __forceinline__ void TmemAlloc(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void TmemRelinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TmemWaitLd() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemWaitSt() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Each thread of the warp reads 32 consecutive 32-bit columns of its own TMEM lane
// (lane = 32 * (warp % 4) + laneid; the lane base travels in bits 16.. of `taddr`).
__device__ __forceinline__ void TmemLd32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void TmemSt32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// ---- tcgen05.mma (dense f16/bf16 inputs, f32 accumulate, one CTA) -----------------------------------
enum : uint32_t { kFmtF16 = 0, kFmtBf16 = 1 };

// Instruction descriptor: D = f32, A and B formats (each f16 or bf16, independently), operand majors
// (0 = K-major, 1 = MN-major), N, M.
__host__ __device__ constexpr uint32_t MakeInstrDesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn_major,
                                                     uint32_t b_mn_major, uint32_t m, uint32_t n) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
           ((m >> 4) << 24);
}

// Shared-memory matrix descriptor for a 128-byte-swizzled tile (tile base 1024-byte aligned):
// start address, leading / stride byte offsets (all >> 4), descriptor version 1, swizzle mode 2.
__device__ __forceinline__ uint64_t MakeSmemDesc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) |
           (static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

// D[tmem] (+)= A[smem] * B[smem]; kAccumulate == false overwrites D.
template <bool kAccumulate>
__device__ __forceinline__ void MmaSS(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
template <bool kAccumulate>
__device__ __forceinline__ void MmaTS(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
// Same with the accumulate flag decided at run time.
__device__ __forceinline__ void MmaTSFlag(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void MmaCommit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace sm100
}  // namespace sca_b200
