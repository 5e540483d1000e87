// Sequence-split decode, cross-GPU step: merge of this GPU's split-K partials, exchange of the merged
// (m, l, O[D]) triples with every peer over NVLink, and the final merge - in ONE kernel, with no
// library collective between the steps.
//
// The reference is single-GPU (its split-K merge is src/backends/decode/decode_splitk.cu:143-182); this
// applies the same max-rescaled merge rule twice: over the local splits, then over the ranks.
//
// Every rank owns one exchange buffer and maps the buffers of all peers (CUDA IPC handles, plain peer
// stores and loads; no multimem, no TMA). Layout of a buffer, identical on all ranks:
//     [0, 256)    uint32 flags[64]    flags[s] = last epoch whose triples rank s has fully pushed here
//     [256, 260)  uint32 arrived      CTAs of the running kernel that have finished pushing
//     [260, 264)  int32  status       0, or 1 after a wait for a peer gave up
//     [264, 268)  uint32 epoch        epochs completed, when the kernel keeps the count itself (params.epoch == 0)
//     [512, ...)  float  data[2][world][rows][2 + D]     (two epochs in turn)
// Per launch (epoch e, parity e & 1) a CTA
//   1. merges the local splits of its rows and stores the triples into data[parity][rank] of EVERY rank;
//   2. fences system-wide and counts itself in `arrived`; the last CTA to do so publishes the epoch in
//      flags[rank] of every rank (release);
//   3. waits (bounded) until the local flags of all ranks show the epoch (acquire), and
//   4. merges data[parity][0 .. world) of its rows into the normalised output.
// The grid never exceeds what is co-resident on the GPU, so step 3 cannot starve step 1 of another CTA.
// A buffer half is overwritten two epochs later; a peer can only be two epochs ahead after this rank has
// published the epoch in between, which it does after finishing step 4 of the older one (stream order).
#include <algorithm>
#include <string>

#include "common.cuh"
#include "sca_b200.h"

namespace sca_b200 {
namespace {

constexpr int kHeaderBytes = 512;
constexpr int kFlagsOffset = 0;      // uint32[64]
constexpr int kArrivedOffset = 256;  // uint32
constexpr int kStatusOffset = 260;   // int32
constexpr int kEpochOffset = 264;    // uint32
constexpr int kMaxRanks = SCA_PEER_MAX_RANKS;
constexpr long long kPeerWaitCycles = 2000000000LL;  // about a second: far beyond any legitimate skew inside a step

struct ExchangeParams {
    unsigned char* peer[kMaxRanks];
    int rank, world;
    int rows, head_dim, splits;
    unsigned epoch;
    const float* partial_m;
    const float* partial_l;
    const float* partial_o;
    void* out;
};

__device__ __forceinline__ unsigned LoadAcquireSys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void StoreReleaseSys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(128)
seqsplit_exchange_kernel(const ExchangeParams p) {
    constexpr int kCols = 2;     // head-dim columns per thread: d = threadIdx.x + 128 c, head_dim <= 256
    const int width = 2 + p.head_dim;
    const size_t half_floats = static_cast<size_t>(p.world) * p.rows * width;
    unsigned char* local = p.peer[p.rank];
    __shared__ int s_ok;
    __shared__ unsigned s_epoch;
    // launched with programmatic stream serialisation behind the split-K partial kernel: blocks may be resident
    // early; nothing is read before that grid has completed (a no-op after an ordinary launch)
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // The epoch is either given by the host or counted in the buffer header, which makes the launch parameters
    // identical from step to step (a captured graph can then replay the step). Every CTA reads the count before it
    // counts itself in `arrived`; the last CTA to arrive advances it, so no CTA can see the new value too early.
    if (threadIdx.x == 0) {
        s_epoch = p.epoch != 0 ? p.epoch : *reinterpret_cast<volatile unsigned*>(local + kEpochOffset) + 1u;
    }
    __syncthreads();
    const unsigned epoch = s_epoch;
    const size_t slot = (epoch & 1u) * half_floats;

    // 1. local splits -> one triple per row, stored into every rank's buffer
    for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const float* m = p.partial_m + static_cast<size_t>(row) * p.splits;
        const float* l = p.partial_l + static_cast<size_t>(row) * p.splits;
        float m_all = -CUDART_INF_F;
        for (int s = 0; s < p.splits; ++s) m_all = fmaxf(m_all, m[s]);
        float l_all = 0.0f, acc[kCols] = {0.0f, 0.0f};
        for (int s = 0; s < p.splits; ++s) {
            const float ms = m[s];
            if (ms == -CUDART_INF_F) continue;
            const float wgt = Exp2((ms - m_all) * kLog2e);
            l_all += l[s] * wgt;
            const float* o = p.partial_o + (static_cast<size_t>(row) * p.splits + s) * p.head_dim;
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                const int d = threadIdx.x + 128 * c;
                if (d < p.head_dim) acc[c] += o[d] * wgt;
            }
        }
        const size_t at = slot + (static_cast<size_t>(p.rank) * p.rows + row) * width;
        for (int r = 0; r < p.world; ++r) {
            float* dst = reinterpret_cast<float*>(p.peer[r] + kHeaderBytes) + at;
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                const int d = threadIdx.x + 128 * c;
                if (d < p.head_dim) dst[2 + d] = acc[c];
            }
            if (threadIdx.x == 0) {
                dst[0] = m_all;
                dst[1] = l_all;
            }
        }
    }

    // 2. publish: every CTA's stores are ordered before its count; the last CTA raises the flags
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* arrived = reinterpret_cast<unsigned*>(local + kArrivedOffset);
        const unsigned before = atomicAdd(arrived, 1u);
        if (before == gridDim.x - 1) {
            *arrived = 0;  // ready for the next launch (same stream)
            *reinterpret_cast<unsigned*>(local + kEpochOffset) = epoch;
            __threadfence_system();
            for (int r = 0; r < p.world; ++r) {
                StoreReleaseSys(reinterpret_cast<unsigned*>(p.peer[r] + kFlagsOffset) + p.rank, epoch);
            }
        }
        // 3. bounded wait for every rank's epoch
        const unsigned* flags = reinterpret_cast<const unsigned*>(local + kFlagsOffset);
        int ok = 1;
        const long long start = clock64();
        for (int s = 0; s < p.world && ok; ++s) {
            while (static_cast<int>(LoadAcquireSys(flags + s) - epoch) < 0) {
                if (clock64() - start > kPeerWaitCycles) {
                    ok = 0;
                    // remember the first step that gave up (the epoch; never 0) until the host clears it
                    atomicCAS(reinterpret_cast<int*>(local + kStatusOffset), 0, static_cast<int>(epoch));
                    break;
                }
                __nanosleep(64);
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) {
        // a peer did not show up: this launch has no result. The rows this CTA owns are filled with NaN so that stale
        // values of an earlier step cannot pass as an answer; the host learns the step from the status word.
        for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                const int d = threadIdx.x + 128 * c;
                if (d < p.head_dim) reinterpret_cast<T*>(p.out)[static_cast<size_t>(row) * p.head_dim + d] = FromFloat<T>(CUDART_NAN_F);
            }
        }
        return;
    }

    // 4. merge over ranks
    const float* data = reinterpret_cast<const float*>(local + kHeaderBytes) + slot;
    for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
        float m_all = -CUDART_INF_F;
        for (int s = 0; s < p.world; ++s) {
            m_all = fmaxf(m_all, __ldcg(data + (static_cast<size_t>(s) * p.rows + row) * width));
        }
        float l_all = 0.0f, acc[kCols] = {0.0f, 0.0f};
        for (int s = 0; s < p.world; ++s) {
            const float* t = data + (static_cast<size_t>(s) * p.rows + row) * width;
            const float ms = __ldcg(t);
            if (ms == -CUDART_INF_F) continue;
            const float wgt = Exp2((ms - m_all) * kLog2e);
            l_all += __ldcg(t + 1) * wgt;
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                const int d = threadIdx.x + 128 * c;
                if (d < p.head_dim) acc[c] += __ldcg(t + 2 + d) * wgt;
            }
        }
        const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
            const int d = threadIdx.x + 128 * c;
            if (d < p.head_dim) reinterpret_cast<T*>(p.out)[static_cast<size_t>(row) * p.head_dim + d] = FromFloat<T>(acc[c] * inv);
        }
    }
}

}  // namespace
}  // namespace sca_b200

using namespace sca_b200;

extern "C" long long sca_peer_buffer_bytes(int32_t world, int64_t rows, int64_t head_dim) {
    if (world < 1 || world > kMaxRanks || rows < 1 || head_dim < 1) return -1;
    return kHeaderBytes + 2LL * world * rows * (2 + head_dim) * 4;
}

extern "C" int sca_peer_buffer_create(int64_t bytes, void** device_ptr, unsigned char* handle_out) {
    ClearError();
    if (bytes < kHeaderBytes || device_ptr == nullptr || handle_out == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "peer buffer: invalid size or null output");
    }
    void* ptr = nullptr;
    if (cudaError_t e = cudaMalloc(&ptr, static_cast<size_t>(bytes)); e != cudaSuccess) return FailCuda(e, "cudaMalloc(peer buffer)");
    if (cudaError_t e = cudaMemset(ptr, 0, static_cast<size_t>(bytes)); e != cudaSuccess) {
        cudaFree(ptr);
        return FailCuda(e, "cudaMemset(peer buffer)");
    }
    cudaIpcMemHandle_t handle;
    if (cudaError_t e = cudaIpcGetMemHandle(&handle, ptr); e != cudaSuccess) {
        cudaFree(ptr);
        return FailCuda(e, "cudaIpcGetMemHandle");
    }
    static_assert(sizeof(handle) == SCA_PEER_HANDLE_BYTES, "IPC handle size");
    std::copy_n(reinterpret_cast<const unsigned char*>(&handle), sizeof(handle), handle_out);
    *device_ptr = ptr;
    return SCA_OK;
}

extern "C" int sca_peer_buffer_open(const unsigned char* handle_in, void** device_ptr) {
    ClearError();
    if (handle_in == nullptr || device_ptr == nullptr) return Fail(SCA_INVALID_ARGUMENT, "peer buffer: null handle");
    cudaIpcMemHandle_t handle;
    std::copy_n(handle_in, sizeof(handle), reinterpret_cast<unsigned char*>(&handle));
    void* ptr = nullptr;
    if (cudaError_t e = cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess); e != cudaSuccess) {
        return FailCuda(e, "cudaIpcOpenMemHandle");
    }
    *device_ptr = ptr;
    return SCA_OK;
}

extern "C" int sca_peer_buffer_close(void* device_ptr) {
    ClearError();
    if (device_ptr == nullptr) return SCA_OK;
    if (cudaError_t e = cudaIpcCloseMemHandle(device_ptr); e != cudaSuccess) return FailCuda(e, "cudaIpcCloseMemHandle");
    return SCA_OK;
}

extern "C" int sca_peer_buffer_destroy(void* device_ptr) {
    ClearError();
    if (device_ptr == nullptr) return SCA_OK;
    if (cudaError_t e = cudaFree(device_ptr); e != cudaSuccess) return FailCuda(e, "cudaFree(peer buffer)");
    return SCA_OK;
}

extern "C" int sca_peer_exchange_status(const void* local_buffer, int32_t* status_out) {
    ClearError();
    if (local_buffer == nullptr || status_out == nullptr) return Fail(SCA_INVALID_ARGUMENT, "peer status: null pointer");
    int value = 0;
    if (cudaError_t e = cudaMemcpy(&value, static_cast<const unsigned char*>(local_buffer) + kStatusOffset, sizeof(int),
                                   cudaMemcpyDeviceToHost);
        e != cudaSuccess) {
        return FailCuda(e, "cudaMemcpy(peer status)");
    }
    *status_out = value;
    return SCA_OK;
}

extern "C" int sca_peer_exchange_clear(void* local_buffer) {
    ClearError();
    if (local_buffer == nullptr) return Fail(SCA_INVALID_ARGUMENT, "peer status: null pointer");
    if (cudaError_t e = cudaMemset(static_cast<unsigned char*>(local_buffer) + kStatusOffset, 0, sizeof(int)); e != cudaSuccess) {
        return FailCuda(e, "cudaMemset(peer status)");
    }
    return SCA_OK;
}

extern "C" int sca_launch_seqsplit_exchange(const ScaSeqSplitExchange* params, void* stream) {
    ClearError();
    if (params == nullptr) return Fail(SCA_INVALID_ARGUMENT, "sequence-split exchange: null parameter block");
    const ScaSeqSplitExchange& x = *params;
    if (x.world < 1 || x.world > kMaxRanks || x.rank < 0 || x.rank >= x.world) {
        return Fail(SCA_INVALID_ARGUMENT, "sequence-split exchange: rank/world out of range (at most " +
                                              std::to_string(kMaxRanks) + " ranks)");
    }
    if (x.rows < 1 || x.rows > 0x7fffffffLL || x.head_dim < 1 || x.head_dim > 256 || x.num_splits < 1) {
        return Fail(SCA_INVALID_ARGUMENT, "sequence-split exchange: rows/head_dim/num_splits out of range (head_dim <= 256)");
    }
    if (x.partial_m == nullptr || x.partial_l == nullptr || x.partial_o == nullptr || x.out == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "sequence-split exchange: null tensor pointer");
    }
    ExchangeParams p{};
    for (int r = 0; r < x.world; ++r) {
        if (x.peer_buffers[r] == nullptr) return Fail(SCA_INVALID_ARGUMENT, "sequence-split exchange: null peer buffer");
        p.peer[r] = static_cast<unsigned char*>(x.peer_buffers[r]);
    }
    p.rank = x.rank;
    p.world = x.world;
    p.rows = static_cast<int>(x.rows);
    p.head_dim = static_cast<int>(x.head_dim);
    p.splits = static_cast<int>(x.num_splits);
    p.epoch = x.epoch;
    p.partial_m = x.partial_m;
    p.partial_l = x.partial_l;
    p.partial_o = x.partial_o;
    p.out = x.out;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // co-resident by construction: at most two 128-thread CTAs per SM
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(x.rows, 2LL * SmCount()));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(128);
    cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    switch (x.out_dtype) {
        case SCA_DTYPE_F16: cudaLaunchKernelEx(&cfg, seqsplit_exchange_kernel<__half>, p); break;
        case SCA_DTYPE_BF16: cudaLaunchKernelEx(&cfg, seqsplit_exchange_kernel<__nv_bfloat16>, p); break;
        case SCA_DTYPE_F32: cudaLaunchKernelEx(&cfg, seqsplit_exchange_kernel<float>, p); break;
        default: return Fail(SCA_INVALID_ARGUMENT, "sequence-split exchange: unsupported dtype id");
    }
    return CheckLaunch("seqsplit_exchange_kernel", s);
}
