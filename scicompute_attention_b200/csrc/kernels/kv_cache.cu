// KV-cache data movement over the block-major pool [num_blocks][block_size][kv_heads][D]:
// scatter-append, block reset and block gather.
//
// Stands in for kv_append_kernel / kv_reset_kernel / kv_gather_kernel
// (src/kv_cache/kv_cache_kernels.cu:17-86), which move one byte per thread (reset, gather) or one
// whole row per thread in a byte loop (append). Here every thread moves 16 bytes, consecutive
// threads touch consecutive 16-byte chunks of the same row (fully coalesced 128-byte lines), and K
// and V are handled in the same pass. Addressing follows src/kv_cache/kv_cache_layout.cuh:32-38.
// Rows whose byte length or base addresses are not 16-byte multiples fall back to a byte loop so
// the result is bit-exact for any geometry.
//
// Algorithmic traffic: append = 2 * tokens * kv_heads * D * elem bytes read + the same written;
// reset = 2 * blocks * block_bytes written; gather = blocks * block_bytes read + written.
#include <algorithm>

#include "common.cuh"

namespace sca_b200 {
namespace {

constexpr int kKvThreads = 256;

template <typename V>
__global__ void __launch_bounds__(kKvThreads)
kv_append_kernel(V* __restrict__ layer_k, V* __restrict__ layer_v, const V* __restrict__ k_new,
                 const V* __restrict__ v_new, const int32_t* __restrict__ slots,
                 const int64_t num_tokens, const ScaKvCacheShape shape, const int64_t token_vecs) {
    // token_vecs = kv_heads * D * elem_bytes / sizeof(V): one token's K (or V) payload is contiguous
    // both in the source [token][head][D] and in the pool [slot][head][D].
    const int64_t total = num_tokens * token_vecs;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t token = idx / token_vecs;
        const int64_t within = idx % token_vecs;
        const int32_t slot = __ldg(slots + token);
        if (slot < 0) continue;                                  // "do not store" sentinel
        if (slot / shape.block_size >= shape.num_blocks) continue;  // never write out of range
        const int64_t dst = static_cast<int64_t>(slot) * token_vecs + within;
        layer_k[dst] = k_new[idx];
        layer_v[dst] = v_new[idx];
    }
}

// Same scatter with the slot computed on the device from the page table: one new token per
// sequence at position seq_lens[s] - 1.
template <typename V>
__global__ void __launch_bounds__(kKvThreads)
kv_append_batched_kernel(V* __restrict__ layer_k, V* __restrict__ layer_v, const V* __restrict__ k_new,
                         const V* __restrict__ v_new, const int32_t* __restrict__ page_table,
                         const int32_t* __restrict__ seq_lens, const int64_t num_seqs,
                         const int64_t max_blocks_per_seq, const ScaKvCacheShape shape,
                         const int64_t token_vecs) {
    const int64_t total = num_seqs * token_vecs;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t seq = idx / token_vecs;
        const int64_t within = idx % token_vecs;
        const int64_t pos = static_cast<int64_t>(__ldg(seq_lens + seq)) - 1;
        if (pos < 0) continue;
        const int64_t logical = pos / shape.block_size;
        if (logical >= max_blocks_per_seq) continue;
        const int32_t phys = __ldg(page_table + seq * max_blocks_per_seq + logical);
        if (phys < 0 || phys >= shape.num_blocks) continue;
        const int64_t slot = static_cast<int64_t>(phys) * shape.block_size + pos % shape.block_size;
        const int64_t dst = slot * token_vecs + within;
        layer_k[dst] = k_new[idx];
        layer_v[dst] = v_new[idx];
    }
}

template <typename V>
__global__ void __launch_bounds__(kKvThreads)
kv_reset_kernel(V* __restrict__ layer_k, V* __restrict__ layer_v, const int32_t* __restrict__ ids,
                const int64_t count, const int64_t num_blocks, const int64_t block_vecs) {
    const int64_t total = count * block_vecs;
    V zero;
    memset(&zero, 0, sizeof(V));
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int32_t phys = __ldg(ids + idx / block_vecs);
        if (phys < 0 || phys >= num_blocks) continue;
        const int64_t dst = static_cast<int64_t>(phys) * block_vecs + idx % block_vecs;
        layer_k[dst] = zero;
        layer_v[dst] = zero;
    }
}

template <typename V>
__global__ void __launch_bounds__(kKvThreads)
kv_gather_kernel(const V* __restrict__ layer, const int32_t* __restrict__ ids, const int64_t count,
                 V* __restrict__ out, const int64_t num_blocks, const int64_t block_vecs) {
    const int64_t total = count * block_vecs;
    V zero;
    memset(&zero, 0, sizeof(V));
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int32_t phys = __ldg(ids + idx / block_vecs);
        out[idx] = (phys < 0 || phys >= num_blocks)
                       ? zero
                       : layer[static_cast<int64_t>(phys) * block_vecs + idx % block_vecs];
    }
}

unsigned GridFor(int64_t items) {
    // enough CTAs to cover the work once, capped at a few waves of the machine: the loops are
    // grid-stride, and HBM is saturated long before more CTAs would help
    const int64_t want = (items + kKvThreads - 1) / kKvThreads;
    const int64_t cap = static_cast<int64_t>(SmCount()) * 32;
    return static_cast<unsigned>(std::max<int64_t>(1, std::min(want, cap)));
}

int CheckShape(const ScaKvCacheShape* shape, int64_t elem_bytes, const char* what) {
    if (shape == nullptr) return Fail(SCA_INVALID_ARGUMENT, std::string(what) + ": null shape");
    if (shape->num_blocks <= 0 || shape->block_size <= 0 || shape->num_kv_heads <= 0 ||
        shape->head_dim <= 0 || elem_bytes <= 0) {
        return Fail(SCA_INVALID_ARGUMENT, std::string(what) + ": non-positive geometry");
    }
    return SCA_OK;
}

// Block-id lists are documented as device memory, but the reference's own PagedKVCache::ResetSeq hands
// KVCache::Reset the ids straight out of a std::vector (src/kv_cache/paged_kv_cache.cpp:150-156), which only
// works where the GPU can read pageable host memory. A list that lives in host memory is therefore copied into
// a stream-ordered temporary first (the copy out of pageable memory completes before the call returns, so the
// caller may drop its vector right away); device and managed pointers are used as they are.
class StagedIds {
public:
    StagedIds() = default;
    StagedIds(const StagedIds&) = delete;
    StagedIds& operator=(const StagedIds&) = delete;
    ~StagedIds() {
        if (staged_ != nullptr && cudaFreeAsync(staged_, stream_) != cudaSuccess) cudaGetLastError();
    }
    int Stage(const int32_t* ids, int64_t count, cudaStream_t stream, const char* what) {
        ids_ = ids;
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, ids) != cudaSuccess) {
            cudaGetLastError();
            return SCA_OK;  // no usable device: the launch below reports it
        }
        if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) return SCA_OK;
        if (attr.type == cudaMemoryTypeHost && attr.devicePointer != nullptr) {
            ids_ = static_cast<const int32_t*>(attr.devicePointer);  // pinned and mapped: readable in place
            return SCA_OK;
        }
        const size_t bytes = static_cast<size_t>(count) * sizeof(int32_t);
        stream_ = stream;
        cudaError_t err = cudaMallocAsync(reinterpret_cast<void**>(&staged_), bytes, stream);
        if (err != cudaSuccess) {
            staged_ = nullptr;
            cudaGetLastError();
            return FailCuda(err, what);
        }
        err = cudaMemcpyAsync(staged_, ids, bytes, cudaMemcpyHostToDevice, stream);
        if (err != cudaSuccess) {
            cudaGetLastError();
            return FailCuda(err, what);
        }
        ids_ = staged_;
        return SCA_OK;
    }
    const int32_t* get() const { return ids_; }

private:
    const int32_t* ids_{nullptr};
    int32_t* staged_{nullptr};
    cudaStream_t stream_{nullptr};
};

}  // namespace
}  // namespace sca_b200

using namespace sca_b200;

extern "C" int sca_launch_kv_append(void* layer_k, void* layer_v, const void* k_new, const void* v_new,
                                    const int32_t* slot_mapping, int64_t num_tokens,
                                    const ScaKvCacheShape* shape, int64_t elem_bytes, void* stream) {
    ClearError();
    if (layer_k == nullptr || layer_v == nullptr || k_new == nullptr || v_new == nullptr ||
        slot_mapping == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "kv append: null pointer");
    }
    if (num_tokens <= 0) return Fail(SCA_INVALID_ARGUMENT, "kv append: num_tokens <= 0");
    if (int rc = CheckShape(shape, elem_bytes, "kv append")) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t token_bytes = shape->num_kv_heads * shape->head_dim * elem_bytes;
    const bool vec = token_bytes % 16 == 0 && Aligned16(layer_k) && Aligned16(layer_v) &&
                     Aligned16(k_new) && Aligned16(v_new);
    if (vec) {
        const int64_t tv = token_bytes / 16;
        kv_append_kernel<uint4><<<GridFor(num_tokens * tv), kKvThreads, 0, s>>>(
            static_cast<uint4*>(layer_k), static_cast<uint4*>(layer_v), static_cast<const uint4*>(k_new),
            static_cast<const uint4*>(v_new), slot_mapping, num_tokens, *shape, tv);
    } else {
        kv_append_kernel<unsigned char><<<GridFor(num_tokens * token_bytes), kKvThreads, 0, s>>>(
            static_cast<unsigned char*>(layer_k), static_cast<unsigned char*>(layer_v),
            static_cast<const unsigned char*>(k_new), static_cast<const unsigned char*>(v_new),
            slot_mapping, num_tokens, *shape, token_bytes);
    }
    return CheckLaunch("kv_append_kernel", s);
}

extern "C" int sca_launch_kv_append_batched(void* layer_k, void* layer_v, const void* k_new,
                                            const void* v_new, const int32_t* page_table,
                                            const int32_t* seq_lens, int64_t num_seqs,
                                            int64_t max_blocks_per_seq, const ScaKvCacheShape* shape,
                                            int64_t elem_bytes, void* stream) {
    ClearError();
    if (layer_k == nullptr || layer_v == nullptr || k_new == nullptr || v_new == nullptr ||
        page_table == nullptr || seq_lens == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "kv append (batched): null pointer");
    }
    if (num_seqs <= 0 || max_blocks_per_seq <= 0) {
        return Fail(SCA_INVALID_ARGUMENT, "kv append (batched): num_seqs/max_blocks_per_seq <= 0");
    }
    if (int rc = CheckShape(shape, elem_bytes, "kv append (batched)")) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t token_bytes = shape->num_kv_heads * shape->head_dim * elem_bytes;
    const bool vec = token_bytes % 16 == 0 && Aligned16(layer_k) && Aligned16(layer_v) &&
                     Aligned16(k_new) && Aligned16(v_new);
    if (vec) {
        const int64_t tv = token_bytes / 16;
        kv_append_batched_kernel<uint4><<<GridFor(num_seqs * tv), kKvThreads, 0, s>>>(
            static_cast<uint4*>(layer_k), static_cast<uint4*>(layer_v), static_cast<const uint4*>(k_new),
            static_cast<const uint4*>(v_new), page_table, seq_lens, num_seqs, max_blocks_per_seq, *shape, tv);
    } else {
        kv_append_batched_kernel<unsigned char><<<GridFor(num_seqs * token_bytes), kKvThreads, 0, s>>>(
            static_cast<unsigned char*>(layer_k), static_cast<unsigned char*>(layer_v),
            static_cast<const unsigned char*>(k_new), static_cast<const unsigned char*>(v_new), page_table,
            seq_lens, num_seqs, max_blocks_per_seq, *shape, token_bytes);
    }
    return CheckLaunch("kv_append_batched_kernel", s);
}

extern "C" int sca_launch_kv_reset_block(void* layer_k, void* layer_v, const int32_t* block_ids,
                                         int64_t num_blocks, const ScaKvCacheShape* shape,
                                         int64_t elem_bytes, void* stream) {
    ClearError();
    if (layer_k == nullptr || layer_v == nullptr || block_ids == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "kv reset: null pointer");
    }
    if (num_blocks <= 0) return SCA_OK;
    if (int rc = CheckShape(shape, elem_bytes, "kv reset")) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StagedIds ids;
    if (int rc = ids.Stage(block_ids, num_blocks, s, "kv reset: staging host block ids")) return rc;
    block_ids = ids.get();
    const int64_t block_bytes = shape->block_size * shape->num_kv_heads * shape->head_dim * elem_bytes;
    if (block_bytes % 16 == 0 && Aligned16(layer_k) && Aligned16(layer_v)) {
        const int64_t bv = block_bytes / 16;
        kv_reset_kernel<uint4><<<GridFor(num_blocks * bv), kKvThreads, 0, s>>>(
            static_cast<uint4*>(layer_k), static_cast<uint4*>(layer_v), block_ids, num_blocks,
            shape->num_blocks, bv);
    } else {
        kv_reset_kernel<unsigned char><<<GridFor(num_blocks * block_bytes), kKvThreads, 0, s>>>(
            static_cast<unsigned char*>(layer_k), static_cast<unsigned char*>(layer_v), block_ids,
            num_blocks, shape->num_blocks, block_bytes);
    }
    return CheckLaunch("kv_reset_kernel", s);
}

extern "C" int sca_launch_kv_gather(const void* layer, const int32_t* block_ids, int64_t num_blocks,
                                    void* out, const ScaKvCacheShape* shape, int64_t elem_bytes,
                                    void* stream) {
    ClearError();
    if (layer == nullptr || block_ids == nullptr || out == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "kv gather: null pointer");
    }
    if (num_blocks <= 0) return SCA_OK;
    if (int rc = CheckShape(shape, elem_bytes, "kv gather")) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    StagedIds ids;
    if (int rc = ids.Stage(block_ids, num_blocks, s, "kv gather: staging host block ids")) return rc;
    block_ids = ids.get();
    const int64_t block_bytes = shape->block_size * shape->num_kv_heads * shape->head_dim * elem_bytes;
    if (block_bytes % 16 == 0 && Aligned16(layer) && Aligned16(out)) {
        const int64_t bv = block_bytes / 16;
        kv_gather_kernel<uint4><<<GridFor(num_blocks * bv), kKvThreads, 0, s>>>(
            static_cast<const uint4*>(layer), block_ids, num_blocks, static_cast<uint4*>(out),
            shape->num_blocks, bv);
    } else {
        kv_gather_kernel<unsigned char><<<GridFor(num_blocks * block_bytes), kKvThreads, 0, s>>>(
            static_cast<const unsigned char*>(layer), block_ids, num_blocks,
            static_cast<unsigned char*>(out), shape->num_blocks, block_bytes);
    }
    return CheckLaunch("kv_gather_kernel", s);
}
