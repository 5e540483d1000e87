// Paged KV cache on the host side: LIFO block allocator with its block table, block-major storage,
// slot mapping, and the multi-sequence page-table bookkeeping. All integer results (block ids handed
// out, table rows, slots, counters, error codes and their wording) are bit-for-bit those of
// src/kv_cache/{block_manager,kv_cache,paged_kv_cache}.cpp in the reference; the data movement goes
// through the C ABI (sca_launch_kv_*), and the page table is mirrored to the device row by row
// instead of as one O(max_seqs * num_blocks) upload.
#include <algorithm>
#include <numeric>
#include <string>

#include "device/cuda_device.hpp"
#include "device/stream.hpp"
#include "internal.hpp"

namespace sca {

using runtime::FromAbi;
using runtime::StreamHandle;

// ================================================================================================
// BlockManager
// ================================================================================================
sci::Result<BlockManager> BlockManager::Create(int64_t num_blocks, int64_t max_num_seqs, int64_t max_blocks_per_seq,
                                               sci::Device& device) {
    if (num_blocks <= 0 || max_num_seqs <= 0 || max_blocks_per_seq <= 0) {
        return sci::MakeUnexpected<BlockManager>(MakeStatus(
            AttnStatusCode::kShapeMismatch,
            "BlockManager::Create invalid arguments: num_blocks=" + std::to_string(num_blocks) + ", max_num_seqs=" +
                std::to_string(max_num_seqs) + ", max_blocks_per_seq=" + std::to_string(max_blocks_per_seq)));
    }
    BlockManager bm;
    bm.num_blocks_ = num_blocks;
    bm.in_use_.assign(static_cast<size_t>(num_blocks), 0);
    // stack with block 0 on top: a fresh pool hands out 0, 1, 2, ...
    bm.free_list_.resize(static_cast<size_t>(num_blocks));
    for (int64_t i = 0; i < num_blocks; ++i) bm.free_list_[static_cast<size_t>(i)] = static_cast<int32_t>(num_blocks - 1 - i);
    bm.table_.max_num_seqs = max_num_seqs;
    bm.table_.max_blocks_per_seq = max_blocks_per_seq;
    bm.table_.host.assign(static_cast<size_t>(max_num_seqs * max_blocks_per_seq), -1);
    bm.table_.device = sci::Tensor(sci::TensorShape({max_num_seqs, max_blocks_per_seq}), sci::DType::kInt32, device);
    if (bm.table_.device.data() == nullptr) {
        return sci::MakeUnexpected<BlockManager>(
            MakeStatus(AttnStatusCode::kKVCapacityExceeded, "BlockManager: page table allocation of " +
                                                                std::to_string(max_num_seqs * max_blocks_per_seq * 4) + " B failed"));
    }
    // the device mirror starts as all -1 (0xFF bytes), so a read before the first sync is well defined
    device.memset(bm.table_.device.data(), 0xFF, bm.table_.host.size() * sizeof(int32_t));
    device.synchronize();
    return sci::Ok(std::move(bm));
}

sci::Result<std::vector<int32_t>> BlockManager::Allocate(int64_t count) {
    if (count <= 0) {
        return sci::MakeUnexpected<std::vector<int32_t>>(
            MakeStatus(AttnStatusCode::kShapeMismatch, "BlockManager::Allocate count=" + std::to_string(count)));
    }
    if (count > NumFreeBlocks()) {
        ++allocation_failures_;
        return sci::MakeUnexpected<std::vector<int32_t>>(MakeStatus(
            AttnStatusCode::kKVCapacityExceeded, "BlockManager::Allocate requested " + std::to_string(count) +
                                                     " blocks but only " + std::to_string(free_list_.size()) + " of " +
                                                     std::to_string(num_blocks_) + " are free"));
    }
    std::vector<int32_t> ids;
    ids.reserve(static_cast<size_t>(count));
    for (int64_t i = 0; i < count; ++i) {
        const int32_t block = free_list_.back();
        free_list_.pop_back();
        in_use_[static_cast<size_t>(block)] = 1;
        ids.push_back(block);
    }
    return sci::Ok(std::move(ids));
}

void BlockManager::Free(const int32_t* block_ids, int64_t count) {
    if (block_ids == nullptr) return;
    for (int64_t i = 0; i < count; ++i) {
        const int32_t block = block_ids[i];
        const bool held = block >= 0 && block < num_blocks_ && in_use_[static_cast<size_t>(block)] != 0;
        if (!held) {
            ++double_free_events_;  // out of range, or not handed out
            continue;
        }
        in_use_[static_cast<size_t>(block)] = 0;
        free_list_.push_back(block);
    }
}

sci::Status BlockManager::AppendToTable(int64_t seq_id, const int32_t* block_ids, int64_t count) {
    if (seq_id < 0 || seq_id >= table_.max_num_seqs) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "BlockManager::AppendToTable seq_id=" + std::to_string(seq_id) +
                                                              " out of range [0," + std::to_string(table_.max_num_seqs) + ")");
    }
    if (block_ids == nullptr || count <= 0) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "BlockManager::AppendToTable requires block_ids and count > 0");
    }
    int32_t* row = table_.host.data() + seq_id * table_.max_blocks_per_seq;
    int64_t used = 0;
    while (used < table_.max_blocks_per_seq && row[used] >= 0) ++used;
    if (used + count > table_.max_blocks_per_seq) {
        return MakeStatus(AttnStatusCode::kKVCapacityExceeded,
                          "BlockManager::AppendToTable sequence " + std::to_string(seq_id) + " would need " +
                              std::to_string(used + count) + " blocks > max_blocks_per_seq=" +
                              std::to_string(table_.max_blocks_per_seq));
    }
    std::copy(block_ids, block_ids + count, row + used);
    ++table_.revision;
    return sci::Status::Ok();
}

sci::Status BlockManager::ResetSeq(int64_t seq_id) {
    if (seq_id < 0 || seq_id >= table_.max_num_seqs) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "BlockManager::ResetSeq seq_id=" + std::to_string(seq_id) + " out of range");
    }
    int32_t* row = table_.host.data() + seq_id * table_.max_blocks_per_seq;
    // frees the first `live` entries, live = number of non-negative entries of the row
    const int64_t live = std::count_if(row, row + table_.max_blocks_per_seq, [](int32_t v) { return v >= 0; });
    if (live > 0) Free(row, live);
    std::fill(row, row + table_.max_blocks_per_seq, -1);
    ++table_.revision;
    return sci::Status::Ok();
}

sci::Status BlockManager::SyncTableToDevice(sci::Stream* stream) {
    if (table_.device.data() == nullptr) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "BlockManager: page table not allocated");
    }
    if (table_.synced_revision == table_.revision) return sci::Status::Ok();
    const size_t bytes = table_.host.size() * sizeof(int32_t);
    if (stream != nullptr) table_.device.device().copy_async(table_.device.data(), table_.host.data(), bytes, *stream);
    else table_.device.copy_from(table_.host.data(), bytes);
    table_.synced_revision = table_.revision;
    return sci::Status::Ok();
}

// ================================================================================================
// KVCache
// ================================================================================================
namespace {

constexpr double kKvBudgetRatio = 0.8;  // share of the currently free device memory a cache may claim

sci::Status CheckKvConfig(const KVCacheConfig& cfg) {
    auto bad = [](AttnStatusCode code, const std::string& text) { return MakeStatus(code, "KVCacheConfig invalid: " + text); };
    if (cfg.num_layers <= 0) return bad(AttnStatusCode::kShapeMismatch, "num_layers=" + std::to_string(cfg.num_layers));
    if (cfg.num_kv_heads <= 0) return bad(AttnStatusCode::kShapeMismatch, "num_kv_heads=" + std::to_string(cfg.num_kv_heads));
    if (SupportedHeadDimIndex(cfg.head_dim) < 0) return bad(AttnStatusCode::kUnsupportedHeadDim, "head_dim=" + std::to_string(cfg.head_dim));
    const int64_t bs = cfg.block_size;
    if (!(bs == 1 || bs == 8 || bs == 16 || bs == 32 || bs == 64)) {
        return bad(AttnStatusCode::kShapeMismatch, "block_size=" + std::to_string(bs) + " (supported: 1, 8, 16, 32, 64)");
    }
    if (cfg.num_blocks <= 0) return bad(AttnStatusCode::kShapeMismatch, "num_blocks=" + std::to_string(cfg.num_blocks));
    if (cfg.max_num_seqs <= 0) return bad(AttnStatusCode::kShapeMismatch, "max_num_seqs=" + std::to_string(cfg.max_num_seqs));
    if (!IsSupportedComputeDtype(cfg.dtype)) return bad(AttnStatusCode::kUnsupportedDtype, std::string("dtype=") + sci::kDTypeName(cfg.dtype));
    if (cfg.layout != KvLayout::kBlockMajor) {
        return bad(AttnStatusCode::kUnsupportedLayout,
                   std::string("layout=") + KvLayoutName(cfg.layout) + " (v1 implements block-major only)");
    }
    return sci::Status::Ok();
}

ScaKvCacheShape AbiShape(const KVCacheConfig& cfg) {
    return ScaKvCacheShape{cfg.num_blocks, cfg.block_size, cfg.num_kv_heads, cfg.head_dim};
}

}  // namespace

sci::Result<size_t> KvCacheBytes(const KVCacheConfig& cfg) {
    if (sci::Status s = CheckKvConfig(cfg); !s.ok()) return sci::MakeUnexpected<size_t>(s);
    const int64_t layer_elems = cfg.num_blocks * cfg.block_size * cfg.num_kv_heads * cfg.head_dim;
    const int64_t total = 2 * cfg.num_layers * layer_elems * DtypeSize(cfg.dtype);
    if (total <= 0) return sci::MakeUnexpected<size_t>(MakeStatus(AttnStatusCode::kShapeMismatch, "KVCacheConfig overflow"));
    return sci::Ok(static_cast<size_t>(total));
}

int64_t MaxBlocksForBudget(const KVCacheConfig& cfg, size_t budget_bytes) {
    const int64_t per_block = 2 * cfg.num_layers * cfg.block_size * cfg.num_kv_heads * cfg.head_dim * DtypeSize(cfg.dtype);
    return per_block > 0 ? static_cast<int64_t>(budget_bytes / static_cast<size_t>(per_block)) : 0;
}

sci::Result<std::vector<int32_t>> ComputeSlotMapping(const int32_t* block_table_row, int64_t seq_start, int64_t num_tokens,
                                                     int64_t block_size, int64_t max_blocks) {
    auto refuse = [](AttnStatusCode code, const std::string& text) {
        return sci::MakeUnexpected<std::vector<int32_t>>(MakeStatus(code, "ComputeSlotMapping: " + text));
    };
    if (block_table_row == nullptr) return refuse(AttnStatusCode::kShapeMismatch, "null block table row");
    if (block_size <= 0 || num_tokens <= 0) return refuse(AttnStatusCode::kShapeMismatch, "block_size/num_tokens <= 0");
    std::vector<int32_t> slots(static_cast<size_t>(num_tokens), -1);
    for (int64_t t = 0; t < num_tokens; ++t) {
        const int64_t pos = seq_start + t, logical = pos / block_size;
        if (logical >= max_blocks) {
            return refuse(AttnStatusCode::kKVCapacityExceeded,
                          "logical block " + std::to_string(logical) + " >= max_blocks=" + std::to_string(max_blocks));
        }
        const int32_t physical = block_table_row[logical];
        if (physical < 0) {
            return refuse(AttnStatusCode::kShapeMismatch, "block table slot " + std::to_string(logical) +
                                                              " is empty (-1) for position " + std::to_string(pos));
        }
        slots[static_cast<size_t>(t)] = static_cast<int32_t>(physical * block_size + pos % block_size);
    }
    return sci::Ok(std::move(slots));
}

sci::Result<KVCache> KVCache::Create(const KVCacheConfig& cfg, sci::Device& device) {
    if (sci::Status s = CheckKvConfig(cfg); !s.ok()) return sci::MakeUnexpected<KVCache>(s);
    const sci::Result<size_t> bytes = KvCacheBytes(cfg);
    if (!bytes.ok()) return sci::MakeUnexpected<KVCache>(bytes.error());

    // an over-budget request is answered with an error code and a suggestion, never with an OOM
    // "free" counts what the tensor pool holds without using it: the cache is allocated from that pool
    const unsigned long long free_b = device.type() == sci::DeviceType::kCUDA ? device.free_memory() : 0;
    if (device.type() == sci::DeviceType::kCUDA && free_b > 0) {
        const double budget = static_cast<double>(free_b) * kKvBudgetRatio;
        if (static_cast<double>(*bytes) > budget) {
            const int64_t fit = MaxBlocksForBudget(cfg, static_cast<size_t>(budget / (2 * cfg.num_layers)));
            const size_t mib = 1024 * 1024;
            return sci::MakeUnexpected<KVCache>(MakeStatus(
                AttnStatusCode::kKVCapacityExceeded,
                "KV cache needs " + std::to_string(*bytes / mib) + " MiB but only " + std::to_string(free_b / mib) +
                    " MiB is free (budget " + std::to_string(budget / mib) + " MiB); suggest num_blocks <= " +
                    std::to_string(std::max<int64_t>(1, fit))));
        }
    }
    KVCache cache;
    cache.cfg_ = cfg;
    cache.layer_elements_ = cfg.num_blocks * cfg.block_size * cfg.num_kv_heads * cfg.head_dim;
    const sci::TensorShape layer_shape({cfg.num_blocks, cfg.block_size, cfg.num_kv_heads, cfg.head_dim});
    for (int64_t layer = 0; layer < cfg.num_layers; ++layer) {
        cache.k_layers_.emplace_back(layer_shape, cfg.dtype, device);
        cache.v_layers_.emplace_back(layer_shape, cfg.dtype, device);
        if (cache.k_layers_.back().data() == nullptr || cache.v_layers_.back().data() == nullptr) {
            return sci::MakeUnexpected<KVCache>(
                MakeStatus(AttnStatusCode::kKVCapacityExceeded, "KV cache allocation failed at layer " + std::to_string(layer) +
                                                                    " (" + std::to_string(*bytes / (1024 * 1024)) + " MiB requested)"));
        }
    }
    cache.stats_.num_blocks = cfg.num_blocks;
    cache.stats_.free_blocks = cfg.num_blocks;
    cache.stats_.bytes = *bytes;
    cache.stats_.peak_bytes = *bytes;
    return sci::Ok(std::move(cache));
}

sci::Status KVCache::Append(int64_t layer, const sci::Tensor& k_new, const sci::Tensor& v_new, const int32_t* slot_mapping,
                            int64_t num_tokens, sci::Stream* stream) {
    if (layer < 0 || layer >= cfg_.num_layers) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "KVCache::Append layer=" + std::to_string(layer) +
                                                              " out of range [0," + std::to_string(cfg_.num_layers) + ")");
    }
    if (k_new.dtype() != cfg_.dtype || v_new.dtype() != cfg_.dtype) {
        return MakeStatus(AttnStatusCode::kUnsupportedDtype, std::string("KVCache::Append dtype mismatch: cache=") +
                                                                 sci::kDTypeName(cfg_.dtype) + ", k=" + sci::kDTypeName(k_new.dtype()));
    }
    if (k_new.ndims() != 3 || k_new.dim(0) != num_tokens || k_new.dim(1) != cfg_.num_kv_heads || k_new.dim(2) != cfg_.head_dim) {
        return MakeStatus(AttnStatusCode::kShapeMismatch,
                          "KVCache::Append expects k_new [num_tokens, num_kv_heads, head_dim]=" + std::to_string(num_tokens) +
                              "x" + std::to_string(cfg_.num_kv_heads) + "x" + std::to_string(cfg_.head_dim));
    }
    if (slot_mapping == nullptr) return MakeStatus(AttnStatusCode::kShapeMismatch, "KVCache::Append null slot_mapping");
    const ScaKvCacheShape shape = AbiShape(cfg_);
    const sci::Status launched = FromAbi(sca_launch_kv_append(
        k_layers_[static_cast<size_t>(layer)].data(), v_layers_[static_cast<size_t>(layer)].data(), k_new.data(), v_new.data(),
        slot_mapping, num_tokens, &shape, DtypeSize(cfg_.dtype), StreamHandle(stream)));
    if (!launched.ok()) return launched;
    ++stats_.num_appends;
    return sci::Status::Ok();
}

sci::Result<sci::Tensor> KVCache::GatherK(int64_t layer, const int32_t* ids, int64_t n, sci::Stream* stream) const {
    return GatherInternal(layer, ids, n, true, stream);
}
sci::Result<sci::Tensor> KVCache::GatherV(int64_t layer, const int32_t* ids, int64_t n, sci::Stream* stream) const {
    return GatherInternal(layer, ids, n, false, stream);
}

sci::Result<sci::Tensor> KVCache::GatherInternal(int64_t layer, const int32_t* block_ids, int64_t num_blocks, bool is_key,
                                                 sci::Stream* stream) const {
    const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(stream));
    const ApiRange nvtx_range("KVCache::GatherInternal");
    if (layer < 0 || layer >= cfg_.num_layers) {
        return sci::MakeUnexpected<sci::Tensor>(
            MakeStatus(AttnStatusCode::kShapeMismatch, "KVCache::Gather layer=" + std::to_string(layer) + " out of range"));
    }
    if (block_ids == nullptr || num_blocks <= 0) {
        return sci::MakeUnexpected<sci::Tensor>(
            MakeStatus(AttnStatusCode::kShapeMismatch, "KVCache::Gather requires block_ids and num_blocks>0"));
    }
    const sci::Tensor& src = (is_key ? k_layers_ : v_layers_)[static_cast<size_t>(layer)];
    sci::Tensor out(sci::TensorShape({num_blocks, cfg_.block_size, cfg_.num_kv_heads, cfg_.head_dim}), cfg_.dtype, src.device());
    if (out.data() == nullptr) {
        return sci::MakeUnexpected<sci::Tensor>(MakeStatus(AttnStatusCode::kWorkspaceExceeded, "KVCache::Gather allocation failed"));
    }
    const ScaKvCacheShape shape = AbiShape(cfg_);
    const sci::Status launched = FromAbi(sca_launch_kv_gather(src.data(), block_ids, num_blocks, out.data(), &shape,
                                                              DtypeSize(cfg_.dtype), StreamHandle(stream)));
    if (!launched.ok()) return sci::MakeUnexpected<sci::Tensor>(launched);
    return sci::Ok(std::move(out));
}

sci::Status KVCache::Reset(const int32_t* block_ids, int64_t num_blocks, sci::Stream* stream) {
    if (block_ids == nullptr) return MakeStatus(AttnStatusCode::kShapeMismatch, "KVCache::Reset null block_ids");
    if (num_blocks <= 0) return sci::Status::Ok();
    const ScaKvCacheShape shape = AbiShape(cfg_);
    for (int64_t layer = 0; layer < cfg_.num_layers; ++layer) {
        const sci::Status launched = FromAbi(sca_launch_kv_reset_block(
            k_layers_[static_cast<size_t>(layer)].data(), v_layers_[static_cast<size_t>(layer)].data(), block_ids, num_blocks,
            &shape, DtypeSize(cfg_.dtype), StreamHandle(stream)));
        if (!launched.ok()) return launched;
    }
    ++stats_.num_resets;
    return sci::Status::Ok();
}

const sci::Tensor& KVCache::K(int64_t layer) const {
    static const sci::Tensor* empty = new sci::Tensor();
    return (layer < 0 || layer >= cfg_.num_layers) ? *empty : k_layers_[static_cast<size_t>(layer)];
}
const sci::Tensor& KVCache::V(int64_t layer) const {
    static const sci::Tensor* empty = new sci::Tensor();
    return (layer < 0 || layer >= cfg_.num_layers) ? *empty : v_layers_[static_cast<size_t>(layer)];
}
KVCacheStats KVCache::Stats() const { return stats_; }
size_t KVCache::MemoryBytes() const noexcept { return stats_.bytes; }

// ================================================================================================
// PagedKVCache
// ================================================================================================
sci::Result<PagedKVCache> PagedKVCache::Create(const KVCacheConfig& cfg, sci::Device& device) {
    if (cfg.max_num_seqs <= 0) {
        return sci::MakeUnexpected<PagedKVCache>(MakeStatus(
            AttnStatusCode::kShapeMismatch, "PagedKVCacheConfig invalid: max_num_seqs=" + std::to_string(cfg.max_num_seqs)));
    }
    sci::Result<KVCache> storage = KVCache::Create(cfg, device);
    if (!storage.ok()) return sci::MakeUnexpected<PagedKVCache>(storage.error());
    // blocks are exclusive, so one sequence can at most own the whole pool: row length = num_blocks
    const int64_t row_len = cfg.num_blocks;
    sci::Result<BlockManager> blocks = BlockManager::Create(cfg.num_blocks, cfg.max_num_seqs, row_len, device);
    if (!blocks.ok()) return sci::MakeUnexpected<PagedKVCache>(blocks.error());

    PagedKVCache cache;
    cache.cfg_ = cfg;
    cache.max_blocks_per_seq_ = row_len;
    cache.storage_ = std::move(*storage);
    cache.blocks_ = std::move(*blocks);
    cache.seq_lengths_.assign(static_cast<size_t>(cfg.max_num_seqs), 0);
    cache.seq_blocks_.assign(static_cast<size_t>(cfg.max_num_seqs), {});
    cache.page_table_host_.assign(static_cast<size_t>(cfg.max_num_seqs * row_len), -1);
    cache.page_table_device_ = sci::Tensor(sci::TensorShape({cfg.max_num_seqs, row_len}), sci::DType::kInt32, device);
    cache.seq_lens_device_ = sci::Tensor(sci::TensorShape({cfg.max_num_seqs}), sci::DType::kInt32, device);
    cache.seq_order_device_ = sci::Tensor(sci::TensorShape({cfg.max_num_seqs}), sci::DType::kInt32, device);
    if (cache.page_table_device_.data() == nullptr || cache.seq_lens_device_.data() == nullptr ||
        cache.seq_order_device_.data() == nullptr) {
        return sci::MakeUnexpected<PagedKVCache>(
            MakeStatus(AttnStatusCode::kKVCapacityExceeded, "PagedKVCache: page table allocation failed"));
    }
    device.memset(cache.page_table_device_.data(), 0xFF, cache.page_table_host_.size() * sizeof(int32_t));
    device.synchronize();
    cache.live_on_device_.assign(static_cast<size_t>(cfg.max_num_seqs), 0);
    cache.revision_ = 1;
    cache.synced_revision_ = 1;
    return sci::Ok(std::move(cache));
}

sci::Status PagedKVCache::AppendTokens(int64_t seq_id, int64_t layer, const sci::Tensor& k_new, const sci::Tensor& v_new,
                                       sci::Stream* stream) {
    const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(stream));
    const ApiRange nvtx_range("PagedKVCache::AppendTokens");
    if (seq_id < 0 || seq_id >= cfg_.max_num_seqs) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "PagedKVCache::AppendTokens seq_id=" + std::to_string(seq_id) +
                                                              " out of range [0," + std::to_string(cfg_.max_num_seqs) + ")");
    }
    if (layer < 0 || layer >= cfg_.num_layers) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "PagedKVCache::AppendTokens layer=" + std::to_string(layer) +
                                                              " out of range [0," + std::to_string(cfg_.num_layers) + ")");
    }
    if (k_new.ndims() != 3 || v_new.ndims() != 3 || k_new.dim(0) != v_new.dim(0)) {
        return MakeStatus(AttnStatusCode::kShapeMismatch,
                          "PagedKVCache::AppendTokens expects [num_tokens, n_kv_heads, head_dim] tensors");
    }
    const int64_t n = k_new.dim(0);
    if (n <= 0) return MakeStatus(AttnStatusCode::kShapeMismatch, "PagedKVCache::AppendTokens: 0 tokens");

    std::vector<int32_t>& owned = seq_blocks_[static_cast<size_t>(seq_id)];
    const int64_t len = seq_lengths_[static_cast<size_t>(seq_id)];
    const int64_t missing = detail::CeilDiv<int64_t>(len + n, cfg_.block_size) - static_cast<int64_t>(owned.size());
    int32_t* row = page_table_host_.data() + seq_id * max_blocks_per_seq_;
    if (missing > 0) {
        sci::Result<std::vector<int32_t>> fresh = blocks_.Allocate(missing);
        if (!fresh.ok()) {  // nothing has changed
            return MakeStatus(AttnStatusCode::kKVCapacityExceeded,
                              "PagedKVCache::AppendTokens seq=" + std::to_string(seq_id) + " needs " + std::to_string(missing) +
                                  " more blocks but only " + std::to_string(blocks_.NumFreeBlocks()) + " are free");
        }
        const sci::Status attached = blocks_.AppendToTable(seq_id, fresh->data(), static_cast<int64_t>(fresh->size()));
        if (!attached.ok()) {
            blocks_.Free(fresh->data(), static_cast<int64_t>(fresh->size()));
            return attached;
        }
        // the row already holds owned[0..size) followed by -1: only the new entries are written
        std::copy(fresh->begin(), fresh->end(), row + owned.size());
        owned.insert(owned.end(), fresh->begin(), fresh->end());
    }
    const sci::Result<std::vector<int32_t>> slots = ComputeSlotMapping(row, len, n, cfg_.block_size, max_blocks_per_seq_);
    if (!slots.ok()) return slots.error();

    if (slot_mapping_capacity_ < n) {
        const int64_t capacity = std::max<int64_t>(n, 1024);
        slot_mapping_device_ = sci::Tensor(sci::TensorShape({capacity}), sci::DType::kInt32, storage_.K(0).device());
        if (slot_mapping_device_.data() == nullptr) {
            slot_mapping_capacity_ = 0;
            return MakeStatus(AttnStatusCode::kKVCapacityExceeded, "PagedKVCache: slot-mapping buffer allocation failed");
        }
        slot_mapping_capacity_ = capacity;
    }
    // blocking 4 B/token upload, as in the reference; AppendTokenBatch is the path without it
    storage_.K(0).device().copy_to_device(slot_mapping_device_.data(), slots->data(), static_cast<size_t>(n) * sizeof(int32_t));
    const sci::Status stored =
        storage_.Append(layer, k_new, v_new, static_cast<const int32_t*>(slot_mapping_device_.data()), n, stream);
    if (!stored.ok()) return stored;  // blocks stay attached; ResetSeq recovers
    seq_lengths_[static_cast<size_t>(seq_id)] = len + n;
    ++revision_;
    ++num_appends_;
    return sci::Status::Ok();
}

sci::Status PagedKVCache::AppendTokenBatch(int64_t num_seqs, int64_t layer, const sci::Tensor& k_new, const sci::Tensor& v_new,
                                           sci::Stream* stream) {
    const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(stream));
    const ApiRange nvtx_range("PagedKVCache::AppendTokenBatch");
    if (num_seqs <= 0 || num_seqs > cfg_.max_num_seqs) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "PagedKVCache::AppendTokenBatch num_seqs=" + std::to_string(num_seqs) +
                                                              " out of range [1," + std::to_string(cfg_.max_num_seqs) + "]");
    }
    if (layer < 0 || layer >= cfg_.num_layers) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "PagedKVCache::AppendTokenBatch layer=" + std::to_string(layer) +
                                                              " out of range [0," + std::to_string(cfg_.num_layers) + ")");
    }
    for (const sci::Tensor* t : {&k_new, &v_new}) {
        if (t->ndims() != 3 || t->dim(0) != num_seqs || t->dim(1) != cfg_.num_kv_heads || t->dim(2) != cfg_.head_dim ||
            t->dtype() != cfg_.dtype) {
            return MakeStatus(AttnStatusCode::kShapeMismatch,
                              "PagedKVCache::AppendTokenBatch expects [num_seqs, n_kv_heads, head_dim] tensors of the cache dtype");
        }
    }
    // all-or-nothing: count the blocks every sequence needs for one more token
    int64_t needed = 0;
    for (int64_t s = 0; s < num_seqs; ++s) {
        if (seq_lengths_[static_cast<size_t>(s)] % cfg_.block_size == 0 &&
            seq_lengths_[static_cast<size_t>(s)] / cfg_.block_size == static_cast<int64_t>(seq_blocks_[static_cast<size_t>(s)].size())) {
            ++needed;
        }
    }
    if (needed > blocks_.NumFreeBlocks()) {
        return MakeStatus(AttnStatusCode::kKVCapacityExceeded,
                          "PagedKVCache::AppendTokenBatch needs " + std::to_string(needed) + " more blocks but only " +
                              std::to_string(blocks_.NumFreeBlocks()) + " are free");
    }
    sci::Device& device = page_table_device_.device();
    sci::Stream current(StreamHandle(stream));
    int32_t* table_dev = static_cast<int32_t*>(page_table_device_.data());
    // rows changed by AppendTokens / ResetSeq since the last sync are brought up to date first
    if (revision_ != synced_revision_) {
        if (sci::Status synced = ForceSyncPageTable(&current); !synced.ok()) return synced;
    }
    for (int64_t s = 0; s < num_seqs; ++s) {
        std::vector<int32_t>& owned = seq_blocks_[static_cast<size_t>(s)];
        const int64_t len = seq_lengths_[static_cast<size_t>(s)];
        if (detail::CeilDiv<int64_t>(len + 1, cfg_.block_size) > static_cast<int64_t>(owned.size())) {
            sci::Result<std::vector<int32_t>> fresh = blocks_.Allocate(1);
            if (!fresh.ok()) return fresh.error();  // cannot happen after the count above
            if (sci::Status a = blocks_.AppendToTable(s, fresh->data(), 1); !a.ok()) {
                blocks_.Free(fresh->data(), 1);
                return a;
            }
            const int64_t col = static_cast<int64_t>(owned.size());
            page_table_host_[static_cast<size_t>(s * max_blocks_per_seq_ + col)] = (*fresh)[0];
            owned.push_back((*fresh)[0]);
            // mirror exactly this entry: the rest of the row on the device is current
            device.copy_async(table_dev + s * max_blocks_per_seq_ + col,
                              &page_table_host_[static_cast<size_t>(s * max_blocks_per_seq_ + col)], sizeof(int32_t), current);
            live_on_device_[static_cast<size_t>(s)] = std::max<int64_t>(live_on_device_[static_cast<size_t>(s)], col + 1);
        }
        seq_lengths_[static_cast<size_t>(s)] = len + 1;
    }
    std::vector<int32_t> lens(static_cast<size_t>(num_seqs));
    for (int64_t s = 0; s < num_seqs; ++s) lens[static_cast<size_t>(s)] = static_cast<int32_t>(seq_lengths_[static_cast<size_t>(s)]);
    device.copy_async(seq_lens_device_.data(), lens.data(), lens.size() * sizeof(int32_t), current);

    const ScaKvCacheShape shape = AbiShape(cfg_);
    const sci::Status launched = FromAbi(sca_launch_kv_append_batched(
        const_cast<void*>(storage_.K(layer).data()), const_cast<void*>(storage_.V(layer).data()), k_new.data(), v_new.data(),
        table_dev, static_cast<const int32_t*>(seq_lens_device_.data()), num_seqs, max_blocks_per_seq_, &shape,
        DtypeSize(cfg_.dtype), current.handle()));
    if (!launched.ok()) {
        // nothing was stored: take the token back. Blocks attached above stay with their sequences (as after a failed
        // AppendTokens, ResetSeq recovers them); the device lengths are now ahead of the host, so force the next sync.
        for (int64_t s = 0; s < num_seqs; ++s) --seq_lengths_[static_cast<size_t>(s)];
        ++revision_;
        return launched;
    }
    ++revision_;
    synced_revision_ = revision_;  // table and lengths on the device already reflect this step
    num_appends_ += num_seqs;
    return sci::Status::Ok();
}

const int32_t* PagedKVCache::SeqLensDevicePtr() const noexcept {
    return static_cast<const int32_t*>(seq_lens_device_.data());
}

sci::Status PagedKVCache::ResetSeq(int64_t seq_id, sci::Stream* stream) {
    if (seq_id < 0 || seq_id >= cfg_.max_num_seqs) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "PagedKVCache::ResetSeq seq_id=" + std::to_string(seq_id) + " out of range");
    }
    std::vector<int32_t>& owned = seq_blocks_[static_cast<size_t>(seq_id)];
    if (!owned.empty()) {
        // order: clear the data, release the blocks, blank the row. The block ids reach the kernel through a
        // small device buffer because KVCache::Reset takes device-resident ids.
        sci::Device& device = storage_.K(0).device();
        sci::Tensor ids(sci::TensorShape({static_cast<sci::index_t>(owned.size())}), sci::DType::kInt32, device);
        if (ids.data() == nullptr) return MakeStatus(AttnStatusCode::kKVCapacityExceeded, "PagedKVCache::ResetSeq: id buffer allocation failed");
        ids.copy_from(owned.data(), owned.size() * sizeof(int32_t));
        const sci::Status cleared = storage_.Reset(static_cast<const int32_t*>(ids.data()), static_cast<int64_t>(owned.size()), stream);
        if (!cleared.ok()) return cleared;
        if (device.type() == sci::DeviceType::kCUDA) {
            sci::Stream used(StreamHandle(stream));
            used.synchronize();  // `ids` is released when this scope ends
        }
    }
    blocks_.ResetSeq(seq_id);
    int32_t* row = page_table_host_.data() + seq_id * max_blocks_per_seq_;
    std::fill(row, row + owned.size(), -1);
    owned.clear();
    seq_lengths_[static_cast<size_t>(seq_id)] = 0;
    ++revision_;
    ++num_resets_;
    return sci::Status::Ok();
}

const int32_t* PagedKVCache::PageTableDevicePtr() const noexcept {
    return static_cast<const int32_t*>(page_table_device_.data());
}
const int32_t* PagedKVCache::SeqOrderDevicePtr(int64_t num_seqs) const noexcept {
    if (seq_order_extent_ < 0 || num_seqs < seq_order_extent_ || num_seqs > cfg_.max_num_seqs) return nullptr;
    return static_cast<const int32_t*>(seq_order_device_.data());
}
int64_t PagedKVCache::LogicalBlockCount(int64_t seq_id) const noexcept {
    return (seq_id < 0 || seq_id >= cfg_.max_num_seqs) ? 0 : static_cast<int64_t>(seq_blocks_[static_cast<size_t>(seq_id)].size());
}
int64_t PagedKVCache::SeqLength(int64_t seq_id) const noexcept {
    return (seq_id < 0 || seq_id >= cfg_.max_num_seqs) ? 0 : seq_lengths_[static_cast<size_t>(seq_id)];
}

sci::Status PagedKVCache::SyncPageTable(sci::Stream* stream) {
    if (revision_ == synced_revision_) return sci::Status::Ok();
    return ForceSyncPageTable(stream);
}

// Brings the device mirror to the host table's state. Row s is uploaded over max(previous live length,
// current live length) entries - everything beyond is -1 on both sides - so the device copy ends up
// identical to a full upload while moving only the live prefix of each row.
sci::Status PagedKVCache::ForceSyncPageTable(sci::Stream* stream) {
    if (page_table_device_.data() == nullptr) return MakeStatus(AttnStatusCode::kShapeMismatch, "PagedKVCache: page table missing");
    sci::Device& device = page_table_device_.device();
    int32_t* table_dev = static_cast<int32_t*>(page_table_device_.data());
    std::vector<int32_t> lens(static_cast<size_t>(cfg_.max_num_seqs));
    for (int64_t s = 0; s < cfg_.max_num_seqs; ++s) {
        const int64_t now = static_cast<int64_t>(seq_blocks_[static_cast<size_t>(s)].size());
        const int64_t span = std::max<int64_t>(now, live_on_device_[static_cast<size_t>(s)]);
        lens[static_cast<size_t>(s)] = static_cast<int32_t>(seq_lengths_[static_cast<size_t>(s)]);
        if (span == 0) continue;
        const int32_t* src = page_table_host_.data() + s * max_blocks_per_seq_;
        int32_t* dst = table_dev + s * max_blocks_per_seq_;
        if (stream != nullptr) device.copy_async(dst, src, static_cast<size_t>(span) * sizeof(int32_t), *stream);
        else device.copy_to_device(dst, src, static_cast<size_t>(span) * sizeof(int32_t));
        live_on_device_[static_cast<size_t>(s)] = now;
    }
    if (stream != nullptr) device.copy_async(seq_lens_device_.data(), lens.data(), lens.size() * sizeof(int32_t), *stream);
    else device.copy_to_device(seq_lens_device_.data(), lens.data(), lens.size() * sizeof(int32_t));
    // launch order for the decode kernel: longest sequence first, ties and empty slots by index, so that the
    // first n entries are a permutation of [0, n) whenever every slot from n on is empty
    std::vector<int32_t> order(lens.size());
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&lens](int32_t a, int32_t b) { return lens[static_cast<size_t>(a)] > lens[static_cast<size_t>(b)]; });
    int64_t extent = 0;
    for (int64_t s = 0; s < cfg_.max_num_seqs; ++s) {
        if (lens[static_cast<size_t>(s)] > 0) extent = s + 1;
    }
    if (stream != nullptr) device.copy_async(seq_order_device_.data(), order.data(), order.size() * sizeof(int32_t), *stream);
    else device.copy_to_device(seq_order_device_.data(), order.data(), order.size() * sizeof(int32_t));
    seq_order_extent_ = extent;
    synced_revision_ = revision_;
    return sci::Status::Ok();
}

KVCacheStats PagedKVCache::Stats() const {
    KVCacheStats s = storage_.Stats();
    s.num_blocks = blocks_.NumTotalBlocks();
    s.free_blocks = blocks_.NumFreeBlocks();
    s.used_blocks = s.num_blocks - s.free_blocks;
    s.num_appends = num_appends_;
    s.num_resets = num_resets_;
    return s;
}

}  // namespace sca
