// Flat C view of the C++ host layer so that scripts (the Python parity tests, language bindings) can
// drive Validate / Select / Explain, the block allocator and the paged cache without a C++ compiler.
// Records: cfg_i = {backend, layout, causal, return_lse, sliding_window, num_splits, allow_fallback,
// has_cu_seqlens_q, has_cu_seqlens_kv}; cfg_f = {scale, softcap}; shape = {batch, seq_q, seq_kv,
// num_heads, num_kv_heads, head_dim}. device_index < 0 selects host memory, otherwise that GPU.
#include <cstring>
#include <memory>
#include <string>

#include "device/cuda_device.hpp"
#include "internal.hpp"

#define SCA_C_API extern "C" __attribute__((visibility("default")))

namespace {

int CopyOut(const std::string& text, char* out, int cap) {
    if (out != nullptr && cap > 0) {
        std::strncpy(out, text.c_str(), static_cast<size_t>(cap - 1));
        out[cap - 1] = '\0';
    }
    return static_cast<int>(text.size());
}

sca::AttentionConfig ConfigFrom(const int64_t* ci, const float* cf) {
    static const int32_t kOffsets[2] = {0, 1};
    sca::AttentionConfig cfg;
    cfg.backend = static_cast<sca::BackendKind>(ci[0]);
    cfg.layout = static_cast<sca::AttnLayout>(ci[1]);
    cfg.causal = ci[2] != 0;
    cfg.return_lse = ci[3] != 0;
    cfg.sliding_window = ci[4];
    cfg.num_splits = ci[5];
    cfg.allow_fallback = ci[6] != 0;
    cfg.cu_seqlens_q = ci[7] != 0 ? kOffsets : nullptr;
    cfg.cu_seqlens_kv = ci[8] != 0 ? kOffsets : nullptr;
    cfg.scale = cf[0];
    cfg.softcap = cf[1];
    return cfg;
}

sca::AttentionShape ShapeFrom(const int64_t* s) {
    sca::AttentionShape shape;
    shape.batch = s[0];
    shape.seq_q = s[1];
    shape.seq_kv = s[2];
    shape.num_heads = s[3];
    shape.num_kv_heads = s[4];
    shape.head_dim = s[5];
    return shape;
}

sci::Device* DeviceFor(int index, std::shared_ptr<sci::Device>* keep) {
    if (index < 0) return &sci::HostDevice();
    *keep = sci::DeviceManager::Instance().get_device(sci::DeviceType::kCUDA, index);
    return keep->get();
}

struct PagedHandle {
    std::shared_ptr<sci::Device> keep;
    sci::Device* device{nullptr};
    sca::KVCacheConfig cfg;
    sca::PagedKVCache cache;
};

struct BlockManagerHandle {
    std::shared_ptr<sci::Device> keep;
    sca::BlockManager manager;
};

}  // namespace

SCA_C_API int sca_c_validate(const int64_t* cfg_i, const float* cfg_f, const int64_t* shape, char* msg, int cap) {
    std::string detail;
    const sci::Status s = sca::Validate(ConfigFrom(cfg_i, cfg_f), ShapeFrom(shape), &detail);
    CopyOut(s.ok() ? detail : s.message(), msg, cap);
    return static_cast<int>(sca::ExtractCode(s));
}
SCA_C_API float sca_c_effective_scale(const int64_t* cfg_i, const float* cfg_f, const int64_t* shape) {
    return sca::EffectiveScale(ConfigFrom(cfg_i, cfg_f), ShapeFrom(shape));
}
SCA_C_API int sca_c_select(const int64_t* cfg_i, const float* cfg_f, const int64_t* shape, char* reason, int cap,
                           int32_t* tile4, int64_t* workspace_bytes) {
    const sca::DispatchDecision d = sca::AttentionDispatcher().Select(ConfigFrom(cfg_i, cfg_f), ShapeFrom(shape));
    CopyOut(d.reason, reason, cap);
    if (tile4 != nullptr) {
        tile4[0] = d.tile.block_m;
        tile4[1] = d.tile.block_n;
        tile4[2] = d.tile.warps;
        tile4[3] = d.tile.stages;
    }
    if (workspace_bytes != nullptr) *workspace_bytes = static_cast<int64_t>(d.workspace_bytes);
    return static_cast<int>(d.backend);
}
SCA_C_API int sca_c_explain(const int64_t* cfg_i, const float* cfg_f, const int64_t* shape, char* out, int cap) {
    return CopyOut(sca::AttentionDispatcher().Explain(ConfigFrom(cfg_i, cfg_f), ShapeFrom(shape)), out, cap);
}
SCA_C_API int sca_c_status_info(int attn_code, int* sci_code, char* name, int cap) {
    const auto code = static_cast<sca::AttnStatusCode>(attn_code);
    *sci_code = static_cast<int>(sca::ToSciCode(code));
    CopyOut(sca::ToString(code), name, cap);
    return static_cast<int>(sca::ExtractCode(sca::MakeStatus(code, "x")));
}
SCA_C_API int sca_c_varlen_validate(const int32_t* cu, int64_t batch, int64_t* max_seq, char* msg, int cap) {
    const sci::Status s = sca::ValidateVarlenHost(cu, batch, max_seq);
    CopyOut(s.message(), msg, cap);
    return static_cast<int>(sca::ExtractCode(s));
}
SCA_C_API const char* sca_c_dispatch_revision() { return sca::tables::kDispatch.revision; }
SCA_C_API int64_t sca_c_decode_splits_for(int64_t seq_kv, int64_t batch, int64_t kv_heads, int64_t group, int64_t sms) {
    return sca::tables::DecodeSplitsFor(seq_kv, batch, kv_heads, group, sms);
}
SCA_C_API int64_t sca_c_paged_splits_for(int64_t typical, int64_t seqs, int64_t kv_heads, int64_t group, int64_t sms) {
    return sca::tables::PagedSplitsFor(typical, seqs, kv_heads, group, sms);
}

// ---- BlockManager -----------------------------------------------------------------------------------------
SCA_C_API void* sca_c_bm_create(int64_t num_blocks, int64_t max_seqs, int64_t max_blocks_per_seq, int device_index,
                                char* msg, int cap) {
    auto handle = std::make_unique<BlockManagerHandle>();
    sci::Device* device = DeviceFor(device_index, &handle->keep);
    if (device == nullptr) {
        CopyOut("no such device", msg, cap);
        return nullptr;
    }
    sci::Result<sca::BlockManager> r = sca::BlockManager::Create(num_blocks, max_seqs, max_blocks_per_seq, *device);
    if (!r.ok()) {
        CopyOut(r.message(), msg, cap);
        return nullptr;
    }
    handle->manager = std::move(*r);
    return handle.release();
}
SCA_C_API void sca_c_bm_destroy(void* h) { delete static_cast<BlockManagerHandle*>(h); }
SCA_C_API int sca_c_bm_allocate(void* h, int64_t count, int32_t* out, char* msg, int cap) {
    sci::Result<std::vector<int32_t>> r = static_cast<BlockManagerHandle*>(h)->manager.Allocate(count);
    if (!r.ok()) {
        CopyOut(r.message(), msg, cap);
        return static_cast<int>(sca::ExtractCode(r.error()));
    }
    std::memcpy(out, r->data(), r->size() * sizeof(int32_t));
    return 0;
}
SCA_C_API void sca_c_bm_free(void* h, const int32_t* ids, int64_t count) {
    static_cast<BlockManagerHandle*>(h)->manager.Free(ids, count);
}
SCA_C_API int sca_c_bm_append_to_table(void* h, int64_t seq, const int32_t* ids, int64_t count, char* msg, int cap) {
    const sci::Status s = static_cast<BlockManagerHandle*>(h)->manager.AppendToTable(seq, ids, count);
    CopyOut(s.message(), msg, cap);
    return static_cast<int>(sca::ExtractCode(s));
}
SCA_C_API int sca_c_bm_reset_seq(void* h, int64_t seq) {
    return static_cast<int>(sca::ExtractCode(static_cast<BlockManagerHandle*>(h)->manager.ResetSeq(seq)));
}
SCA_C_API int64_t sca_c_bm_num_free(void* h) { return static_cast<BlockManagerHandle*>(h)->manager.NumFreeBlocks(); }
SCA_C_API int64_t sca_c_bm_allocation_failures(void* h) { return static_cast<BlockManagerHandle*>(h)->manager.AllocationFailures(); }
SCA_C_API int64_t sca_c_bm_double_free_events(void* h) { return static_cast<BlockManagerHandle*>(h)->manager.DoubleFreeEvents(); }
SCA_C_API uint64_t sca_c_bm_revision(void* h) { return static_cast<BlockManagerHandle*>(h)->manager.Table().revision; }
SCA_C_API const int32_t* sca_c_bm_table(void* h) { return static_cast<BlockManagerHandle*>(h)->manager.Table().host.data(); }

// ---- slot mapping / budget ---------------------------------------------------------------------------------------
SCA_C_API int sca_c_slot_mapping(const int32_t* row, int64_t start, int64_t n, int64_t bs, int64_t max_blocks, int32_t* out,
                                 char* msg, int cap) {
    sci::Result<std::vector<int32_t>> r = sca::ComputeSlotMapping(row, start, n, bs, max_blocks);
    if (!r.ok()) {
        CopyOut(r.message(), msg, cap);
        return static_cast<int>(sca::ExtractCode(r.error()));
    }
    std::memcpy(out, r->data(), r->size() * sizeof(int32_t));
    return 0;
}

static sca::KVCacheConfig KvConfig(int64_t layers, int64_t blocks, int64_t bs, int64_t hkv, int64_t d, int dtype, int64_t seqs) {
    sca::KVCacheConfig cfg;
    cfg.num_layers = layers;
    cfg.num_blocks = blocks;
    cfg.block_size = bs;
    cfg.num_kv_heads = hkv;
    cfg.head_dim = d;
    cfg.dtype = static_cast<sci::DType>(dtype);
    cfg.max_num_seqs = seqs;
    return cfg;
}
SCA_C_API int64_t sca_c_kv_cache_bytes(int64_t layers, int64_t blocks, int64_t bs, int64_t hkv, int64_t d, int dtype,
                                       char* msg, int cap) {
    sci::Result<size_t> r = sca::KvCacheBytes(KvConfig(layers, blocks, bs, hkv, d, dtype, 1));
    if (!r.ok()) {
        CopyOut(r.message(), msg, cap);
        return -static_cast<int64_t>(sca::ExtractCode(r.error()));
    }
    return static_cast<int64_t>(*r);
}
SCA_C_API int64_t sca_c_max_blocks_for_budget(int64_t layers, int64_t bs, int64_t hkv, int64_t d, int dtype, uint64_t budget) {
    return sca::MaxBlocksForBudget(KvConfig(layers, 1, bs, hkv, d, dtype, 1), budget);
}

// ---- PagedKVCache (k_new / v_new are HOST buffers here; they are staged to the cache's device) ------------------------
SCA_C_API void* sca_c_paged_create(int64_t layers, int64_t blocks, int64_t bs, int64_t hkv, int64_t d, int dtype,
                                   int64_t seqs, int device_index, char* msg, int cap) {
    auto handle = std::make_unique<PagedHandle>();
    handle->device = DeviceFor(device_index, &handle->keep);
    if (handle->device == nullptr) {
        CopyOut("no such device", msg, cap);
        return nullptr;
    }
    handle->cfg = KvConfig(layers, blocks, bs, hkv, d, dtype, seqs);
    sci::Result<sca::PagedKVCache> r = sca::PagedKVCache::Create(handle->cfg, *handle->device);
    if (!r.ok()) {
        CopyOut(r.message(), msg, cap);
        return nullptr;
    }
    handle->cache = std::move(*r);
    return handle.release();
}
SCA_C_API void sca_c_paged_destroy(void* h) { delete static_cast<PagedHandle*>(h); }
SCA_C_API int sca_c_paged_append(void* h, int64_t seq, int64_t layer, const void* k_host, const void* v_host, int64_t n,
                                 char* msg, int cap) {
    auto* p = static_cast<PagedHandle*>(h);
    const sci::TensorShape shape({n, p->cfg.num_kv_heads, p->cfg.head_dim});
    sci::Tensor k(shape, p->cfg.dtype, *p->device), v(shape, p->cfg.dtype, *p->device);
    k.copy_from(k_host, k.num_bytes());
    v.copy_from(v_host, v.num_bytes());
    const sci::Status s = p->cache.AppendTokens(seq, layer, k, v, nullptr);
    p->device->synchronize();
    CopyOut(s.message(), msg, cap);
    return s.ok() ? 0 : (sca::ExtractCode(s) != sca::AttnStatusCode::kOk ? static_cast<int>(sca::ExtractCode(s))
                                                                          : static_cast<int>(s.code()));
}
SCA_C_API int sca_c_paged_append_batch(void* h, int64_t num_seqs, int64_t layer, const void* k_host, const void* v_host,
                                       char* msg, int cap) {
    auto* p = static_cast<PagedHandle*>(h);
    const sci::TensorShape shape({num_seqs, p->cfg.num_kv_heads, p->cfg.head_dim});
    sci::Tensor k(shape, p->cfg.dtype, *p->device), v(shape, p->cfg.dtype, *p->device);
    k.copy_from(k_host, k.num_bytes());
    v.copy_from(v_host, v.num_bytes());
    const sci::Status s = p->cache.AppendTokenBatch(num_seqs, layer, k, v, nullptr);
    p->device->synchronize();
    CopyOut(s.message(), msg, cap);
    return s.ok() ? 0 : (sca::ExtractCode(s) != sca::AttnStatusCode::kOk ? static_cast<int>(sca::ExtractCode(s))
                                                                          : static_cast<int>(s.code()));
}
SCA_C_API int sca_c_paged_reset_seq(void* h, int64_t seq) {
    return static_cast<int>(sca::ExtractCode(static_cast<PagedHandle*>(h)->cache.ResetSeq(seq, nullptr)));
}
SCA_C_API int64_t sca_c_paged_seq_length(void* h, int64_t seq) { return static_cast<PagedHandle*>(h)->cache.SeqLength(seq); }
SCA_C_API int64_t sca_c_paged_logical_blocks(void* h, int64_t seq) { return static_cast<PagedHandle*>(h)->cache.LogicalBlockCount(seq); }
SCA_C_API int64_t sca_c_paged_max_blocks_per_seq(void* h) { return static_cast<PagedHandle*>(h)->cache.MaxBlocksPerSeq(); }
// Syncs, then copies the DEVICE page table ([max_seqs, max_blocks]) and sequence lengths to host buffers.
SCA_C_API int sca_c_paged_read_table(void* h, int32_t* table_out, int32_t* lens_out) {
    auto* p = static_cast<PagedHandle*>(h);
    const sci::Status s = p->cache.SyncPageTable(nullptr);
    if (!s.ok()) return static_cast<int>(sca::ExtractCode(s));
    p->device->synchronize();
    const size_t entries = static_cast<size_t>(p->cfg.max_num_seqs * p->cache.MaxBlocksPerSeq());
    p->device->copy_to_host(table_out, p->cache.PageTableDevicePtr(), entries * sizeof(int32_t));
    if (lens_out != nullptr) {
        p->device->copy_to_host(lens_out, p->cache.SeqLensDevicePtr(), static_cast<size_t>(p->cfg.max_num_seqs) * sizeof(int32_t));
    }
    return 0;
}
SCA_C_API void sca_c_paged_read_layer(void* h, int64_t layer, int is_key, void* out) {
    auto* p = static_cast<PagedHandle*>(h);
    const sci::Tensor& t = is_key ? p->cache.Storage().K(layer) : p->cache.Storage().V(layer);
    p->device->synchronize();
    p->device->copy_to_host(out, t.data(), t.num_bytes());
}
SCA_C_API void sca_c_paged_stats(void* h, int64_t* out7) {
    const sca::KVCacheStats s = static_cast<PagedHandle*>(h)->cache.Stats();
    out7[0] = s.num_blocks;
    out7[1] = s.used_blocks;
    out7[2] = s.free_blocks;
    out7[3] = s.num_appends;
    out7[4] = s.num_resets;
    out7[5] = static_cast<int64_t>(s.peak_bytes);
    out7[6] = static_cast<int64_t>(s.bytes);
}
// Paged decode through the C++ API with the cache's own table and lengths; q_host / out_host are host
// buffers of [num_seqs, heads, 1, D] elements of the cache dtype.
SCA_C_API int sca_c_paged_attention(void* h, const void* q_host, int64_t num_seqs, int64_t heads, int64_t num_splits,
                                    void* out_host, int64_t* splits_used, char* msg, int cap) {
    auto* p = static_cast<PagedHandle*>(h);
    const sci::TensorShape shape({num_seqs, heads, 1, p->cfg.head_dim});
    sci::Tensor q(shape, p->cfg.dtype, *p->device);
    q.copy_from(q_host, q.num_bytes());
    if (sci::Status s = p->cache.SyncPageTable(nullptr); !s.ok()) {
        CopyOut(s.message(), msg, cap);
        return static_cast<int>(s.code());
    }
    sca::PagedAttentionParams params;
    params.page_table = p->cache.PageTableDevicePtr();
    params.seq_lens = p->cache.SeqLensDevicePtr();
    params.num_seqs = num_seqs;
    params.block_size = p->cache.BlockSize();
    params.max_blocks_per_seq = p->cache.MaxBlocksPerSeq();
    sca::AttentionConfig cfg;
    cfg.num_splits = num_splits;
    const sci::Result<sca::AttentionResult> r = sca::paged_attention(q, p->cache, params, cfg);
    if (!r.ok()) {
        CopyOut(r.message(), msg, cap);
        return static_cast<int>(r.error().code());
    }
    p->device->synchronize();
    p->device->copy_to_host(out_host, r->out.data(), r->out.num_bytes());
    if (splits_used != nullptr) *splits_used = r->stats.num_splits;
    return 0;
}
