// TEST INFRASTRUCTURE - C-ABI wrapper around the REFERENCE'S OWN host code. Not part of the product.
//
// oracle/build_ref.sh compiles this file together with the reference's unmodified sources (where
// they lie in the reference checkout, CPU-only "stub" mode) into oracle/_ref/libsca_ref.so. The
// library exists to pin oracle/*.c against the real thing and to generate tests/golden/*.json; it
// is never shipped and never loaded by the product.
//
// Wrapped reference code:
//   tests/common/test_utils.hpp                RandomFloats, fp16/bf16 rounding, ReferenceAttention
//   src/kv_cache/block_manager.cpp             BlockManager
//   src/kv_cache/kv_cache.cpp                  ComputeSlotMapping, KvCacheBytes, MaxBlocksForBudget
//   src/kv_cache/paged_kv_cache.cpp            PagedKVCache bookkeeping
//   src/api/api_validate.cpp, src/api/status.cpp   Validate, EffectiveScale, status mapping
//   src/runtime/dispatcher.cpp                 AttentionDispatcher::Select / Explain
// The three KV data-movement launchers, which the reference's CPU build stubs out with an error,
// are defined here as byte copies that follow src/kv_cache/kv_cache_kernels.cu:17-86, so that
// PagedKVCache::AppendTokens runs to completion on the host.
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "common/test_utils.hpp"
#include "kv_cache/kv_cache_kernels.cuh"
#include "scicompute_attention/attention.hpp"

namespace sca {
namespace cuda {

sci::Status LaunchKvAppend(void* layer_k, void* layer_v, const void* k_new, const void* v_new,
                           const int32_t* slots, int64_t num_tokens, const KVCacheShape& shape,
                           int64_t elem_bytes, sci::Stream*) {
    if (!layer_k || !layer_v || !k_new || !v_new || !slots)
        return sci::Status::InvalidArgument("kv append: null pointer");
    if (num_tokens <= 0) return sci::Status::InvalidArgument("kv append: num_tokens <= 0");
    const int64_t row_bytes = shape.head_dim * elem_bytes;
    for (int64_t t = 0; t < num_tokens; ++t) {
        const int32_t slot = slots[t];
        if (slot < 0) continue;
        const int64_t block = slot / shape.block_size;
        const int64_t off = slot % shape.block_size;
        if (block >= shape.num_blocks) continue;
        for (int64_t h = 0; h < shape.num_kv_heads; ++h) {
            const int64_t dst = KvOffset(shape, block, off, h, 0) * elem_bytes;
            const int64_t src = (t * shape.num_kv_heads + h) * row_bytes;
            std::memcpy(static_cast<uint8_t*>(layer_k) + dst, static_cast<const uint8_t*>(k_new) + src, row_bytes);
            std::memcpy(static_cast<uint8_t*>(layer_v) + dst, static_cast<const uint8_t*>(v_new) + src, row_bytes);
        }
    }
    return sci::Status::Ok();
}

sci::Status LaunchKvResetBlock(void* layer_k, void* layer_v, const int32_t* ids, int64_t count,
                               const KVCacheShape& shape, int64_t elem_bytes, sci::Stream*) {
    if (!layer_k || !layer_v || !ids) return sci::Status::InvalidArgument("kv reset: null pointer");
    const int64_t per_block = shape.block_size * shape.num_kv_heads * shape.head_dim * elem_bytes;
    for (int64_t i = 0; i < count; ++i) {
        if (ids[i] < 0 || ids[i] >= shape.num_blocks) continue;
        std::memset(static_cast<uint8_t*>(layer_k) + ids[i] * per_block, 0, per_block);
        std::memset(static_cast<uint8_t*>(layer_v) + ids[i] * per_block, 0, per_block);
    }
    return sci::Status::Ok();
}

sci::Status LaunchKvGather(const void* layer, const int32_t* ids, int64_t count, void* out,
                           const KVCacheShape& shape, int64_t elem_bytes, sci::Stream*) {
    if (!layer || !ids || !out) return sci::Status::InvalidArgument("kv gather: null pointer");
    const int64_t per_block = shape.block_size * shape.num_kv_heads * shape.head_dim * elem_bytes;
    for (int64_t i = 0; i < count; ++i) {
        uint8_t* dst = static_cast<uint8_t*>(out) + i * per_block;
        if (ids[i] < 0 || ids[i] >= shape.num_blocks) std::memset(dst, 0, per_block);
        else std::memcpy(dst, static_cast<const uint8_t*>(layer) + ids[i] * per_block, per_block);
    }
    return sci::Status::Ok();
}

}  // namespace cuda
}  // namespace sca

namespace {

int CopyMessage(const std::string& text, char* out, int cap) {
    if (out != nullptr && cap > 0) {
        std::strncpy(out, text.c_str(), static_cast<size_t>(cap - 1));
        out[cap - 1] = '\0';
    }
    return static_cast<int>(text.size());
}

sca::AttentionShape MakeShape(const int64_t* s) {
    sca::AttentionShape shape;
    shape.batch = s[0];
    shape.seq_q = s[1];
    shape.seq_kv = s[2];
    shape.num_heads = s[3];
    shape.num_kv_heads = s[4];
    shape.head_dim = s[5];
    return shape;
}

// cfg as a flat record: backend, layout, causal, return_lse, sliding_window, num_splits,
// allow_fallback, has_cu_q, has_cu_kv (ints) + scale, softcap (floats).
sca::AttentionConfig MakeConfig(const int64_t* ci, const float* cf) {
    static const int32_t kDummy[2] = {0, 1};
    sca::AttentionConfig cfg;
    cfg.backend = static_cast<sca::BackendKind>(ci[0]);
    cfg.layout = static_cast<sca::AttnLayout>(ci[1]);
    cfg.causal = ci[2] != 0;
    cfg.return_lse = ci[3] != 0;
    cfg.sliding_window = ci[4];
    cfg.num_splits = ci[5];
    cfg.allow_fallback = ci[6] != 0;
    cfg.cu_seqlens_q = ci[7] != 0 ? kDummy : nullptr;
    cfg.cu_seqlens_kv = ci[8] != 0 ? kDummy : nullptr;
    cfg.scale = cf[0];
    cfg.softcap = cf[1];
    return cfg;
}

struct RefPaged {
    sca::PagedKVCache cache;
    sca::KVCacheConfig cfg;
};

}  // namespace

extern "C" {

void ref_random_floats(float* out, uint64_t count, uint32_t seed, float low, float high) {
    const std::vector<float> v = sca_test::RandomFloats(count, seed, low, high);
    std::memcpy(out, v.data(), count * sizeof(float));
}
uint16_t ref_float_to_half_bits(float v) { return sca_test::FloatToHalfBits(v); }
float ref_half_bits_to_float(uint16_t h) { return sca_test::HalfBitsToFloat(h); }
uint16_t ref_float_to_bf16_bits(float v) { return sca_test::FloatToBf16Bits(v); }
float ref_bf16_bits_to_float(uint16_t h) { return sca_test::Bf16BitsToFloat(h); }

void ref_attention(const float* q, const float* k, const float* v, int64_t batch, int64_t heads_q,
                   int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int64_t head_dim, int causal,
                   double* out) {
    const std::vector<float> qv(q, q + batch * heads_q * seq_q * head_dim);
    const std::vector<float> kv(k, k + batch * heads_kv * seq_kv * head_dim);
    const std::vector<float> vv(v, v + batch * heads_kv * seq_kv * head_dim);
    const std::vector<double> r = sca_test::ReferenceAttention(qv, kv, vv, batch, heads_q, heads_kv,
                                                               seq_q, seq_kv, head_dim, causal != 0);
    std::memcpy(out, r.data(), r.size() * sizeof(double));
}

void ref_tolerance(int dtype, double* max_abs, double* mean_abs) {
    const sca_test::Tolerance t = sca_test::ToleranceFor(static_cast<sci::DType>(dtype), false);
    *max_abs = t.max_abs;
    *mean_abs = t.mean_abs;
}

// ---- BlockManager -------------------------------------------------------------------------
void* ref_bm_create(int64_t num_blocks, int64_t max_seqs, int64_t max_blocks_per_seq, char* msg, int cap) {
    sci::Result<sca::BlockManager> r =
        sca::BlockManager::Create(num_blocks, max_seqs, max_blocks_per_seq, sci::StubHostDevice());
    if (!r.ok()) {
        CopyMessage(r.message(), msg, cap);
        return nullptr;
    }
    return new sca::BlockManager(std::move(*r));
}
void ref_bm_destroy(void* h) { delete static_cast<sca::BlockManager*>(h); }
int ref_bm_allocate(void* h, int64_t count, int32_t* out, char* msg, int cap) {
    sci::Result<std::vector<int32_t>> r = static_cast<sca::BlockManager*>(h)->Allocate(count);
    if (!r.ok()) {
        CopyMessage(r.message(), msg, cap);
        return static_cast<int>(sca::ExtractCode(r.error()));
    }
    std::memcpy(out, r->data(), r->size() * sizeof(int32_t));
    return 0;
}
void ref_bm_free(void* h, const int32_t* ids, int64_t count) {
    static_cast<sca::BlockManager*>(h)->Free(ids, count);
}
int ref_bm_append_to_table(void* h, int64_t seq, const int32_t* ids, int64_t count, char* msg, int cap) {
    const sci::Status s = static_cast<sca::BlockManager*>(h)->AppendToTable(seq, ids, count);
    CopyMessage(s.message(), msg, cap);
    return static_cast<int>(sca::ExtractCode(s));
}
int ref_bm_reset_seq(void* h, int64_t seq) {
    return static_cast<int>(sca::ExtractCode(static_cast<sca::BlockManager*>(h)->ResetSeq(seq)));
}
int64_t ref_bm_num_free(void* h) { return static_cast<sca::BlockManager*>(h)->NumFreeBlocks(); }
int64_t ref_bm_allocation_failures(void* h) { return static_cast<sca::BlockManager*>(h)->AllocationFailures(); }
int64_t ref_bm_double_free_events(void* h) { return static_cast<sca::BlockManager*>(h)->DoubleFreeEvents(); }
uint64_t ref_bm_revision(void* h) { return static_cast<sca::BlockManager*>(h)->Table().revision; }
const int32_t* ref_bm_table(void* h) { return static_cast<sca::BlockManager*>(h)->Table().host.data(); }

// ---- slot mapping / budget ---------------------------------------------------------------------
int ref_slot_mapping(const int32_t* row, int64_t start, int64_t n, int64_t bs, int64_t max_blocks,
                     int32_t* out, char* msg, int cap) {
    sci::Result<std::vector<int32_t>> r = sca::ComputeSlotMapping(row, start, n, bs, max_blocks);
    if (!r.ok()) {
        CopyMessage(r.message(), msg, cap);
        return static_cast<int>(sca::ExtractCode(r.error()));
    }
    std::memcpy(out, r->data(), r->size() * sizeof(int32_t));
    return 0;
}

static sca::KVCacheConfig KvCfg(int64_t layers, int64_t blocks, int64_t bs, int64_t hkv, int64_t d,
                                int dtype, int64_t max_seqs) {
    sca::KVCacheConfig cfg;
    cfg.num_layers = layers;
    cfg.num_blocks = blocks;
    cfg.block_size = bs;
    cfg.num_kv_heads = hkv;
    cfg.head_dim = d;
    cfg.dtype = static_cast<sci::DType>(dtype);
    cfg.max_num_seqs = max_seqs;
    return cfg;
}

int64_t ref_kv_cache_bytes(int64_t layers, int64_t blocks, int64_t bs, int64_t hkv, int64_t d,
                           int dtype, char* msg, int cap) {
    sci::Result<size_t> r = sca::KvCacheBytes(KvCfg(layers, blocks, bs, hkv, d, dtype, 1));
    if (!r.ok()) {
        CopyMessage(r.message(), msg, cap);
        return -static_cast<int64_t>(sca::ExtractCode(r.error()));
    }
    return static_cast<int64_t>(*r);
}
int64_t ref_max_blocks_for_budget(int64_t layers, int64_t bs, int64_t hkv, int64_t d, int dtype,
                                  uint64_t budget) {
    return sca::MaxBlocksForBudget(KvCfg(layers, 1, bs, hkv, d, dtype, 1), budget);
}

// ---- PagedKVCache ---------------------------------------------------------------------------------
void* ref_paged_create(int64_t layers, int64_t blocks, int64_t bs, int64_t hkv, int64_t d, int dtype,
                       int64_t max_seqs, char* msg, int cap) {
    const sca::KVCacheConfig cfg = KvCfg(layers, blocks, bs, hkv, d, dtype, max_seqs);
    sci::Result<sca::PagedKVCache> r = sca::PagedKVCache::Create(cfg, sci::StubHostDevice());
    if (!r.ok()) {
        CopyMessage(r.message(), msg, cap);
        return nullptr;
    }
    auto* p = new RefPaged{std::move(*r), cfg};
    return p;
}
void ref_paged_destroy(void* h) { delete static_cast<RefPaged*>(h); }
int ref_paged_append(void* h, int64_t seq, int64_t layer, const void* k_new, const void* v_new,
                     int64_t n, char* msg, int cap) {
    auto* p = static_cast<RefPaged*>(h);
    const sci::TensorShape shape({n, p->cfg.num_kv_heads, p->cfg.head_dim});
    sci::Tensor kt(shape, p->cfg.dtype, sci::StubHostDevice(), const_cast<void*>(k_new), false);
    sci::Tensor vt(shape, p->cfg.dtype, sci::StubHostDevice(), const_cast<void*>(v_new), false);
    const sci::Status s = p->cache.AppendTokens(seq, layer, kt, vt, nullptr);
    CopyMessage(s.message(), msg, cap);
    return static_cast<int>(sca::ExtractCode(s));
}
int ref_paged_reset_seq(void* h, int64_t seq) {
    return static_cast<int>(sca::ExtractCode(static_cast<RefPaged*>(h)->cache.ResetSeq(seq, nullptr)));
}
int64_t ref_paged_seq_length(void* h, int64_t seq) { return static_cast<RefPaged*>(h)->cache.SeqLength(seq); }
int64_t ref_paged_logical_blocks(void* h, int64_t seq) { return static_cast<RefPaged*>(h)->cache.LogicalBlockCount(seq); }
int64_t ref_paged_max_blocks_per_seq(void* h) { return static_cast<RefPaged*>(h)->cache.MaxBlocksPerSeq(); }
const int32_t* ref_paged_synced_table(void* h) {
    auto* p = static_cast<RefPaged*>(h);
    p->cache.SyncPageTable(nullptr);
    return p->cache.PageTableDevicePtr();
}
const void* ref_paged_layer(void* h, int64_t layer, int is_key) {
    auto* p = static_cast<RefPaged*>(h);
    return is_key ? p->cache.Storage().K(layer).data() : p->cache.Storage().V(layer).data();
}
void ref_paged_stats(void* h, int64_t* out7) {
    const sca::KVCacheStats s = static_cast<RefPaged*>(h)->cache.Stats();
    out7[0] = s.num_blocks;
    out7[1] = s.used_blocks;
    out7[2] = s.free_blocks;
    out7[3] = s.num_appends;
    out7[4] = s.num_resets;
    out7[5] = static_cast<int64_t>(s.peak_bytes);
    out7[6] = static_cast<int64_t>(s.bytes);
}

// ---- validation / dispatch ---------------------------------------------------------------------------
int ref_validate(const int64_t* cfg_i, const float* cfg_f, const int64_t* shape, char* msg, int cap) {
    std::string detail;
    const sci::Status s = sca::Validate(MakeConfig(cfg_i, cfg_f), MakeShape(shape), &detail);
    CopyMessage(s.ok() ? detail : s.message(), msg, cap);
    return static_cast<int>(sca::ExtractCode(s));
}
float ref_effective_scale(const int64_t* cfg_i, const float* cfg_f, const int64_t* shape) {
    return sca::EffectiveScale(MakeConfig(cfg_i, cfg_f), MakeShape(shape));
}
int ref_select(const int64_t* cfg_i, const float* cfg_f, const int64_t* shape, char* reason, int cap) {
    const sca::AttentionDispatcher d;
    const sca::DispatchDecision dec = d.Select(MakeConfig(cfg_i, cfg_f), MakeShape(shape));
    CopyMessage(dec.reason, reason, cap);
    return static_cast<int>(dec.backend);
}
int ref_explain(const int64_t* cfg_i, const float* cfg_f, const int64_t* shape, char* out, int cap) {
    const sca::AttentionDispatcher d;
    return CopyMessage(d.Explain(MakeConfig(cfg_i, cfg_f), MakeShape(shape)), out, cap);
}
int ref_status_info(int attn_code, int* sci_code, char* name, int cap) {
    const auto code = static_cast<sca::AttnStatusCode>(attn_code);
    *sci_code = static_cast<int>(sca::ToSciCode(code));
    CopyMessage(sca::ToString(code), name, cap);
    const sci::Status s = sca::MakeStatus(code, "x");
    return static_cast<int>(sca::ExtractCode(s));
}
int ref_varlen_validate(const int32_t* cu, int64_t batch, int64_t* max_seq, char* msg, int cap) {
    const sci::Status s = sca::ValidateVarlenHost(cu, batch, max_seq);
    CopyMessage(s.message(), msg, cap);
    return static_cast<int>(sca::ExtractCode(s));
}

}  // extern "C"
