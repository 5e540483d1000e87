// Public C++ API of the attention runtime - every declaration callers of the reference library use,
// in one header. The per-topic headers next to this file (attention.hpp, kv_cache.hpp, ...) only
// include it, so sources written against the reference's include/scicompute_attention/ compile
// unchanged. Conventions: no exception crosses the API; value-returning calls give sci::Result<T>,
// the others sci::Status; a null stream means sci::Stream::GetCurrent(); inputs are borrowed;
// AttentionResult::out is a newly allocated contiguous [B, H_q, S_q, D] tensor on q's device.
#pragma once

#include <cstddef>
#include <cstdint>
#include <limits>
#include <memory>
#include <string>
#include <vector>

#include "core/status.hpp"
#include "core/types.hpp"
#include "tensor/tensor.hpp"

#if defined(__GNUC__) || defined(__clang__)
#define SCI_ATTENTION_API __attribute__((visibility("default")))
#define SCI_ATTENTION_INTERNAL __attribute__((visibility("hidden")))
#else
#define SCI_ATTENTION_API
#define SCI_ATTENTION_INTERNAL
#endif

#define SCI_ATTENTION_VERSION_MAJOR 0
#define SCI_ATTENTION_VERSION_MINOR 1
#define SCI_ATTENTION_VERSION_PATCH 0
#define SCI_ATTENTION_VERSION_STRING "0.1.0"

namespace sci {
class Stream;
class Device;
}  // namespace sci

namespace sca {

SCI_ATTENTION_API const char* VersionString() noexcept;

// ================================================================================================
// status (reference: include/scicompute_attention/status.hpp)
// ================================================================================================
// Attention-domain codes travel inside the message as "[SCA-<code>] ..." next to the nearest
// sci::StatusCode, so callers can branch on either.
enum class AttnStatusCode : int32_t {
    kOk = 0,
    kUnsupportedHeadDim = 2001,
    kUnsupportedDtype = 2002,
    kUnsupportedLayout = 2003,
    kLayoutMismatch = 2004,
    kShapeMismatch = 2005,
    kSeqTooLong = 2006,
    kKVCapacityExceeded = 2007,
    kWorkspaceExceeded = 2008,
    kUnsupportedFeature = 2009,
    kDeviceCapability = 2010,
};

SCI_ATTENTION_API const char* ToString(AttnStatusCode code) noexcept;
SCI_ATTENTION_API sci::StatusCode ToSciCode(AttnStatusCode code) noexcept;
SCI_ATTENTION_API sci::Status MakeStatus(AttnStatusCode code, std::string detail);
SCI_ATTENTION_API AttnStatusCode ExtractCode(const sci::Status& status) noexcept;
inline bool IsOk(const sci::Status& status) noexcept { return status.ok(); }

// ================================================================================================
// types (attention_types.hpp)
// ================================================================================================
enum class AttnLayout : int32_t { kBHSD = 0, kBSHD = 1 };  // [B,H,S,D] / [B,S,H,D]
enum class KvLayout : int32_t { kBlockMajor = 0 };
enum class BackendKind : int32_t { kAuto = 0, kNaive, kTiled, kFlash, kDecode, kPaged };

struct AttentionShape {
    int64_t batch{0};
    int64_t seq_q{0};
    int64_t seq_kv{0};
    int64_t num_heads{0};
    int64_t num_kv_heads{0};
    int64_t head_dim{0};

    int64_t QueryElements() const noexcept { return batch * seq_q * num_heads * head_dim; }
    int64_t KvElements() const noexcept { return batch * seq_kv * num_kv_heads * head_dim; }
    int64_t OutputElements() const noexcept { return QueryElements(); }
    bool IsGqa() const noexcept { return num_kv_heads > 0 && num_kv_heads != num_heads; }
    int64_t GroupSize() const noexcept { return num_kv_heads > 0 ? num_heads / num_kv_heads : 0; }
};

inline constexpr int64_t kMinSupportedHeadDim = 32;
inline constexpr int64_t kMaxSupportedHeadDim = 256;
inline constexpr int64_t kSupportedHeadDims[] = {32, 64, 96, 128, 160, 192, 256};
inline constexpr int64_t kNumSupportedHeadDims = 7;

SCI_ATTENTION_API int SupportedHeadDimIndex(int64_t head_dim) noexcept;  // -1 when unsupported
SCI_ATTENTION_API const char* LayoutName(AttnLayout layout) noexcept;
SCI_ATTENTION_API const char* BackendName(BackendKind kind) noexcept;
SCI_ATTENTION_API const char* KvLayoutName(KvLayout layout) noexcept;
SCI_ATTENTION_API bool IsSupportedComputeDtype(sci::DType dtype) noexcept;
SCI_ATTENTION_API int64_t DtypeSize(sci::DType dtype) noexcept;

// ================================================================================================
// detail:: helpers that the public types mention (detail/*.hpp)
// ================================================================================================
// block_m: query rows per tile, block_n: keys per pipeline step, warps per CTA, pipeline depth,
// and whether the tiles are moved by the TMA unit.
struct TileConfig {
    int32_t block_m{0};
    int32_t block_n{0};
    int32_t warps{0};
    int32_t stages{0};
    bool use_tma{false};

    constexpr int Threads() const noexcept { return warps * 32; }
    constexpr bool Empty() const noexcept { return block_m == 0 || block_n == 0 || warps == 0; }

    static constexpr int32_t kSmemPadElems = 8;
    // Footprint formula of the reference's padded-row layout (Q + stages * (K + V), 8 pad elements per
    // row); kept because callers compute with it. -1 for a structurally invalid configuration.
    static constexpr int64_t SmemBytesFlash(int32_t head_dim, int64_t elem_bytes, int32_t block_m, int32_t block_n,
                                            int32_t warps, int32_t stages) {
        if (head_dim <= 0 || block_m <= 0 || block_n <= 0 || warps <= 0 || stages <= 0) return -1;
        const int64_t row = (static_cast<int64_t>(head_dim) + kSmemPadElems) * elem_bytes;
        return block_m * row + 2 * static_cast<int64_t>(stages) * block_n * row;
    }
    int64_t SmemBytesFlash(int32_t head_dim, int64_t elem_bytes) const {
        return SmemBytesFlash(head_dim, elem_bytes, block_m, block_n, warps, stages);
    }
    std::string ToString() const {
        return "bm=" + std::to_string(block_m) + ",bn=" + std::to_string(block_n) + ",warps=" + std::to_string(warps) +
               ",stages=" + std::to_string(stages) + (use_tma ? ",tma=on" : ",tma=off");
    }
};

namespace detail {

template <typename T>
inline constexpr T CeilDiv(T value, T divisor) noexcept { return (value + divisor - 1) / divisor; }
template <typename T>
inline constexpr bool IsAligned(T value, T alignment) noexcept { return alignment != 0 && (value % alignment) == 0; }
template <typename T>
inline constexpr T AlignUp(T value, T alignment) noexcept { return CeilDiv(value, alignment) * alignment; }
template <typename T>
inline constexpr T Min(T a, T b) noexcept { return a < b ? a : b; }
template <typename T>
inline constexpr T Max(T a, T b) noexcept { return a > b ? a : b; }

inline bool CheckedMul(int64_t a, int64_t b, int64_t* out) noexcept {
    if (a < 0 || b < 0) return false;
    if (a != 0 && b > std::numeric_limits<int64_t>::max() / a) return false;
    *out = a * b;
    return true;
}
inline bool CheckedMulSize(size_t a, size_t b, size_t* out) noexcept {
    if (a != 0 && b > std::numeric_limits<size_t>::max() / a) return false;
    *out = a * b;
    return true;
}

// Element strides of a [B,H,S,D] or [B,S,H,D] tensor; the head dimension is contiguous.
struct Strides {
    int64_t s_b{0}, s_h{0}, s_s{0}, s_d{0};
};
inline Strides StridesFor(AttnLayout layout, int64_t seq, int64_t heads, int64_t head_dim) {
    Strides s{};
    s.s_d = 1;
    if (layout == AttnLayout::kBHSD) {
        s.s_s = head_dim;
        s.s_h = seq * head_dim;
        s.s_b = heads * seq * head_dim;
    } else {
        s.s_h = head_dim;
        s.s_s = heads * head_dim;
        s.s_b = seq * heads * head_dim;
    }
    return s;
}
inline int64_t Offset(const Strides& s, int64_t b, int64_t h, int64_t t, int64_t d) noexcept {
    return b * s.s_b + h * s.s_h + t * s.s_s + d * s.s_d;
}
inline int64_t OffsetBHSD(int64_t b, int64_t h, int64_t t, int64_t d, int64_t seq, int64_t heads, int64_t head_dim) noexcept {
    return ((b * heads + h) * seq + t) * head_dim + d;
}
inline int64_t OffsetBSHD(int64_t b, int64_t t, int64_t h, int64_t d, int64_t seq, int64_t heads, int64_t head_dim) noexcept {
    return ((b * seq + t) * heads + h) * head_dim + d;
}
inline bool LayoutSupported(AttnLayout layout) noexcept { return layout == AttnLayout::kBHSD || layout == AttnLayout::kBSHD; }

template <sci::DType kDtype>
struct DTypeTraits;
template <>
struct DTypeTraits<sci::DType::kFloat32> {
    using HostType = float;
    static constexpr int64_t kBytes = 4;
    static constexpr bool kSupportsMma = false;
};
template <>
struct DTypeTraits<sci::DType::kFloat16> {
    using HostType = uint16_t;
    static constexpr int64_t kBytes = 2;
    static constexpr bool kSupportsMma = true;
};
template <>
struct DTypeTraits<sci::DType::kBFloat16> {
    using HostType = uint16_t;
    static constexpr int64_t kBytes = 2;
    static constexpr bool kSupportsMma = true;
};
inline constexpr int64_t kMmaK = 16;    // K extent of one tcgen05.mma / mma.sync step for 16-bit inputs
inline constexpr int64_t kMmaM = 16;
inline constexpr int64_t kMmaN = 8;
inline constexpr int64_t kVectorBytes = 16;

}  // namespace detail

// ================================================================================================
// per-call configuration and validation (attention_config.hpp)
// ================================================================================================
struct AttentionConfig {
    BackendKind backend{BackendKind::kAuto};
    AttnLayout layout{AttnLayout::kBHSD};
    bool causal{false};
    bool return_lse{false};
    float scale{0.0f};                 // 0 -> 1/sqrt(head_dim)
    float softcap{0.0f};               // 0 -> off
    int64_t sliding_window{0};         // > 0 is rejected (kUnsupportedFeature)
    int64_t num_splits{0};             // decode split-K; 0 -> automatic
    size_t workspace_limit_bytes{0};   // 0 -> derived from the device
    bool allow_fallback{false};        // false: never degrade silently
    const int32_t* cu_seqlens_q{nullptr};   // varlen: host int32 offsets, length num_seqs + 1
    const int32_t* cu_seqlens_kv{nullptr};
    sci::Stream* stream{nullptr};
};

SCI_ATTENTION_API float EffectiveScale(const AttentionConfig& cfg, const AttentionShape& shape) noexcept;
SCI_ATTENTION_API sci::Status Validate(const AttentionConfig& cfg, const AttentionShape& shape, std::string* detail = nullptr);
SCI_ATTENTION_API TileConfig RecommendTile(const AttentionConfig& cfg, const AttentionShape& shape);
SCI_ATTENTION_API sci::Status ValidateVarlenHost(const int32_t* host_cu_seqlens, int64_t batch, int64_t* max_seq_out = nullptr);

// ================================================================================================
// results (attention_result.hpp)
// ================================================================================================
struct AttentionRuntimeStats {
    BackendKind used_backend{BackendKind::kAuto};
    TileConfig tile{};
    size_t workspace_bytes{0};
    size_t kv_bytes{0};
    std::string note;                        // how the call was executed; any clamp or fallback is named here
    int64_t num_splits{0};                   // decode / paged only
    int64_t materialized_score_bytes{0};     // bytes of a [B,H_q,S_q,S_kv] score matrix written to HBM (0 for flash)
};

struct AttentionResult {
    sci::Tensor out;   // [B, H_q, S_q, D], newly allocated
    sci::Tensor lse;   // fp32 [B, H_q, S_q]; empty unless cfg.return_lse
    AttentionRuntimeStats stats;
};

// ================================================================================================
// backends (backends.hpp)
// ================================================================================================
struct CapabilityReport {
    bool supported{false};
    std::string reason;
    BackendKind recommended_backend{BackendKind::kAuto};
    TileConfig tile{};
    size_t workspace_bytes{0};
};

class SCI_ATTENTION_API IAttentionBackend {
public:
    virtual ~IAttentionBackend() = default;
    virtual BackendKind Kind() const noexcept = 0;
    virtual const char* Name() const noexcept = 0;
    virtual CapabilityReport Supports(const AttentionConfig& cfg, const AttentionShape& shape) const = 0;
    virtual size_t WorkspaceBytes(const AttentionConfig& cfg, const AttentionShape& shape) const = 0;
    virtual sci::Result<AttentionResult> Forward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                                 const AttentionConfig& cfg) const = 0;
    virtual sci::Result<AttentionResult> ForwardVarlen(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                                       int64_t num_seqs, const int32_t* cu_seqlens_q,
                                                       const int32_t* cu_seqlens_kv, int64_t max_seq_q,
                                                       int64_t max_seq_kv, const AttentionConfig& cfg) const = 0;
};

SCI_ATTENTION_API const IAttentionBackend* GetBackend(BackendKind kind) noexcept;  // never null (unknown -> naive)
SCI_ATTENTION_API const char* BackendTypeName(BackendKind kind) noexcept;
SCI_ATTENTION_API bool ParseBackendName(const char* name, BackendKind* out) noexcept;

// ================================================================================================
// device capability (capability.hpp)
// ================================================================================================
struct DeviceCapability {
    std::string device_name;
    int major{0};
    int minor{0};
    int sm_count{0};
    size_t smem_per_sm{0};
    size_t smem_per_block_default{0};
    size_t smem_per_block_optin{0};
    size_t regs_per_sm{0};
    size_t max_threads_per_sm{0};
    size_t l2_bytes{0};
    size_t total_mem_bytes{0};
    size_t free_mem_bytes{0};
    bool has_mma_m16n8k16{false};
    bool has_cp_async{false};
    bool has_tma_bulk{false};
    bool has_wgmma{false};      // always false: sm_100a replaced it with tcgen05
    bool has_fp8_mma{false};
    // Blackwell additions
    bool has_tcgen05{false};
    int tmem_columns{0};
    int max_cluster_size{0};

    SCI_ATTENTION_API static const DeviceCapability& ForDevice(int device_id = 0);  // probes once, then cached
    SCI_ATTENTION_API static sci::Status Refresh(int device_id = 0);
    SCI_ATTENTION_API static size_t SmemLimitPerBlock(const DeviceCapability& cap) noexcept;  // honours SCI_ATTENTION_MAX_SMEM_BYTES
    SCI_ATTENTION_API static bool CudaAvailable() noexcept;
};

// ================================================================================================
// dispatcher (dispatcher.hpp)
// ================================================================================================
struct DispatchDecision {
    BackendKind backend{BackendKind::kAuto};
    TileConfig tile{};
    size_t workspace_bytes{0};
    std::string reason;
};

class SCI_ATTENTION_API AttentionDispatcher {
public:
    AttentionDispatcher() = default;
    explicit AttentionDispatcher(const AttentionConfig& default_cfg) : default_cfg_(default_cfg) {}

    DispatchDecision Select(const AttentionConfig& cfg, const AttentionShape& shape) const;
    sci::Result<AttentionResult> Forward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                         const AttentionConfig& cfg) const;
    sci::Result<AttentionResult> Forward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v) const;
    std::string Explain(const AttentionConfig& cfg, const AttentionShape& shape) const;
    static sci::Status ReloadDispatchTable(const char* path = nullptr);
    const AttentionConfig& DefaultConfig() const noexcept { return default_cfg_; }

private:
    AttentionConfig default_cfg_{};
};

SCI_ATTENTION_API sci::Result<AttentionShape> InferShape(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                                         AttnLayout layout);

// ================================================================================================
// workspace (workspace.hpp)
// ================================================================================================
class SCI_ATTENTION_API Workspace {
public:
    Workspace();
    Workspace(const Workspace&) = default;
    Workspace& operator=(const Workspace&) = default;
    ~Workspace();

    static sci::Result<Workspace> Create(size_t bytes, sci::Device& device);
    void* Data() noexcept;
    const void* Data() const noexcept;
    size_t Bytes() const noexcept;
    bool Valid() const noexcept;
    sci::Result<void*> Slice(size_t offset, size_t bytes, size_t align = 256);
    sci::Status Reset();
    size_t PeakBytes() const noexcept;
    size_t AllocatedSlices() const noexcept;

private:
    struct Impl;
    std::shared_ptr<Impl> impl_;
};

// ================================================================================================
// KV cache (block_manager.hpp, kv_cache.hpp, paged_kv_cache.hpp)
// ================================================================================================
struct BlockTable {
    std::vector<int32_t> host;     // [max_num_seqs, max_blocks_per_seq], -1 = empty
    sci::Tensor device;            // int32 mirror
    uint64_t revision{0};
    uint64_t synced_revision{0};
    int64_t max_num_seqs{0};
    int64_t max_blocks_per_seq{0};
};

// Exclusive LIFO block allocator with a block table; no reference counting, no sharing.
class SCI_ATTENTION_API BlockManager {
public:
    BlockManager() = default;
    static sci::Result<BlockManager> Create(int64_t num_blocks, int64_t max_num_seqs, int64_t max_blocks_per_seq,
                                            sci::Device& device);
    sci::Result<std::vector<int32_t>> Allocate(int64_t count);   // all or nothing
    void Free(const int32_t* block_ids, int64_t count);
    int64_t NumFreeBlocks() const noexcept { return static_cast<int64_t>(free_list_.size()); }
    int64_t NumTotalBlocks() const noexcept { return num_blocks_; }
    int64_t AllocationFailures() const noexcept { return allocation_failures_; }
    int64_t DoubleFreeEvents() const noexcept { return double_free_events_; }
    sci::Status AppendToTable(int64_t seq_id, const int32_t* block_ids, int64_t count);
    sci::Status ResetSeq(int64_t seq_id);
    sci::Status SyncTableToDevice(sci::Stream* stream);
    const BlockTable& Table() const noexcept { return table_; }

private:
    int64_t num_blocks_{0};
    std::vector<int32_t> free_list_;
    std::vector<uint8_t> in_use_;
    BlockTable table_;
    int64_t allocation_failures_{0};
    int64_t double_free_events_{0};
};

struct KVCacheConfig {
    int64_t num_layers{0};
    int64_t num_kv_heads{0};
    int64_t head_dim{0};
    int64_t block_size{16};
    int64_t num_blocks{0};
    int64_t max_num_seqs{1};
    sci::DType dtype{sci::DType::kFloat16};
    KvLayout layout{KvLayout::kBlockMajor};
    bool enable_stats{true};
};

struct KVCacheStats {
    int64_t num_blocks{0};
    int64_t used_blocks{0};
    int64_t free_blocks{0};
    int64_t num_appends{0};
    int64_t num_resets{0};
    size_t peak_bytes{0};
    size_t bytes{0};
};

// Block-major storage: per layer K and V are [num_blocks][block_size][num_kv_heads][head_dim].
class SCI_ATTENTION_API KVCache {
public:
    KVCache() = default;
    static sci::Result<KVCache> Create(const KVCacheConfig& cfg, sci::Device& device);
    // k_new / v_new: [num_tokens, num_kv_heads, head_dim] on the device; slot_mapping: device int32,
    // slot = block * block_size + offset, negative = skip.
    sci::Status Append(int64_t layer, const sci::Tensor& k_new, const sci::Tensor& v_new, const int32_t* slot_mapping,
                       int64_t num_tokens, sci::Stream* stream);
    sci::Result<sci::Tensor> GatherK(int64_t layer, const int32_t* block_ids, int64_t num_blocks, sci::Stream* stream) const;
    sci::Result<sci::Tensor> GatherV(int64_t layer, const int32_t* block_ids, int64_t num_blocks, sci::Stream* stream) const;
    sci::Status Reset(const int32_t* block_ids, int64_t num_blocks, sci::Stream* stream);
    const sci::Tensor& K(int64_t layer) const;
    const sci::Tensor& V(int64_t layer) const;
    KVCacheStats Stats() const;
    size_t MemoryBytes() const noexcept;
    int64_t LayerElements() const noexcept { return layer_elements_; }
    const KVCacheConfig& Config() const noexcept { return cfg_; }

private:
    sci::Result<sci::Tensor> GatherInternal(int64_t layer, const int32_t* block_ids, int64_t num_blocks, bool is_key,
                                            sci::Stream* stream) const;
    KVCacheConfig cfg_{};
    int64_t layer_elements_{0};
    std::vector<sci::Tensor> k_layers_;
    std::vector<sci::Tensor> v_layers_;
    KVCacheStats stats_{};
};

SCI_ATTENTION_API sci::Result<std::vector<int32_t>> ComputeSlotMapping(const int32_t* block_table_row, int64_t seq_start,
                                                                       int64_t num_tokens, int64_t block_size,
                                                                       int64_t max_blocks);
SCI_ATTENTION_API sci::Result<size_t> KvCacheBytes(const KVCacheConfig& cfg);
SCI_ATTENTION_API int64_t MaxBlocksForBudget(const KVCacheConfig& cfg, size_t budget_bytes);

class SCI_ATTENTION_API PagedKVCache {
public:
    PagedKVCache() = default;
    static sci::Result<PagedKVCache> Create(const KVCacheConfig& cfg, sci::Device& device);
    sci::Status AppendTokens(int64_t seq_id, int64_t layer, const sci::Tensor& k_new, const sci::Tensor& v_new,
                             sci::Stream* stream);
    sci::Status ResetSeq(int64_t seq_id, sci::Stream* stream);
    const int32_t* PageTableDevicePtr() const noexcept;
    int64_t LogicalBlockCount(int64_t seq_id) const noexcept;
    int64_t SeqLength(int64_t seq_id) const noexcept;
    int64_t BlockSize() const noexcept { return cfg_.block_size; }
    int64_t MaxBlocksPerSeq() const noexcept { return max_blocks_per_seq_; }
    int64_t MaxNumSeqs() const noexcept { return cfg_.max_num_seqs; }
    const KVCache& Storage() const noexcept { return storage_; }
    KVCache& MutableStorage() noexcept { return storage_; }
    const BlockManager& Blocks() const noexcept { return blocks_; }
    sci::Status SyncPageTable(sci::Stream* stream);
    KVCacheStats Stats() const;
    sci::Status ForceSyncPageTable(sci::Stream* stream);

    // Addition (no counterpart in the reference): appends ONE token to each of the first `num_seqs`
    // sequences with one kernel launch. k_new / v_new are [num_seqs, num_kv_heads, head_dim]. Block
    // allocation, table rows and lengths change exactly as num_seqs AppendTokens calls in sequence order
    // would change them; only the rows that changed are uploaded. On failure nothing has changed.
    sci::Status AppendTokenBatch(int64_t num_seqs, int64_t layer, const sci::Tensor& k_new, const sci::Tensor& v_new,
                                 sci::Stream* stream);
    // Device int32 [max_num_seqs] sequence lengths as of the last AppendTokenBatch / SyncPageTable.
    const int32_t* SeqLensDevicePtr() const noexcept;
    // Addition: device int32 permutation of [0, num_seqs), longest sequence first as of the last table
    // sync - a scheduling hint for paged_attention (thread blocks of long sequences start first). Null
    // when the stored order does not reduce to a permutation of the first `num_seqs` slots.
    const int32_t* SeqOrderDevicePtr(int64_t num_seqs) const noexcept;

private:
    KVCacheConfig cfg_{};
    int64_t max_blocks_per_seq_{0};
    KVCache storage_{};
    BlockManager blocks_{};
    std::vector<int64_t> seq_lengths_;
    std::vector<std::vector<int32_t>> seq_blocks_;
    std::vector<int32_t> page_table_host_;
    sci::Tensor page_table_device_;
    sci::Tensor slot_mapping_device_;
    int64_t slot_mapping_capacity_{0};
    uint64_t revision_{0};
    uint64_t synced_revision_{0};
    int64_t num_appends_{0};
    int64_t num_resets_{0};
    // incremental sync state (additions): leading entries of each device row that may differ from -1
    std::vector<int64_t> live_on_device_;
    sci::Tensor seq_lens_device_;
    sci::Tensor seq_order_device_;
    int64_t seq_order_extent_{-1};  // slots at or beyond this index were empty when the order was built; -1 = none built
};

// ================================================================================================
// entry points (attention.hpp, flash_attention.hpp, decode_attention.hpp, paged_attention.hpp, ...)
// ================================================================================================
SCI_ATTENTION_API sci::Result<AttentionResult> attention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                                         const AttentionConfig& cfg = {});
inline sci::Result<AttentionResult> flash(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                          const AttentionConfig& cfg = {}) {
    AttentionConfig c = cfg;
    c.backend = BackendKind::kFlash;
    return attention(q, k, v, c);
}
SCI_ATTENTION_API sci::Result<AttentionResult> decode(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                                      const AttentionConfig& cfg = {});
SCI_ATTENTION_API sci::Result<AttentionResult> paged(const sci::Tensor& q, const PagedKVCache& kv,
                                                     const AttentionConfig& cfg = {});
SCI_ATTENTION_API std::string ExplainAttention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                               const AttentionConfig& cfg = {});

SCI_ATTENTION_API sci::Result<AttentionResult> naive_attention(const sci::Tensor& q, const sci::Tensor& k,
                                                               const sci::Tensor& v, const AttentionConfig& cfg);
SCI_ATTENTION_API sci::Result<AttentionResult> tiled_attention(const sci::Tensor& q, const sci::Tensor& k,
                                                               const sci::Tensor& v, const AttentionConfig& cfg);
SCI_ATTENTION_API sci::Result<AttentionResult> flash_attention(const sci::Tensor& q, const sci::Tensor& k,
                                                               const sci::Tensor& v, const AttentionConfig& cfg);
// Packed batches: q [total_q, H_q, D], k/v [total_kv, H_kv, D]; cu_seqlens_* are HOST int32 arrays of
// length num_seqs + 1, strictly increasing from 0. LSE is not available here.
SCI_ATTENTION_API sci::Result<AttentionResult> flash_attention_varlen(const sci::Tensor& q, const sci::Tensor& k,
                                                                      const sci::Tensor& v, int64_t num_seqs,
                                                                      const int32_t* cu_seqlens_q,
                                                                      const int32_t* cu_seqlens_kv, int64_t max_seq_q,
                                                                      int64_t max_seq_kv, const AttentionConfig& cfg);

// Addition (no counterpart in the reference): whether every flash launch on `device_id` so far ran to completion.
// All waits inside the flash kernel are bounded; a launch whose wait ran out leaves its output undefined, and this
// call - made after synchronising the stream - is how a caller learns of it (kCudaError with the role that gave
// up). Reading clears the record.
SCI_ATTENTION_API sci::Status FlashLaunchStatus(int device_id = 0);

struct DecodeConfig {
    int64_t num_splits{0};   // 0 -> automatic
    int64_t max_splits{64};  // cap of the automatic choice on B200 (the reference's laptop-GPU table stops at 16)
    bool use_splitk{true};
};
SCI_ATTENTION_API DecodeConfig RecommendDecodeConfig(const AttentionShape& shape, const DeviceCapability& cap);
SCI_ATTENTION_API sci::Result<AttentionResult> decode_attention(const sci::Tensor& q, const sci::Tensor& k,
                                                                const sci::Tensor& v, const AttentionConfig& cfg);
SCI_ATTENTION_API sci::Result<AttentionResult> decode_attention(const sci::Tensor& q, const sci::Tensor& k,
                                                                const sci::Tensor& v, const AttentionConfig& cfg,
                                                                const DecodeConfig& decode_cfg);

struct PagedAttentionParams {
    const int32_t* page_table{nullptr};  // device [num_seqs, max_blocks_per_seq]
    const int32_t* seq_lens{nullptr};    // device [num_seqs], includes the new token
    int64_t num_seqs{0};
    int64_t block_size{16};
    int64_t max_blocks_per_seq{0};
    int64_t layer{0};
};
SCI_ATTENTION_API sci::Result<AttentionResult> paged_attention(const sci::Tensor& q, const PagedKVCache& kv,
                                                               const PagedAttentionParams& params,
                                                               const AttentionConfig& cfg);
SCI_ATTENTION_API sci::Result<AttentionResult> paged_attention(const sci::Tensor& q, const PagedKVCache& kv,
                                                               const AttentionConfig& cfg);
// Addition (no counterpart in the reference, which names it as the step after the packed prefill:
// docs/flash_attention.md:95): chunked prefill over the paged cache in one launch. `q` holds the NEW tokens of
// `num_seqs` sequences packed as [total_q, H_q, D] (sequence s = cache slot s); cu_seqlens_q is a HOST int32 array of
// num_seqs + 1 offsets. The keys and values of those tokens must already be in the cache (AppendTokens, then
// SyncPageTable): sequence s attends over its kv.SeqLength(s) cached tokens with the bottom-right aligned causal
// mask. Returns out [total_q, H_q, D]. fp16 / bf16, block sizes 8 / 16 / 32 / 64.
SCI_ATTENTION_API sci::Result<AttentionResult> paged_prefill(const sci::Tensor& q, const PagedKVCache& kv, int64_t num_seqs,
                                                             const int32_t* cu_seqlens_q, int64_t layer,
                                                             const AttentionConfig& cfg);

}  // namespace sca
