// Status mapping, names, the single validation entry point, and the geometry tables.
// Behaviour (codes and message wording) follows src/api/status.cpp, src/api/api_validate.cpp and
// src/api/attention_api.cpp of the reference, whose tests assert on field names and values.
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "internal.hpp"

namespace sca {

const char* VersionString() noexcept { return SCI_ATTENTION_VERSION_STRING; }

// ---- status -------------------------------------------------------------------------------------------
namespace {
struct CodeRow {
    AttnStatusCode code;
    const char* name;
    sci::StatusCode sci_code;
};
constexpr CodeRow kCodes[] = {
    {AttnStatusCode::kOk, "OK", sci::StatusCode::kOk},
    {AttnStatusCode::kUnsupportedHeadDim, "UnsupportedHeadDim", sci::StatusCode::kInvalidArgument},
    {AttnStatusCode::kUnsupportedDtype, "UnsupportedDtype", sci::StatusCode::kInvalidArgument},
    {AttnStatusCode::kUnsupportedLayout, "UnsupportedLayout", sci::StatusCode::kInvalidArgument},
    {AttnStatusCode::kLayoutMismatch, "LayoutMismatch", sci::StatusCode::kInvalidArgument},
    {AttnStatusCode::kShapeMismatch, "ShapeMismatch", sci::StatusCode::kInvalidArgument},
    {AttnStatusCode::kSeqTooLong, "SeqTooLong", sci::StatusCode::kInvalidArgument},
    {AttnStatusCode::kKVCapacityExceeded, "KVCapacityExceeded", sci::StatusCode::kResourceExhausted},
    {AttnStatusCode::kWorkspaceExceeded, "WorkspaceExceeded", sci::StatusCode::kResourceExhausted},
    {AttnStatusCode::kUnsupportedFeature, "UnsupportedFeature", sci::StatusCode::kNotImplemented},
    {AttnStatusCode::kDeviceCapability, "DeviceCapability", sci::StatusCode::kInvalidOperation},
};
const CodeRow* FindCode(AttnStatusCode code) {
    for (const CodeRow& row : kCodes) {
        if (row.code == code) return &row;
    }
    return nullptr;
}
}  // namespace

const char* ToString(AttnStatusCode code) noexcept {
    const CodeRow* row = FindCode(code);
    return row != nullptr ? row->name : "UnknownAttnStatus";
}

sci::StatusCode ToSciCode(AttnStatusCode code) noexcept {
    const CodeRow* row = FindCode(code);
    return row != nullptr ? row->sci_code : sci::StatusCode::kError;
}

sci::Status MakeStatus(AttnStatusCode code, std::string detail) {
    return sci::Status(ToSciCode(code), "[SCA-" + std::to_string(static_cast<int32_t>(code)) + "] " + detail);
}

AttnStatusCode ExtractCode(const sci::Status& status) noexcept {
    const std::string& text = status.message();
    const size_t at = text.find("[SCA-");
    if (at == std::string::npos) return AttnStatusCode::kOk;
    return static_cast<AttnStatusCode>(std::atoi(text.c_str() + at + 5));
}

// ---- names ----------------------------------------------------------------------------------------------
int SupportedHeadDimIndex(int64_t head_dim) noexcept {
    for (int i = 0; i < kNumSupportedHeadDims; ++i) {
        if (kSupportedHeadDims[i] == head_dim) return i;
    }
    return -1;
}

const char* LayoutName(AttnLayout layout) noexcept {
    return layout == AttnLayout::kBHSD ? "bhsd" : layout == AttnLayout::kBSHD ? "bshd" : "unknown-layout";
}
const char* KvLayoutName(KvLayout layout) noexcept {
    return layout == KvLayout::kBlockMajor ? "block-major" : "unknown-kv-layout";
}
const char* BackendName(BackendKind kind) noexcept {
    switch (kind) {
        case BackendKind::kAuto: return "auto";
        case BackendKind::kNaive: return "naive";
        case BackendKind::kTiled: return "tiled";
        case BackendKind::kFlash: return "flash";
        case BackendKind::kDecode: return "decode";
        case BackendKind::kPaged: return "paged";
    }
    return "unknown-backend";
}
const char* BackendTypeName(BackendKind kind) noexcept { return BackendName(kind); }

bool ParseBackendName(const char* name, BackendKind* out) noexcept {
    if (name == nullptr || out == nullptr) return false;
    for (BackendKind kind : {BackendKind::kAuto, BackendKind::kNaive, BackendKind::kTiled, BackendKind::kFlash,
                             BackendKind::kDecode, BackendKind::kPaged}) {
        if (std::strcmp(name, BackendName(kind)) == 0) {
            *out = kind;
            return true;
        }
    }
    return false;
}

bool IsSupportedComputeDtype(sci::DType dtype) noexcept {
    return dtype == sci::DType::kFloat32 || dtype == sci::DType::kFloat16 || dtype == sci::DType::kBFloat16;
}
int64_t DtypeSize(sci::DType dtype) noexcept { return static_cast<int64_t>(sci::kDTypeSize(dtype)); }

const IAttentionBackend* GetBackend(BackendKind kind) noexcept {
    switch (kind) {
        case BackendKind::kTiled: return runtime::TiledBackendInstance();
        case BackendKind::kFlash: return runtime::FlashBackendInstance();
        case BackendKind::kDecode: return runtime::DecodeBackendInstance();
        case BackendKind::kPaged: return runtime::PagedBackendInstance();
        default: return runtime::NaiveBackendInstance();
    }
}

// ---- validation -------------------------------------------------------------------------------------------
float EffectiveScale(const AttentionConfig& cfg, const AttentionShape& shape) noexcept {
    if (cfg.scale > 0.0f) return cfg.scale;
    if (shape.head_dim <= 0) return 0.0f;
    return static_cast<float>(1.0 / std::sqrt(static_cast<double>(shape.head_dim)));
}

sci::Status Validate(const AttentionConfig& cfg, const AttentionShape& shape, std::string* detail) {
    AttnStatusCode code = AttnStatusCode::kOk;
    std::string msg;
    auto reject = [&](AttnStatusCode c, std::string text) {
        code = c;
        msg = std::move(text);
    };
    auto at_least_one = [&](const char* field, int64_t value) {
        if (code == AttnStatusCode::kOk && value < 1) {
            reject(AttnStatusCode::kShapeMismatch,
                   std::string("AttentionShape invalid: ") + field + "=" + std::to_string(value) + " (must be >= 1)");
        }
    };
    const bool reference_level = cfg.backend == BackendKind::kNaive || cfg.backend == BackendKind::kTiled ||
                                 cfg.backend == BackendKind::kDecode || cfg.backend == BackendKind::kPaged;

    if (!detail::LayoutSupported(cfg.layout)) {
        reject(AttnStatusCode::kUnsupportedLayout,
               "AttentionConfig invalid: layout=" + std::to_string(static_cast<int>(cfg.layout)) + " (supported: bhsd, bshd)");
    }
    at_least_one("batch", shape.batch);
    at_least_one("seq_q", shape.seq_q);
    at_least_one("seq_kv", shape.seq_kv);
    at_least_one("num_heads", shape.num_heads);
    at_least_one("num_kv_heads", shape.num_kv_heads);
    if (code == AttnStatusCode::kOk) {
        if (SupportedHeadDimIndex(shape.head_dim) < 0) {
            std::string list;
            for (int i = 0; i < kNumSupportedHeadDims; ++i) list += (i ? "," : "") + std::to_string(kSupportedHeadDims[i]);
            reject(AttnStatusCode::kUnsupportedHeadDim,
                   "AttentionConfig invalid: head_dim=" + std::to_string(shape.head_dim) + " (supported: " + list + ")");
        } else if (shape.num_heads % shape.num_kv_heads != 0) {
            reject(AttnStatusCode::kShapeMismatch,
                   "AttentionShape invalid: num_heads=" + std::to_string(shape.num_heads) + " % num_kv_heads=" +
                       std::to_string(shape.num_kv_heads) + " != 0 (GQA requires an integer group size)");
        } else if (cfg.causal && shape.seq_kv < shape.seq_q) {
            reject(AttnStatusCode::kShapeMismatch, "AttentionConfig invalid: causal=true but seq_kv(" +
                                                       std::to_string(shape.seq_kv) + ") < seq_q(" +
                                                       std::to_string(shape.seq_q) + ")");
        } else if (shape.num_kv_heads > shape.num_heads) {
            reject(AttnStatusCode::kShapeMismatch,
                   "AttentionShape invalid: num_kv_heads=" + std::to_string(shape.num_kv_heads) + " > num_heads=" +
                       std::to_string(shape.num_heads) + " (MQA/GQA require H_kv <= H_q)");
        } else if (cfg.sliding_window > 0) {
            reject(AttnStatusCode::kUnsupportedFeature, "AttentionConfig invalid: sliding_window=" +
                                                            std::to_string(cfg.sliding_window) +
                                                            " is not implemented in v1 (see README Roadmap)");
        } else if (cfg.softcap < 0.0f) {
            reject(AttnStatusCode::kShapeMismatch,
                   "AttentionConfig invalid: softcap=" + std::to_string(cfg.softcap) + " (must be 0 or > 0)");
        } else if (cfg.softcap > 0.0f && reference_level) {
            reject(AttnStatusCode::kUnsupportedFeature,
                   "AttentionConfig invalid: softcap=" + std::to_string(cfg.softcap) +
                       " is implemented in the flash backend only, backend=" + BackendName(cfg.backend));
        } else if (cfg.scale < 0.0f) {
            reject(AttnStatusCode::kShapeMismatch, "AttentionConfig invalid: scale=" + std::to_string(cfg.scale) +
                                                       " (must be 0 for the 1/sqrt(head_dim) default or > 0)");
        } else if (cfg.num_splits < 0) {
            reject(AttnStatusCode::kShapeMismatch,
                   "AttentionConfig invalid: num_splits=" + std::to_string(cfg.num_splits) + " (must be >= 0)");
        } else if (cfg.cu_seqlens_q != nullptr && cfg.cu_seqlens_kv == nullptr) {
            reject(AttnStatusCode::kShapeMismatch, "AttentionConfig invalid: cu_seqlens_q is set but cu_seqlens_kv is null");
        }
    }
    if (code == AttnStatusCode::kOk) {
        if (detail != nullptr) *detail = "ok";
        return sci::Status::Ok();
    }
    if (detail != nullptr) *detail = msg;
    return MakeStatus(code, msg);
}

TileConfig RecommendTile(const AttentionConfig&, const AttentionShape& shape) {
    TileConfig tile;
    if (const tables::FlashTile* entry = tables::FindFlashTile(shape.head_dim)) {
        tile.block_m = entry->block_m;
        tile.block_n = entry->block_n;
        tile.warps = entry->warps;
        tile.stages = entry->stages;
        tile.use_tma = true;
    }
    return tile;
}

sci::Status ValidateVarlenHost(const int32_t* host_cu_seqlens, int64_t batch, int64_t* max_seq_out) {
    if (host_cu_seqlens == nullptr) return MakeStatus(AttnStatusCode::kShapeMismatch, "cu_seqlens is null");
    if (batch < 1) {
        return MakeStatus(AttnStatusCode::kShapeMismatch, "varlen batch=" + std::to_string(batch) + " (must be >= 1)");
    }
    if (host_cu_seqlens[0] != 0) {
        return MakeStatus(AttnStatusCode::kShapeMismatch,
                          "cu_seqlens[0]=" + std::to_string(host_cu_seqlens[0]) + " (must start at 0)");
    }
    int64_t longest = 0;
    for (int64_t i = 0; i < batch; ++i) {
        const int32_t lo = host_cu_seqlens[i], hi = host_cu_seqlens[i + 1];
        if (hi <= lo) {
            return MakeStatus(AttnStatusCode::kShapeMismatch, "cu_seqlens not strictly increasing at index " +
                                                                  std::to_string(i) + ": [" + std::to_string(lo) + ", " +
                                                                  std::to_string(hi) + "]");
        }
        longest = detail::Max<int64_t>(longest, hi - lo);
    }
    if (max_seq_out != nullptr) *max_seq_out = longest;
    return sci::Status::Ok();
}

// ---- tables -----------------------------------------------------------------------------------------------
namespace tables {

namespace {
// warps = 12: TMA producer, MMA issuer, TMEM owner, one spare, two softmax groups of four.
// stages = slots of the K/V ring (32 KiB each at the 128 geometry, 16 KiB at 64, 32 KiB at 256).
constexpr FlashTile kFlashTiles[] = {
    {32, 128, 128, 12, 8, 64},   {64, 128, 128, 12, 8, 64},   {96, 128, 128, 12, 5, 128},  {128, 128, 128, 12, 5, 128},
    {160, 128, 64, 12, 4, 256},  {192, 128, 64, 12, 4, 256},  {256, 128, 64, 12, 4, 256},
};
}  // namespace

const FlashTile* FindFlashTile(int64_t head_dim) {
    for (const FlashTile& t : kFlashTiles) {
        if (t.head_dim == head_dim) return &t;
    }
    return nullptr;
}

int64_t FlashTileSmemBytes(const FlashTile& tile, int64_t elem_bytes) {
    // two query tiles (one at the 256 geometry) + ring + barriers/alignment, as laid out by the kernel
    const int64_t q_tiles = tile.padded_dim == 256 ? 1 : 2;
    const int64_t q = q_tiles * tile.block_m * tile.padded_dim * elem_bytes;
    const int64_t slot = static_cast<int64_t>(tile.block_n) * tile.padded_dim * elem_bytes;
    return q + tile.stages * slot + 1024 + 256;
}

std::string FlashTileString(const FlashTile& tile) {
    return "bm=" + std::to_string(tile.block_m) + ",bn=" + std::to_string(tile.block_n) + ",warps=" +
           std::to_string(tile.warps) + ",stages=" + std::to_string(tile.stages) + ",geometry=" +
           std::to_string(tile.padded_dim);
}

const DispatchThresholds kDispatch{
    /* decode_max_seq_q     */ 1,
    /* decode_min_seq_kv    */ 256,
    /* tiled_max_seq_kv     */ 128,
    /* min_tokens_per_split */ 256,
    /* max_splits           */ 64,
    /* revision             */ "b200-r1",
};

// The decode kernel runs one wave of resident CTAs (2 per SM). Every (kv head, head chunk) column gets the same
// number of them, and they split the column's list of 64-token steps (sequence after sequence) into equal contiguous
// shares; a sequence cut by share boundaries yields one partial per piece. The split count is therefore the number of
// partial SLOTS per row: the pieces the longest sequence can be cut into, plus one for a share that starts in its
// middle. Fewer slots than that only make the kernel use larger shares (fewer busy CTAs), never a wrong result.
int64_t SlotsForSchedule(int64_t column_steps, int64_t longest_steps, int64_t columns, int64_t sm_count) {
    if (column_steps <= 0 || longest_steps <= 1) return 1;
    const int64_t resident = 2 * (sm_count > 0 ? sm_count : 148);
    const int64_t sharers = detail::Max<int64_t>(1, resident / detail::Max<int64_t>(1, columns));
    const int64_t per_cta = detail::Max<int64_t>(1, detail::CeilDiv<int64_t>(column_steps, sharers));
    const int64_t slots = detail::CeilDiv<int64_t>(longest_steps, per_cta) + 1;
    return detail::Max<int64_t>(2, detail::Min(slots, kDispatch.max_splits));
}

int64_t DecodeSplitsFor(int64_t seq_kv, int64_t batch, int64_t kv_heads, int64_t group, int64_t sm_count) {
    if (seq_kv <= 0) return 1;
    const int64_t steps = detail::CeilDiv<int64_t>(seq_kv, kDecodeStepTokens);
    return SlotsForSchedule(detail::Max<int64_t>(1, batch) * steps, steps, kv_heads * ((group + 15) / 16), sm_count);
}

// Ragged batches: `typical_len` is the mean length; the longest sequence is taken as twice that (exact callers use
// SlotsForSchedule with the true lengths).
int64_t PagedSplitsFor(int64_t typical_len, int64_t num_seqs, int64_t kv_heads, int64_t group, int64_t sm_count) {
    if (typical_len <= 0) return 1;
    const int64_t steps = detail::CeilDiv<int64_t>(typical_len, kDecodeStepTokens);
    return SlotsForSchedule(detail::Max<int64_t>(1, num_seqs) * steps, 2 * steps, kv_heads * ((group + 15) / 16), sm_count);
}

}  // namespace tables
}  // namespace sca
