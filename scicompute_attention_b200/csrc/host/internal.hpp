// Declarations shared by the host translation units (not part of the public API).
#pragma once

#include <cstddef>
#include <string>

#include "sca_b200.h"
#include "scicompute_attention/sca_api.hpp"

namespace sca {
namespace runtime {

const IAttentionBackend* NaiveBackendInstance() noexcept;
const IAttentionBackend* TiledBackendInstance() noexcept;
const IAttentionBackend* FlashBackendInstance() noexcept;
const IAttentionBackend* DecodeBackendInstance() noexcept;
const IAttentionBackend* PagedBackendInstance() noexcept;

// Grow-only fp32 scratch per (device, kind); see scratch.cpp.
enum class ScratchKind : int { kScoresFp32 = 0, kDecodePartials = 1, kGeneric = 2, kCount = 3 };
sci::Result<float*> AcquireScratchFp32(ScratchKind kind, size_t elements, sci::Device& device);
sci::Status ReleaseScratch();
size_t ScratchHighWaterMarkBytes();

// Maps a C-ABI return code (+ sca_last_error()) onto a sci::Status.
sci::Status FromAbi(int rc);
// cudaStream_t (as void*) of `stream`, or of the current stream when null.
void* StreamHandle(sci::Stream* stream);

}  // namespace runtime

// ---- tables that Explain() and the kernels share -------------------------------------------------------
namespace tables {

// Flash prefill geometry on sm_100a by head dim: one CTA = two 128-row query tiles, 128 keys per step.
struct FlashTile {
    int64_t head_dim;
    int32_t block_m, block_n, warps, stages;
    int32_t padded_dim;   // tile geometry the head dim runs on (TMA zero-fills the difference)
};
const FlashTile* FindFlashTile(int64_t head_dim);
int64_t FlashTileSmemBytes(const FlashTile& tile, int64_t elem_bytes);
std::string FlashTileString(const FlashTile& tile);

// Dispatch thresholds; the revision string is part of every Explain() answer.
struct DispatchThresholds {
    int64_t decode_max_seq_q;
    int64_t decode_min_seq_kv;
    int64_t tiled_max_seq_kv;
    int64_t min_tokens_per_split;
    int64_t max_splits;
    const char* revision;
};
extern const DispatchThresholds kDispatch;

// Split-K policy (B200): number of partial slots per row for the decode kernel's equal-share schedule.
constexpr int64_t kDecodeStepTokens = 64;  // tokens one CTA consumes per step (4 warps x 16)
int64_t SlotsForSchedule(int64_t column_steps, int64_t longest_steps, int64_t columns, int64_t sm_count);
int64_t DecodeSplitsFor(int64_t seq_kv, int64_t batch, int64_t kv_heads, int64_t group, int64_t sm_count);
int64_t PagedSplitsFor(int64_t typical_len, int64_t num_seqs, int64_t kv_heads, int64_t group, int64_t sm_count);
inline int64_t PartialElements(int64_t batch, int64_t heads, int64_t splits, int64_t head_dim) {
    return batch * heads * splits * (2 + head_dim);
}

}  // namespace tables
}  // namespace sca

namespace sca {
// NVTX range around one public entry point (domain "sci_attention"): a profiler that is attached sees every API call
// with its name around the kernels it launches; without one the NVTX stubs return at once.
class ApiRange {
public:
    explicit ApiRange(const char* name);
    ~ApiRange();
    ApiRange(const ApiRange&) = delete;
    ApiRange& operator=(const ApiRange&) = delete;
};
}  // namespace sca
