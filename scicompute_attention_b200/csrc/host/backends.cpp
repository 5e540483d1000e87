// The five IAttentionBackend adapters and their public entry points. Each adapter answers
// Supports() with concrete numbers, allocates the result tensors, packs the C-ABI parameter block
// and calls libsca_b200 - nothing here computes attention and nothing falls back to the CPU.
// Capability wording, status codes and stats fields follow the reference adapters
// (src/backends/{naive,tiled,flash,decode,paged}/*_backend.cpp), with the tile / split tables of
// tables:: (api.cpp) in place of the laptop-GPU ones.
#include <string>
#include <vector>

#include "device/cuda_device.hpp"
#include "internal.hpp"

namespace sca {
namespace {

using runtime::FromAbi;
using runtime::StreamHandle;

template <typename T>
sci::Result<AttentionResult> Refuse(AttnStatusCode code, const std::string& text) {
    return sci::MakeUnexpected<AttentionResult>(MakeStatus(code, text));
}
sci::Result<AttentionResult> Refuse(AttnStatusCode code, const std::string& text) {
    return sci::MakeUnexpected<AttentionResult>(MakeStatus(code, text));
}

int DtypeId(sci::DType dtype) {
    switch (dtype) {
        case sci::DType::kFloat32: return SCA_DTYPE_F32;
        case sci::DType::kFloat16: return SCA_DTYPE_F16;
        case sci::DType::kBFloat16: return SCA_DTYPE_BF16;
        default: return -1;
    }
}

const char* kHeadDimSet = "{32,64,96,128,160,192,256}";

// out [B,H_q,S_q,D] (+ lse [B,H_q,S_q] fp32 when asked for) on q's device
sci::Status AllocateOutputs(const sci::Tensor& q, const AttentionShape& s, bool want_lse, AttentionResult* result) {
    sci::Device& device = q.device();
    result->out = sci::Tensor(sci::TensorShape({s.batch, s.num_heads, s.seq_q, s.head_dim}), q.dtype(), device);
    if (result->out.data() == nullptr) {
        return MakeStatus(AttnStatusCode::kWorkspaceExceeded, "allocation of the attention output failed");
    }
    if (want_lse) {
        result->lse = sci::Tensor(sci::TensorShape({s.batch, s.num_heads, s.seq_q}), sci::DType::kFloat32, device);
        if (result->lse.data() == nullptr) {
            return MakeStatus(AttnStatusCode::kWorkspaceExceeded, "allocation of the LSE buffer failed");
        }
    }
    return sci::Status::Ok();
}

ScaFlashFwdParams PackForward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v, AttentionResult* result,
                              const AttentionConfig& cfg, const AttentionShape& s) {
    const detail::Strides qs = detail::StridesFor(cfg.layout, s.seq_q, s.num_heads, s.head_dim);
    const detail::Strides ks = detail::StridesFor(cfg.layout, s.seq_kv, s.num_kv_heads, s.head_dim);
    const detail::Strides os = detail::StridesFor(AttnLayout::kBHSD, s.seq_q, s.num_heads, s.head_dim);
    ScaFlashFwdParams p{};
    p.q = q.data();
    p.k = k.data();
    p.v = v.data();
    p.out = result->out.data();
    p.lse = cfg.return_lse ? static_cast<float*>(result->lse.data()) : nullptr;
    p.batch = s.batch;
    p.num_heads = s.num_heads;
    p.num_kv_heads = s.num_kv_heads;
    p.seq_q = s.seq_q;
    p.seq_kv = s.seq_kv;
    p.head_dim = s.head_dim;
    p.q_sb = qs.s_b; p.q_sh = qs.s_h; p.q_ss = qs.s_s;
    p.k_sb = ks.s_b; p.k_sh = ks.s_h; p.k_ss = ks.s_s;
    p.v_sb = ks.s_b; p.v_sh = ks.s_h; p.v_ss = ks.s_s;
    p.o_sb = os.s_b; p.o_sh = os.s_h; p.o_ss = os.s_s;
    p.scale = EffectiveScale(cfg, s);
    p.causal = cfg.causal ? 1 : 0;
    p.return_lse = cfg.return_lse ? 1 : 0;
    p.diagonal = cfg.causal ? (s.seq_kv - s.seq_q) : 0;
    p.dtype_id = DtypeId(q.dtype());
    return p;
}

sci::Result<AttentionResult> VarlenUnsupported(const char* who) {
    return Refuse(AttnStatusCode::kUnsupportedFeature,
                  std::string(who) + " backend does not implement the varlen entry point; use flash_attention_varlen");
}

size_t ScoreBytes(const AttentionShape& s) {
    return static_cast<size_t>(s.batch) * static_cast<size_t>(s.num_heads) * static_cast<size_t>(s.seq_q) *
           static_cast<size_t>(s.seq_kv) * sizeof(float);
}

// =================================================================================================
// naive: reference-level backend. As in the reference the fp32 score matrix is materialised in pooled scratch
// (three plain kernels: scores, row softmax, P.V), reported in the stats, and bounded by the workspace limit.
// =================================================================================================
size_t NaiveWorkspaceLimit(const AttentionConfig& cfg) {
    if (cfg.workspace_limit_bytes != 0) return cfg.workspace_limit_bytes;
    return DeviceCapability::ForDevice(0).free_mem_bytes / 2;
}

class NaiveBackend final : public IAttentionBackend {
public:
    BackendKind Kind() const noexcept override { return BackendKind::kNaive; }
    const char* Name() const noexcept override { return "naive"; }

    CapabilityReport Supports(const AttentionConfig& cfg, const AttentionShape& shape) const override {
        CapabilityReport r;
        r.recommended_backend = BackendKind::kNaive;
        r.workspace_bytes = ScoreBytes(shape);
        std::string no;
        if (!DeviceCapability::CudaAvailable()) {
            no = "no CUDA device available (DeviceCapability reports cuda-unavailable)";
        } else if (SupportedHeadDimIndex(shape.head_dim) < 0) {
            no = "head_dim=" + std::to_string(shape.head_dim) + " is outside " + kHeadDimSet;
        } else if (cfg.sliding_window > 0) {
            no = "sliding_window=" + std::to_string(cfg.sliding_window) + " is not implemented by the naive backend";
        } else {
            const size_t limit = NaiveWorkspaceLimit(cfg);
            if (limit != 0 && r.workspace_bytes > limit) {
                no = "score matrix needs " + std::to_string(r.workspace_bytes) + " B > workspace limit " +
                     std::to_string(limit) + " B; use the tiled or flash backend";
            }
        }
        r.supported = no.empty();
        r.reason = r.supported ? "B*H_q*S_q*S_kv*4 = " + std::to_string(r.workspace_bytes) +
                                     " B of FP32 score storage fits the workspace limit"
                               : no;
        return r;
    }
    size_t WorkspaceBytes(const AttentionConfig&, const AttentionShape& shape) const override { return ScoreBytes(shape); }

    sci::Result<AttentionResult> Forward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                         const AttentionConfig& cfg) const override {
        const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(cfg.stream));
        const ApiRange nvtx_range("NaiveBackend::Forward");
        const sci::Result<AttentionShape> inferred = InferShape(q, k, v, cfg.layout);
        if (!inferred.ok()) return sci::MakeUnexpected<AttentionResult>(inferred.error());
        const AttentionShape shape = *inferred;
        const sci::Status valid = Validate(cfg, shape);
        if (!valid.ok()) return sci::MakeUnexpected<AttentionResult>(valid);
        const size_t need = ScoreBytes(shape), limit = NaiveWorkspaceLimit(cfg);
        if (limit != 0 && need > limit) {
            return Refuse(AttnStatusCode::kWorkspaceExceeded,
                          "naive score matrix requires " + std::to_string(need) + " B but the workspace limit is " +
                              std::to_string(limit) + " B; switch to tiled/flash or raise workspace_limit_bytes");
        }
        if (DtypeId(q.dtype()) < 0) {
            return Refuse(AttnStatusCode::kUnsupportedDtype,
                          std::string("dtype=") + sci::kDTypeName(q.dtype()) + " is not a compute dtype");
        }
        AttentionResult result;
        if (sci::Status s = AllocateOutputs(q, shape, cfg.return_lse, &result); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        const sci::Result<float*> scores =
            runtime::AcquireScratchFp32(runtime::ScratchKind::kScoresFp32, need / sizeof(float), q.device());
        if (!scores.ok()) return sci::MakeUnexpected<AttentionResult>(scores.error());
        const ScaFlashFwdParams p = PackForward(q, k, v, &result, cfg, shape);
        if (sci::Status s = FromAbi(sca_launch_naive_forward(&p, *scores, StreamHandle(cfg.stream))); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        result.stats.used_backend = BackendKind::kNaive;
        result.stats.workspace_bytes = need;
        result.stats.materialized_score_bytes = static_cast<int64_t>(need);
        result.stats.note = std::string("reference path: FP32 score matrix materialized in HBM (") + std::to_string(need) +
                            " B); layout=" + LayoutName(cfg.layout);
        if (cfg.causal) result.stats.note += ", causal(alignment=bottom-right)";
        return sci::Ok(std::move(result));
    }
    sci::Result<AttentionResult> ForwardVarlen(const sci::Tensor&, const sci::Tensor&, const sci::Tensor&, int64_t,
                                               const int32_t*, const int32_t*, int64_t, int64_t,
                                               const AttentionConfig&) const override {
        return VarlenUnsupported("naive");
    }
};

// =================================================================================================
// tiled: short-sequence backend of the dispatcher table (seq_kv <= 128). Same SIMT kernel; keeps the
// reference's head_dim <= 128 contract and answers with the warp-per-row geometry it really uses.
// =================================================================================================
constexpr int64_t kTiledMaxHeadDim = 128;

TileConfig TiledGeometry() {
    TileConfig t;
    t.block_m = 4;   // query rows per CTA (one warp each)
    t.block_n = 1;   // keys per step of a warp
    t.warps = 4;
    t.stages = 1;
    return t;
}

class TiledBackend final : public IAttentionBackend {
public:
    BackendKind Kind() const noexcept override { return BackendKind::kTiled; }
    const char* Name() const noexcept override { return "tiled"; }

    CapabilityReport Supports(const AttentionConfig& cfg, const AttentionShape& shape) const override {
        CapabilityReport r;
        r.recommended_backend = BackendKind::kTiled;
        std::string no;
        if (!DeviceCapability::CudaAvailable()) {
            no = "no CUDA device available";
        } else if (SupportedHeadDimIndex(shape.head_dim) < 0) {
            no = "head_dim=" + std::to_string(shape.head_dim) + " is outside " + kHeadDimSet;
        } else if (shape.head_dim > kTiledMaxHeadDim) {
            no = "head_dim=" + std::to_string(shape.head_dim) + " > " + std::to_string(kTiledMaxHeadDim) +
                 " is served by the flash backend (smem budget for tiled)";
        } else if (cfg.sliding_window > 0) {
            no = "sliding_window is not implemented by the tiled backend";
        } else {
            r.tile = TiledGeometry();
        }
        r.supported = no.empty();
        r.reason = r.supported ? "tiled tile=" + r.tile.ToString() + " keeps S in registers (workspace 0 B)" : no;
        return r;
    }
    size_t WorkspaceBytes(const AttentionConfig&, const AttentionShape&) const override { return 0; }

    sci::Result<AttentionResult> Forward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                         const AttentionConfig& cfg) const override {
        const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(cfg.stream));
        const ApiRange nvtx_range("TiledBackend::Forward");
        const sci::Result<AttentionShape> inferred = InferShape(q, k, v, cfg.layout);
        if (!inferred.ok()) return sci::MakeUnexpected<AttentionResult>(inferred.error());
        const AttentionShape shape = *inferred;
        const sci::Status valid = Validate(cfg, shape);
        if (!valid.ok()) return sci::MakeUnexpected<AttentionResult>(valid);
        if (shape.head_dim > kTiledMaxHeadDim) {
            return Refuse(AttnStatusCode::kDeviceCapability,
                          "tiled supports head_dim <= " + std::to_string(kTiledMaxHeadDim) + "; head_dim=" +
                              std::to_string(shape.head_dim) + " needs the flash backend");
        }
        if (DtypeId(q.dtype()) < 0) {
            return Refuse(AttnStatusCode::kUnsupportedDtype,
                          std::string("dtype=") + sci::kDTypeName(q.dtype()) + " is not a compute dtype");
        }
        AttentionResult result;
        if (sci::Status s = AllocateOutputs(q, shape, cfg.return_lse, &result); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        const ScaFlashFwdParams p = PackForward(q, k, v, &result, cfg, shape);
        if (sci::Status s = FromAbi(sca_launch_simt_forward(&p, StreamHandle(cfg.stream))); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        result.stats.used_backend = BackendKind::kTiled;
        result.stats.tile = TiledGeometry();
        result.stats.workspace_bytes = 0;
        result.stats.materialized_score_bytes = 0;
        result.stats.note = std::string("online softmax, one warp per query row; workspace 0 B; layout=") + LayoutName(cfg.layout);
        return sci::Ok(std::move(result));
    }
    sci::Result<AttentionResult> ForwardVarlen(const sci::Tensor&, const sci::Tensor&, const sci::Tensor&, int64_t,
                                               const int32_t*, const int32_t*, int64_t, int64_t,
                                               const AttentionConfig&) const override {
        return VarlenUnsupported("tiled");
    }
};

// =================================================================================================
// flash: tcgen05 prefill
// =================================================================================================
TileConfig ToTileConfig(const tables::FlashTile& t) {
    TileConfig c;
    c.block_m = t.block_m;
    c.block_n = t.block_n;
    c.warps = t.warps;
    c.stages = t.stages;
    c.use_tma = true;
    return c;
}

sci::Status CheckFlashRequest(sci::DType dtype, const AttentionConfig& cfg, const AttentionShape& shape,
                              const tables::FlashTile** tile_out) {
    if (!DeviceCapability::CudaAvailable()) {
        return MakeStatus(AttnStatusCode::kUnsupportedFeature, "flash backend: no CUDA device available");
    }
    if (dtype != sci::DType::kFloat16 && dtype != sci::DType::kBFloat16) {
        return MakeStatus(AttnStatusCode::kUnsupportedDtype,
                          std::string("flash backend computes in fp16/bf16; dtype=") + sci::kDTypeName(dtype) +
                              " is served by the naive (reference) or tiled backend");
    }
    const tables::FlashTile* tile = tables::FindFlashTile(shape.head_dim);
    if (tile == nullptr) {
        return MakeStatus(AttnStatusCode::kUnsupportedHeadDim,
                          "flash tile table has no entry for head_dim=" + std::to_string(shape.head_dim));
    }
    const DeviceCapability& cap = DeviceCapability::ForDevice(0);
    const size_t limit = DeviceCapability::SmemLimitPerBlock(cap);
    const int64_t smem = tables::FlashTileSmemBytes(*tile, DtypeSize(dtype));
    if (smem < 0 || static_cast<size_t>(smem) > limit) {
        return MakeStatus(AttnStatusCode::kDeviceCapability,
                          "flash tile " + tables::FlashTileString(*tile) + " needs " + std::to_string(smem) +
                              " B > smem limit " + std::to_string(limit) + " B for head_dim=" + std::to_string(shape.head_dim));
    }
    if (cfg.sliding_window > 0) {
        return MakeStatus(AttnStatusCode::kUnsupportedFeature, "flash backend: sliding_window=" +
                                                                   std::to_string(cfg.sliding_window) + " is not implemented in v1");
    }
    if (tile_out != nullptr) *tile_out = tile;
    return sci::Status::Ok();
}

class FlashBackend final : public IAttentionBackend {
public:
    BackendKind Kind() const noexcept override { return BackendKind::kFlash; }
    const char* Name() const noexcept override { return "flash"; }

    CapabilityReport Supports(const AttentionConfig& cfg, const AttentionShape& shape) const override {
        CapabilityReport r;
        r.recommended_backend = BackendKind::kFlash;
        const tables::FlashTile* tile = tables::FindFlashTile(shape.head_dim);
        std::string no;
        if (!DeviceCapability::CudaAvailable()) {
            no = "no CUDA device available";
        } else if (tile == nullptr) {
            no = "head_dim=" + std::to_string(shape.head_dim) + " has no flash tile (supported: 32,64,96,128,160,192,256)";
        } else if (cfg.sliding_window > 0) {
            no = "sliding_window=" + std::to_string(cfg.sliding_window) + " not implemented";
        } else {
            const size_t limit = DeviceCapability::SmemLimitPerBlock(DeviceCapability::ForDevice(0));
            const int64_t smem = tables::FlashTileSmemBytes(*tile, 2);
            if (static_cast<size_t>(smem) > limit) {
                no = "tile " + tables::FlashTileString(*tile) + " needs " + std::to_string(smem) + " B > smem limit " +
                     std::to_string(limit) + " B";
            } else {
                r.tile = ToTileConfig(*tile);
            }
        }
        r.supported = no.empty();
        r.reason = r.supported ? "online softmax in registers (workspace 0 B), tile " + tables::FlashTileString(*tile) : no;
        return r;
    }
    size_t WorkspaceBytes(const AttentionConfig&, const AttentionShape&) const override { return 0; }

    sci::Result<AttentionResult> Forward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                         const AttentionConfig& cfg) const override {
        const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(cfg.stream));
        const ApiRange nvtx_range("FlashBackend::Forward");
        const sci::Result<AttentionShape> inferred = InferShape(q, k, v, cfg.layout);
        if (!inferred.ok()) return sci::MakeUnexpected<AttentionResult>(inferred.error());
        const AttentionShape shape = *inferred;
        const sci::Status valid = Validate(cfg, shape);
        if (!valid.ok()) return sci::MakeUnexpected<AttentionResult>(valid);
        const tables::FlashTile* tile = nullptr;
        if (sci::Status s = CheckFlashRequest(q.dtype(), cfg, shape, &tile); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        AttentionResult result;
        if (sci::Status s = AllocateOutputs(q, shape, cfg.return_lse, &result); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        const ScaFlashFwdParams p = PackForward(q, k, v, &result, cfg, shape);
        if (sci::Status s = FromAbi(sca_launch_flash_fwd(&p, StreamHandle(cfg.stream))); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        result.stats.used_backend = BackendKind::kFlash;
        result.stats.tile = ToTileConfig(*tile);
        result.stats.workspace_bytes = 0;
        result.stats.materialized_score_bytes = 0;
        result.stats.note = "flash: tcgen05.mma with S/P/O in tensor memory + TMA ring, tile " +
                            tables::FlashTileString(*tile) + "; layout=" + LayoutName(cfg.layout);
        return sci::Ok(std::move(result));
    }

    // Packed [T, H, D] tensors with host offsets: one launch per sequence over the packed buffers
    // (a packed tensor is a BSHD tensor with B = 1).
    sci::Result<AttentionResult> ForwardVarlen(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                               int64_t num_seqs, const int32_t* cu_q, const int32_t* cu_kv,
                                               int64_t max_seq_q, int64_t max_seq_kv,
                                               const AttentionConfig& cfg) const override {
        const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(cfg.stream));
        const ApiRange nvtx_range("FlashBackend::ForwardVarlen");
        if (cu_q == nullptr || cu_kv == nullptr) {
            return Refuse(AttnStatusCode::kShapeMismatch, "varlen requires host-resident cu_seqlens_q/kv");
        }
        if (num_seqs < 1) {
            return Refuse(AttnStatusCode::kShapeMismatch, "varlen num_seqs=" + std::to_string(num_seqs) + " (must be >= 1)");
        }
        if (cfg.return_lse) {
            return Refuse(AttnStatusCode::kUnsupportedFeature,
                          "varlen does not expose LSE yet; call the per-sequence entry point if it is needed");
        }
        if (cfg.causal && max_seq_kv < max_seq_q) {
            return Refuse(AttnStatusCode::kShapeMismatch, "varlen causal requires max_seq_kv >= max_seq_q");
        }
        for (const sci::Tensor* t : {&q, &k, &v}) {
            if (t->ndims() != 3) {
                return Refuse(AttnStatusCode::kShapeMismatch,
                              "varlen expects packed [T, H, D] tensors; got ndims=" + std::to_string(t->ndims()));
            }
            if (t->device_type() != sci::DeviceType::kCUDA) {
                return Refuse(AttnStatusCode::kUnsupportedFeature, "varlen requires CUDA tensors");
            }
        }
        if (q.dtype() != sci::DType::kFloat16 && q.dtype() != sci::DType::kBFloat16) {
            return Refuse(AttnStatusCode::kUnsupportedDtype, "flash varlen supports fp16/bf16 only");
        }
        if (q.dtype() != k.dtype() || q.dtype() != v.dtype()) {
            return Refuse(AttnStatusCode::kUnsupportedDtype, "varlen requires q/k/v to share one dtype");
        }
        const int64_t heads = q.dim(1), d = q.dim(2), kv_heads = k.dim(1);
        if (k.dim(2) != d || v.dim(2) != d || v.dim(1) != kv_heads) {
            return Refuse(AttnStatusCode::kShapeMismatch, "varlen expects k/v head dims to match q; got D=" + std::to_string(d));
        }
        if (kv_heads < 1 || heads % kv_heads != 0) {
            return Refuse(AttnStatusCode::kShapeMismatch, "varlen requires H_q % H_kv == 0");
        }
        AttentionShape probe;
        probe.batch = 1;
        probe.seq_q = max_seq_q;
        probe.seq_kv = max_seq_kv;
        probe.num_heads = heads;
        probe.num_kv_heads = kv_heads;
        probe.head_dim = d;
        const tables::FlashTile* tile = nullptr;
        if (sci::Status s = CheckFlashRequest(q.dtype(), cfg, probe, &tile); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        AttentionResult result;
        result.out = sci::Tensor(sci::TensorShape({q.dim(0), heads, d}), q.dtype(), q.device());
        if (result.out.data() == nullptr) {
            return Refuse(AttnStatusCode::kWorkspaceExceeded, "allocation of the varlen output failed");
        }
        // the same per-sequence checks, with the same messages, as the reference's launch loop
        for (int64_t s = 0; s < num_seqs; ++s) {
            const int64_t sq = cu_q[s + 1] - cu_q[s], skv = cu_kv[s + 1] - cu_kv[s];
            if (sq <= 0 || skv <= 0) {
                return Refuse(AttnStatusCode::kShapeMismatch, "varlen sequence " + std::to_string(s) + " has S_q=" +
                                                                  std::to_string(sq) + ", S_kv=" + std::to_string(skv) +
                                                                  " (both must be > 0)");
            }
            if (cfg.causal && skv < sq) {
                return Refuse(AttnStatusCode::kShapeMismatch, "varlen sequence " + std::to_string(s) +
                                                                  " is causal with S_kv=" + std::to_string(skv) +
                                                                  " < S_q=" + std::to_string(sq));
            }
        }
        // one launch for the whole batch: the kernel's work list spans all sequences
        const int64_t ws_bytes = sca_flash_varlen_workspace_bytes(num_seqs, q.dim(0));
        sci::Tensor workspace(sci::TensorShape({ws_bytes}), sci::DType::kUInt8, q.device());
        if (workspace.data() == nullptr) {
            return Refuse(AttnStatusCode::kWorkspaceExceeded, "allocation of the varlen work list failed");
        }
        ScaFlashVarlenParams p{};
        p.q = q.data();
        p.k = k.data();
        p.v = v.data();
        p.out = result.out.data();
        p.total_q = q.dim(0);
        p.total_kv = k.dim(0);
        p.num_heads = heads;
        p.num_kv_heads = kv_heads;
        p.head_dim = d;
        p.num_seqs = num_seqs;
        p.cu_seqlens_q = cu_q;
        p.cu_seqlens_kv = cu_kv;
        p.scale = EffectiveScale(cfg, probe);
        p.causal = cfg.causal ? 1 : 0;
        p.dtype_id = DtypeId(q.dtype());
        p.workspace = workspace.data();
        p.workspace_bytes = ws_bytes;
        if (sci::Status st = FromAbi(sca_launch_flash_varlen(&p, StreamHandle(cfg.stream))); !st.ok()) {
            return sci::MakeUnexpected<AttentionResult>(st);
        }
        result.stats.used_backend = BackendKind::kFlash;
        result.stats.tile = ToTileConfig(*tile);
        result.stats.workspace_bytes = static_cast<size_t>(ws_bytes);
        result.stats.note = "varlen: " + std::to_string(num_seqs) + " sequences in one launch over packed buffers (tile " +
                            tables::FlashTileString(*tile) + ")";
        return sci::Ok(std::move(result));
    }
};

// =================================================================================================
// decode: split-K, seq_q == 1
// =================================================================================================
constexpr int64_t kDecodeSeqQ = 1;

int64_t ResolveSplits(const AttentionConfig& cfg, const AttentionShape& shape, const DeviceCapability& cap) {
    if (cfg.num_splits > 0) return detail::Min<int64_t>(cfg.num_splits, tables::kDispatch.max_splits);
    return tables::DecodeSplitsFor(shape.seq_kv, shape.batch, shape.num_kv_heads, shape.GroupSize(), cap.sm_count);
}

class DecodeBackend final : public IAttentionBackend {
public:
    BackendKind Kind() const noexcept override { return BackendKind::kDecode; }
    const char* Name() const noexcept override { return "decode"; }

    CapabilityReport Supports(const AttentionConfig& cfg, const AttentionShape& shape) const override {
        CapabilityReport r;
        r.recommended_backend = BackendKind::kDecode;
        const int64_t splits = ResolveSplits(cfg, shape, DeviceCapability::ForDevice(0));
        r.workspace_bytes = static_cast<size_t>(tables::PartialElements(shape.batch, shape.num_heads, splits, shape.head_dim)) * sizeof(float);
        std::string no;
        if (!DeviceCapability::CudaAvailable()) {
            no = "no CUDA device available";
        } else if (shape.seq_q != kDecodeSeqQ) {
            no = "decode kernel handles seq_q=" + std::to_string(kDecodeSeqQ) + "; seq_q=" + std::to_string(shape.seq_q) +
                 " is routed to the flash backend (grouped decode is a Roadmap item)";
        } else if (SupportedHeadDimIndex(shape.head_dim) < 0) {
            no = "head_dim=" + std::to_string(shape.head_dim) + " is unsupported";
        } else if (shape.head_dim % 32 != 0) {
            no = "decode requires head_dim % 32 == 0; head_dim=" + std::to_string(shape.head_dim);
        } else if (cfg.sliding_window > 0) {
            no = "sliding_window is not implemented by the decode backend";
        }
        r.supported = no.empty();
        r.reason = r.supported ? "split-K decode with " + std::to_string(splits) + " splits, workspace " +
                                     std::to_string(r.workspace_bytes) + " B (FP32 partials)"
                               : no;
        return r;
    }
    size_t WorkspaceBytes(const AttentionConfig& cfg, const AttentionShape& shape) const override {
        const int64_t splits = ResolveSplits(cfg, shape, DeviceCapability::ForDevice(0));
        return static_cast<size_t>(tables::PartialElements(shape.batch, shape.num_heads, splits, shape.head_dim)) * sizeof(float);
    }

    sci::Result<AttentionResult> Forward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                         const AttentionConfig& cfg) const override {
        const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(cfg.stream));
        const ApiRange nvtx_range("DecodeBackend::Forward");
        const sci::Result<AttentionShape> inferred = InferShape(q, k, v, cfg.layout);
        if (!inferred.ok()) return sci::MakeUnexpected<AttentionResult>(inferred.error());
        const AttentionShape shape = *inferred;
        const sci::Status valid = Validate(cfg, shape);
        if (!valid.ok()) return sci::MakeUnexpected<AttentionResult>(valid);
        if (shape.seq_q != kDecodeSeqQ) {
            return Refuse(AttnStatusCode::kUnsupportedFeature,
                          "decode backend requires seq_q=" + std::to_string(kDecodeSeqQ) + "; seq_q=" +
                              std::to_string(shape.seq_q) + " belongs to the flash backend");
        }
        if (shape.head_dim % 32 != 0) {
            return Refuse(AttnStatusCode::kUnsupportedHeadDim,
                          "decode requires head_dim % 32 == 0; head_dim=" + std::to_string(shape.head_dim));
        }
        if (DtypeId(q.dtype()) < 0) {
            return Refuse(AttnStatusCode::kUnsupportedDtype,
                          std::string("dtype=") + sci::kDTypeName(q.dtype()) + " is not a compute dtype");
        }
        const int64_t splits = ResolveSplits(cfg, shape, DeviceCapability::ForDevice(0));
        const int64_t elements = tables::PartialElements(shape.batch, shape.num_heads, splits, shape.head_dim);
        const sci::Result<float*> scratch =
            runtime::AcquireScratchFp32(runtime::ScratchKind::kDecodePartials, static_cast<size_t>(elements), q.device());
        if (!scratch.ok()) return sci::MakeUnexpected<AttentionResult>(scratch.error());

        AttentionResult result;
        if (sci::Status s = AllocateOutputs(q, shape, false, &result); !s.ok()) {
            return Refuse(AttnStatusCode::kWorkspaceExceeded, "allocation of the decode output failed");
        }
        const int64_t base = shape.batch * shape.num_heads * splits;
        const detail::Strides qs = detail::StridesFor(cfg.layout, shape.seq_q, shape.num_heads, shape.head_dim);
        const detail::Strides ks = detail::StridesFor(cfg.layout, shape.seq_kv, shape.num_kv_heads, shape.head_dim);
        const detail::Strides os = detail::StridesFor(AttnLayout::kBHSD, shape.seq_q, shape.num_heads, shape.head_dim);
        ScaDecodeFwdParams p{};
        p.q = q.data();
        p.k = k.data();
        p.v = v.data();
        p.out = result.out.data();
        p.partial_m = *scratch;
        p.partial_l = *scratch + base;
        p.partial_o = *scratch + 2 * base;
        p.batch = shape.batch;
        p.num_heads = shape.num_heads;
        p.num_kv_heads = shape.num_kv_heads;
        p.seq_kv = shape.seq_kv;
        p.head_dim = shape.head_dim;
        p.num_splits = splits;
        p.q_stride = {qs.s_b, qs.s_h, qs.s_s};
        p.k_stride = {ks.s_b, ks.s_h, ks.s_s};
        p.v_stride = p.k_stride;
        p.o_stride = {os.s_b, os.s_h, os.s_s};
        p.scale = EffectiveScale(cfg, shape);
        p.dtype = DtypeId(q.dtype());
        if (sci::Status s = FromAbi(sca_launch_decode_splitk(&p, StreamHandle(cfg.stream))); !s.ok()) {
            return sci::MakeUnexpected<AttentionResult>(s);
        }
        result.stats.used_backend = BackendKind::kDecode;
        result.stats.workspace_bytes = static_cast<size_t>(elements) * sizeof(float);
        result.stats.num_splits = splits;
        result.stats.note = "split-K decode: " + std::to_string(splits) + " splits, FP32 partials in workspace; layout=" +
                            std::string(LayoutName(cfg.layout));
        return sci::Ok(std::move(result));
    }
    sci::Result<AttentionResult> ForwardVarlen(const sci::Tensor&, const sci::Tensor&, const sci::Tensor&, int64_t,
                                               const int32_t*, const int32_t*, int64_t, int64_t,
                                               const AttentionConfig&) const override {
        return Refuse(AttnStatusCode::kUnsupportedFeature, "decode backend does not implement varlen; use flash_attention_varlen");
    }
};

// =================================================================================================
// paged: decode over page-table-indirected K/V
// =================================================================================================
sci::Result<AttentionResult> RunPaged(const sci::Tensor& q, const PagedKVCache& kv, const PagedAttentionParams& params,
                                      const AttentionConfig& cfg) {
    const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(cfg.stream));
    const ApiRange nvtx_range("RunPaged");
    if (q.ndims() != 4) {
        return Refuse(AttnStatusCode::kShapeMismatch,
                      "paged_attention expects q=[num_seqs, H_q, seq_q, D]; got ndims=" + std::to_string(q.ndims()));
    }
    const int64_t num_seqs = q.dim(0), heads = q.dim(1), seq_q = q.dim(2), d = q.dim(3);
    const KVCacheConfig& kcfg = kv.Storage().Config();
    if (seq_q != kDecodeSeqQ) {
        return Refuse(AttnStatusCode::kUnsupportedFeature,
                      "paged attention implements the decode form only (seq_q=1); got seq_q=" + std::to_string(seq_q));
    }
    if (num_seqs <= 0 || num_seqs > kv.MaxNumSeqs()) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_attention num_seqs=" + std::to_string(num_seqs) +
                                                          " exceeds the cache's max_num_seqs=" + std::to_string(kv.MaxNumSeqs()));
    }
    if (params.layer < 0 || params.layer >= kcfg.num_layers) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_attention layer=" + std::to_string(params.layer) +
                                                          " out of range [0," + std::to_string(kcfg.num_layers) + ")");
    }
    if (DtypeId(q.dtype()) < 0) {
        return Refuse(AttnStatusCode::kUnsupportedDtype, std::string("dtype=") + sci::kDTypeName(q.dtype()) + " is not a compute dtype");
    }
    if (d % 32 != 0 || SupportedHeadDimIndex(d) < 0) {
        return Refuse(AttnStatusCode::kUnsupportedHeadDim,
                      "paged attention requires head_dim % 32 == 0 within {32..256}; got " + std::to_string(d));
    }
    if (kcfg.num_kv_heads < 1 || heads % kcfg.num_kv_heads != 0) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_attention num_heads=" + std::to_string(heads) +
                                                          " is not a multiple of the cache's num_kv_heads=" +
                                                          std::to_string(kcfg.num_kv_heads));
    }
    const int32_t* table = params.page_table != nullptr ? params.page_table : kv.PageTableDevicePtr();
    if (table == nullptr) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_attention has no page table (call PagedKVCache::SyncPageTable first)");
    }
    const int64_t block_size = params.block_size > 0 ? params.block_size : kv.BlockSize();
    const int64_t max_blocks = params.max_blocks_per_seq > 0 ? params.max_blocks_per_seq : kv.MaxBlocksPerSeq();
    const int64_t upper = kcfg.num_blocks * block_size;  // bound of any sequence; true lengths come from seq_lens

    // slot count: the cache object knows every sequence's length on the host, which is what the kernel's schedule
    // depends on (steps in total, steps of the longest sequence); without device lengths every sequence is scanned
    // over the whole table row. An explicit request wins.
    int64_t splits;
    if (cfg.num_splits > 0) {
        splits = detail::Min<int64_t>(cfg.num_splits, tables::kDispatch.max_splits);
    } else {
        const int64_t columns = kcfg.num_kv_heads * ((heads / kcfg.num_kv_heads + 15) / 16);
        const int64_t row_tokens = detail::Min<int64_t>(upper, max_blocks * block_size);
        int64_t total_steps = 0, longest_steps = 0;
        for (int64_t s = 0; s < num_seqs; ++s) {
            const int64_t n = params.seq_lens != nullptr ? kv.SeqLength(s) : row_tokens;
            const int64_t steps = detail::Max<int64_t>(1, detail::CeilDiv<int64_t>(n, tables::kDecodeStepTokens));
            total_steps += steps;
            longest_steps = detail::Max(longest_steps, steps);
        }
        splits = tables::SlotsForSchedule(total_steps, longest_steps, columns, DeviceCapability::ForDevice(0).sm_count);
    }
    const int64_t elements = tables::PartialElements(num_seqs, heads, splits, d);
    const sci::Result<float*> scratch =
        runtime::AcquireScratchFp32(runtime::ScratchKind::kDecodePartials, static_cast<size_t>(elements), q.device());
    if (!scratch.ok()) return sci::MakeUnexpected<AttentionResult>(scratch.error());

    AttentionResult result;
    result.out = sci::Tensor(sci::TensorShape({num_seqs, heads, seq_q, d}), q.dtype(), q.device());
    if (result.out.data() == nullptr) {
        return Refuse(AttnStatusCode::kWorkspaceExceeded, "allocation of the paged output failed");
    }
    const int64_t base = num_seqs * heads * splits;
    AttentionShape shape;
    shape.batch = num_seqs;
    shape.seq_q = seq_q;
    shape.seq_kv = upper;
    shape.num_heads = heads;
    shape.num_kv_heads = kcfg.num_kv_heads;
    shape.head_dim = d;

    ScaPagedDecodeParams pp{};
    ScaDecodeFwdParams& p = pp.base;
    p.q = q.data();
    p.k = kv.Storage().K(params.layer).data();
    p.v = kv.Storage().V(params.layer).data();
    p.out = result.out.data();
    p.partial_m = *scratch;
    p.partial_l = *scratch + base;
    p.partial_o = *scratch + 2 * base;
    p.batch = num_seqs;
    p.num_heads = heads;
    p.num_kv_heads = kcfg.num_kv_heads;
    p.seq_kv = upper;
    p.head_dim = d;
    p.num_splits = splits;
    p.q_stride = {heads * seq_q * d, seq_q * d, d};
    p.o_stride = p.q_stride;
    p.k_stride = {0, d, kcfg.num_kv_heads * d};  // one pool row = one token: [kv_heads][D]
    p.v_stride = p.k_stride;
    p.scale = EffectiveScale(cfg, shape);
    p.dtype = DtypeId(q.dtype());
    p.seq_lens = params.seq_lens;
    pp.page_table = table;
    pp.block_size = block_size;
    pp.max_blocks_per_seq = max_blocks;
    pp.num_kv_blocks = kcfg.num_blocks;
    // scheduling hint only: any permutation gives the same result
    const int32_t* order = kv.SeqOrderDevicePtr(num_seqs);
    if (sci::Status s = FromAbi(sca_launch_paged_attention_ordered(&pp, order, StreamHandle(cfg.stream))); !s.ok()) {
        return sci::MakeUnexpected<AttentionResult>(s);
    }
    result.stats.used_backend = BackendKind::kPaged;
    result.stats.workspace_bytes = static_cast<size_t>(elements) * sizeof(float);
    result.stats.num_splits = splits;
    result.stats.kv_bytes = kv.Storage().MemoryBytes();
    result.stats.note = "paged decode: " + std::to_string(splits) + " splits, block_size=" + std::to_string(block_size) +
                        ", layer=" + std::to_string(params.layer);
    return sci::Ok(std::move(result));
}

class PagedBackend final : public IAttentionBackend {
public:
    BackendKind Kind() const noexcept override { return BackendKind::kPaged; }
    const char* Name() const noexcept override { return "paged"; }
    CapabilityReport Supports(const AttentionConfig&, const AttentionShape& shape) const override {
        CapabilityReport r;
        r.recommended_backend = BackendKind::kDecode;
        std::string no;
        if (!DeviceCapability::CudaAvailable()) no = "no CUDA device available";
        else if (shape.seq_q != kDecodeSeqQ) no = "paged attention implements the decode form only (seq_q=1)";
        else if (shape.head_dim % 32 != 0) no = "paged attention requires head_dim % 32 == 0";
        r.supported = no.empty();
        r.reason = r.supported ? "paged decode over non-contiguous pages (page-table addressing)" : no;
        return r;
    }
    size_t WorkspaceBytes(const AttentionConfig& cfg, const AttentionShape& shape) const override {
        const int64_t splits = cfg.num_splits > 0 ? cfg.num_splits
                                                  : tables::PagedSplitsFor(shape.seq_kv, shape.batch, shape.num_kv_heads,
                                                                           shape.GroupSize(), DeviceCapability::ForDevice(0).sm_count);
        return static_cast<size_t>(tables::PartialElements(shape.batch, shape.num_heads, splits, shape.head_dim)) * sizeof(float);
    }
    sci::Result<AttentionResult> Forward(const sci::Tensor&, const sci::Tensor&, const sci::Tensor&,
                                         const AttentionConfig&) const override {
        return Refuse(AttnStatusCode::kUnsupportedFeature,
                      "paged attention needs the KV cache: call sca::paged_attention(q, kv, params, cfg)");
    }
    sci::Result<AttentionResult> ForwardVarlen(const sci::Tensor&, const sci::Tensor&, const sci::Tensor&, int64_t,
                                               const int32_t*, const int32_t*, int64_t, int64_t,
                                               const AttentionConfig&) const override {
        return Refuse(AttnStatusCode::kUnsupportedFeature, "paged backend does not implement varlen; use flash_attention_varlen");
    }
};

const NaiveBackend kNaive;
const TiledBackend kTiled;
const FlashBackend kFlash;
const DecodeBackend kDecode;
const PagedBackend kPaged;

}  // namespace

namespace runtime {
const IAttentionBackend* NaiveBackendInstance() noexcept { return &kNaive; }
const IAttentionBackend* TiledBackendInstance() noexcept { return &kTiled; }
const IAttentionBackend* FlashBackendInstance() noexcept { return &kFlash; }
const IAttentionBackend* DecodeBackendInstance() noexcept { return &kDecode; }
const IAttentionBackend* PagedBackendInstance() noexcept { return &kPaged; }
}  // namespace runtime

sci::Result<AttentionResult> naive_attention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                             const AttentionConfig& cfg) {
    return kNaive.Forward(q, k, v, cfg);
}
sci::Result<AttentionResult> tiled_attention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                             const AttentionConfig& cfg) {
    return kTiled.Forward(q, k, v, cfg);
}
sci::Result<AttentionResult> flash_attention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                             const AttentionConfig& cfg) {
    return kFlash.Forward(q, k, v, cfg);
}
sci::Status FlashLaunchStatus(int device_id) {
    int32_t code = 0;
    if (sci::Status s = FromAbi(sca_flash_status(device_id, &code)); !s.ok()) return s;
    if (code == 0) return sci::Status::Ok();
    return sci::Status(sci::StatusCode::kCudaError, "flash attention: an earlier launch gave up waiting on a barrier (role " +
                                                         std::to_string(code) + "); its output is invalid");
}
sci::Result<AttentionResult> flash_attention_varlen(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                                    int64_t num_seqs, const int32_t* cu_q, const int32_t* cu_kv,
                                                    int64_t max_seq_q, int64_t max_seq_kv, const AttentionConfig& cfg) {
    return kFlash.ForwardVarlen(q, k, v, num_seqs, cu_q, cu_kv, max_seq_q, max_seq_kv, cfg);
}

DecodeConfig RecommendDecodeConfig(const AttentionShape& shape, const DeviceCapability& cap) {
    DecodeConfig cfg;
    cfg.max_splits = tables::kDispatch.max_splits;
    cfg.num_splits = tables::DecodeSplitsFor(shape.seq_kv, shape.batch, shape.num_kv_heads, shape.GroupSize(), cap.sm_count);
    return cfg;
}
sci::Result<AttentionResult> decode_attention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                              const AttentionConfig& cfg) {
    return kDecode.Forward(q, k, v, cfg);
}
sci::Result<AttentionResult> decode_attention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                              const AttentionConfig& cfg, const DecodeConfig& decode_cfg) {
    AttentionConfig resolved = cfg;
    resolved.num_splits = decode_cfg.num_splits;
    return kDecode.Forward(q, k, v, resolved);
}

sci::Result<AttentionResult> paged_attention(const sci::Tensor& q, const PagedKVCache& kv, const PagedAttentionParams& params,
                                             const AttentionConfig& cfg) {
    return RunPaged(q, kv, params, cfg);
}
sci::Result<AttentionResult> paged_prefill(const sci::Tensor& q, const PagedKVCache& kv, int64_t num_seqs,
                                           const int32_t* cu_seqlens_q, int64_t layer, const AttentionConfig& cfg) {
    const sci::StreamOrderedScope allocations_on_call_stream(StreamHandle(cfg.stream));
    const ApiRange nvtx_range("paged_prefill");
    const KVCacheConfig& kcfg = kv.Storage().Config();
    if (q.ndims() != 3 || cu_seqlens_q == nullptr) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_prefill expects q=[total_q, H_q, D] and host cu_seqlens_q");
    }
    const int64_t total_q = q.dim(0), heads = q.dim(1), d = q.dim(2);
    if (num_seqs < 1 || num_seqs > kv.MaxNumSeqs()) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_prefill num_seqs=" + std::to_string(num_seqs) +
                                                          " out of range [1," + std::to_string(kv.MaxNumSeqs()) + "]");
    }
    if (layer < 0 || layer >= kcfg.num_layers) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_prefill layer=" + std::to_string(layer) + " out of range [0," +
                                                          std::to_string(kcfg.num_layers) + ")");
    }
    if (q.dtype() != kcfg.dtype || (q.dtype() != sci::DType::kFloat16 && q.dtype() != sci::DType::kBFloat16)) {
        return Refuse(AttnStatusCode::kUnsupportedDtype, "paged_prefill computes in fp16/bf16 and q must have the cache's dtype");
    }
    if (d != kcfg.head_dim || SupportedHeadDimIndex(d) < 0 || kcfg.num_kv_heads < 1 || heads % kcfg.num_kv_heads != 0) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_prefill: q [*, " + std::to_string(heads) + ", " + std::to_string(d) +
                                                          "] does not fit the cache's heads / head_dim");
    }
    if (cu_seqlens_q[0] != 0 || cu_seqlens_q[num_seqs] != total_q) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_prefill: cu_seqlens_q must run from 0 to total_q");
    }
    std::vector<int32_t> have(static_cast<size_t>(num_seqs));
    for (int64_t s = 0; s < num_seqs; ++s) {
        const int64_t fresh = static_cast<int64_t>(cu_seqlens_q[s + 1]) - cu_seqlens_q[s];
        have[static_cast<size_t>(s)] = static_cast<int32_t>(kv.SeqLength(s));
        if (fresh < 1 || kv.SeqLength(s) < fresh) {
            return Refuse(AttnStatusCode::kShapeMismatch,
                          "paged_prefill: sequence " + std::to_string(s) + " brings " + std::to_string(fresh) +
                              " new tokens but the cache holds " + std::to_string(kv.SeqLength(s)) +
                              " (append the new tokens' K/V first)");
        }
    }
    if (kv.PageTableDevicePtr() == nullptr) {
        return Refuse(AttnStatusCode::kShapeMismatch, "paged_prefill has no page table (call PagedKVCache::SyncPageTable first)");
    }
    AttentionResult result;
    result.out = sci::Tensor(sci::TensorShape({total_q, heads, d}), q.dtype(), q.device());
    const long long ws_bytes = sca_flash_varlen_workspace_bytes(num_seqs, total_q);
    sci::Tensor workspace(sci::TensorShape({static_cast<sci::index_t>(ws_bytes > 0 ? ws_bytes : 16)}), sci::DType::kUInt8, q.device());
    if (result.out.data() == nullptr || workspace.data() == nullptr) {
        return Refuse(AttnStatusCode::kWorkspaceExceeded, "allocation of the paged prefill output failed");
    }
    AttentionShape shape;
    shape.batch = num_seqs;
    shape.seq_q = total_q;
    shape.seq_kv = total_q;
    shape.num_heads = heads;
    shape.num_kv_heads = kcfg.num_kv_heads;
    shape.head_dim = d;
    ScaFlashPagedParams p{};
    p.q = q.data();
    p.out = result.out.data();
    p.k_pool = kv.Storage().K(layer).data();
    p.v_pool = kv.Storage().V(layer).data();
    p.page_table = kv.PageTableDevicePtr();
    p.total_q = total_q;
    p.num_heads = heads;
    p.num_kv_heads = kcfg.num_kv_heads;
    p.head_dim = d;
    p.num_seqs = num_seqs;
    p.num_blocks = kcfg.num_blocks;
    p.block_size = kv.BlockSize();
    p.max_blocks_per_seq = kv.MaxBlocksPerSeq();
    p.cu_seqlens_q = cu_seqlens_q;
    p.seq_lens_kv = have.data();
    p.scale = EffectiveScale(cfg, shape);
    p.causal = cfg.causal ? 1 : 0;
    p.dtype_id = DtypeId(q.dtype());
    p.workspace = workspace.data();
    p.workspace_bytes = ws_bytes;
    if (sci::Status s = FromAbi(sca_launch_flash_paged(&p, StreamHandle(cfg.stream))); !s.ok()) {
        return sci::MakeUnexpected<AttentionResult>(s);
    }
    // `workspace` is released when this scope ends: the free is ordered on the call's stream, behind the kernel
    result.stats.used_backend = BackendKind::kFlash;
    result.stats.workspace_bytes = 0;
    result.stats.materialized_score_bytes = 0;
    result.stats.kv_bytes = kv.Storage().MemoryBytes();
    result.stats.note = "chunked prefill over the paged cache: " + std::to_string(num_seqs) + " sequences, " +
                        std::to_string(total_q) + " new tokens, block_size=" + std::to_string(kv.BlockSize()) +
                        ", layer=" + std::to_string(layer);
    return sci::Ok(std::move(result));
}

sci::Result<AttentionResult> paged_attention(const sci::Tensor& q, const PagedKVCache& kv, const AttentionConfig& cfg) {
    PagedAttentionParams params;
    params.page_table = kv.PageTableDevicePtr();
    params.num_seqs = kv.MaxNumSeqs();
    params.block_size = kv.BlockSize();
    params.max_blocks_per_seq = kv.MaxBlocksPerSeq();
    params.layer = 0;
    // The cache keeps a device copy of its sequence lengths (current after SyncPageTable / AppendTokenBatch, which this
    // form needs anyway for the table). The reference passes no lengths here and scans every mapped slot, so the
    // zero-filled tail of a sequence's last block takes softmax weight; with the lengths the result is the attention
    // over exactly the stored tokens. Identical whenever every length is a multiple of block_size.
    params.seq_lens = kv.SeqLensDevicePtr();
    return RunPaged(q, kv, params, cfg);
}

}  // namespace sca
