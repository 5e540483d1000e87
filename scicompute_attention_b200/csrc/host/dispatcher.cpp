// Shape inference and table-driven backend selection. Select() and Explain() share one code path, so
// the explanation can never drift from what Forward() executes. Decision rules and reason wording follow
// src/runtime/dispatcher.cpp:38-246 of the reference; thresholds come from tables::kDispatch.
#include <initializer_list>

#include "internal.hpp"

namespace sca {
namespace {

std::string ShapeSummary(const AttentionShape& s) {
    return "B=" + std::to_string(s.batch) + ",Hq=" + std::to_string(s.num_heads) + ",Hkv=" +
           std::to_string(s.num_kv_heads) + ",Sq=" + std::to_string(s.seq_q) + ",Skv=" + std::to_string(s.seq_kv) +
           ",D=" + std::to_string(s.head_dim);
}

std::string DimList(const sci::Tensor& t) {
    return "[" + std::to_string(t.dim(0)) + "," + std::to_string(t.dim(1)) + "," + std::to_string(t.dim(2)) + "," +
           std::to_string(t.dim(3)) + "]";
}

// Next candidates when the preferred backend cannot serve a request and the caller opted in.
std::initializer_list<BackendKind> FallbackCandidates(BackendKind preferred) {
    static constexpr std::initializer_list<BackendKind> after_flash = {BackendKind::kTiled, BackendKind::kNaive};
    static constexpr std::initializer_list<BackendKind> after_decode = {BackendKind::kFlash, BackendKind::kTiled, BackendKind::kNaive};
    static constexpr std::initializer_list<BackendKind> after_paged = {BackendKind::kDecode, BackendKind::kTiled, BackendKind::kNaive};
    static constexpr std::initializer_list<BackendKind> after_tiled = {BackendKind::kNaive};
    static constexpr std::initializer_list<BackendKind> none = {};
    switch (preferred) {
        case BackendKind::kFlash: return after_flash;
        case BackendKind::kDecode: return after_decode;
        case BackendKind::kPaged: return after_paged;
        case BackendKind::kTiled: return after_tiled;
        default: return none;
    }
}

}  // namespace

sci::Result<AttentionShape> InferShape(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v, AttnLayout layout) {
    auto fail = [](AttnStatusCode code, const std::string& text) {
        return sci::MakeUnexpected<AttentionShape>(MakeStatus(code, text));
    };
    if (!detail::LayoutSupported(layout)) {
        return fail(AttnStatusCode::kUnsupportedLayout, std::string("layout=") + LayoutName(layout) + " (supported: bhsd, bshd)");
    }
    for (const sci::Tensor* t : {&q, &k, &v}) {
        if (t->ndims() != 4) {
            return fail(AttnStatusCode::kShapeMismatch, "tensor ndims=" + std::to_string(t->ndims()) + " (expected 4)");
        }
        if (!t->is_contiguous()) {
            return fail(AttnStatusCode::kLayoutMismatch,
                        "non-contiguous input rejected; call .clone() or pass a contiguous tensor");
        }
        if (!IsSupportedComputeDtype(t->dtype())) {
            return fail(AttnStatusCode::kUnsupportedDtype, std::string("dtype=") + sci::kDTypeName(t->dtype()) +
                                                               " (supported: float32, float16, bfloat16)");
        }
        if (t->device_type() != sci::DeviceType::kCUDA) {
            return fail(AttnStatusCode::kUnsupportedFeature, std::string("device=") + sci::kDeviceTypeName(t->device_type()) +
                                                                 " (v1 executes attention kernels on CUDA devices only)");
        }
    }
    if (q.dtype() != k.dtype() || q.dtype() != v.dtype()) {
        return fail(AttnStatusCode::kUnsupportedDtype, std::string("dtype mismatch: q=") + sci::kDTypeName(q.dtype()) +
                                                           ", k=" + sci::kDTypeName(k.dtype()) + ", v=" +
                                                           sci::kDTypeName(v.dtype()));
    }
    const bool bhsd = layout == AttnLayout::kBHSD;
    const int head_axis = bhsd ? 1 : 2, seq_axis = bhsd ? 2 : 1;
    AttentionShape shape;
    shape.batch = q.dim(0);
    shape.num_heads = q.dim(head_axis);
    shape.seq_q = q.dim(seq_axis);
    shape.head_dim = q.dim(3);
    shape.num_kv_heads = k.dim(head_axis);
    shape.seq_kv = k.dim(seq_axis);
    if (v.dim(head_axis) != shape.num_kv_heads || v.dim(seq_axis) != shape.seq_kv || v.dim(3) != shape.head_dim) {
        return fail(AttnStatusCode::kShapeMismatch,
                    bhsd ? "k/v shape mismatch: k=[B,Hkv,Skv,D]=" + ShapeSummary(shape) + ", v=" + DimList(v)
                         : "k/v shape mismatch for bshd: v=" + DimList(v));
    }
    if (k.dim(0) != shape.batch || v.dim(0) != shape.batch) {
        return fail(AttnStatusCode::kShapeMismatch, "batch mismatch: q=" + std::to_string(shape.batch) + ", k=" +
                                                        std::to_string(k.dim(0)) + ", v=" + std::to_string(v.dim(0)));
    }
    return sci::Ok(shape);
}

DispatchDecision AttentionDispatcher::Select(const AttentionConfig& cfg, const AttentionShape& shape) const {
    DispatchDecision decision;
    std::string detail;
    if (!Validate(cfg, shape, &detail).ok()) {
        decision.reason = "invalid: " + detail;
        return decision;
    }
    const tables::DispatchThresholds& th = tables::kDispatch;
    const std::string sq = std::to_string(shape.seq_q), skv = std::to_string(shape.seq_kv);
    BackendKind preferred = cfg.backend;
    std::string prefix = "auto", why;
    if (preferred != BackendKind::kAuto) {
        prefix = "explicit";
        why = std::string("backend=") + BackendName(preferred);
    } else if (shape.seq_q <= th.decode_max_seq_q && shape.seq_kv >= th.decode_min_seq_kv) {
        preferred = BackendKind::kDecode;
        why = "seq_q=" + sq + " <=" + std::to_string(th.decode_max_seq_q) + " and seq_kv=" + skv + " >= " +
              std::to_string(th.decode_min_seq_kv) + " => decode (low arithmetic intensity)";
    } else if (shape.seq_q * 8 <= shape.seq_kv && shape.seq_kv >= th.decode_min_seq_kv) {
        preferred = BackendKind::kFlash;
        why = "seq_q*8=" + std::to_string(shape.seq_q * 8) + " <= seq_kv=" + skv +
              " => grouped small-q prefill on flash (decode kernel is S_q=1 only)";
    } else if (shape.seq_kv <= th.tiled_max_seq_kv) {
        preferred = BackendKind::kTiled;
        why = "seq_kv=" + skv + " <= " + std::to_string(th.tiled_max_seq_kv) + " => tiled (short sequence, smem resident)";
    } else {
        preferred = BackendKind::kFlash;
        why = "seq_q=" + sq + ", seq_kv=" + skv + " => flash (tile + online softmax)";
    }

    decision.backend = preferred;
    decision.tile = RecommendTile(cfg, shape);
    const CapabilityReport report = GetBackend(preferred)->Supports(cfg, shape);
    decision.workspace_bytes = report.workspace_bytes;
    const std::string head = prefix + ": " + why;
    if (report.supported) {
        if (!report.tile.Empty()) decision.tile = report.tile;
        decision.reason = head + " [table=" + th.revision + ", workspace=" + std::to_string(decision.workspace_bytes) + " B]";
        return decision;
    }
    const std::string refusal = head + " => unsupported(" + BackendName(preferred) + "): " + report.reason;
    if (!cfg.allow_fallback) {
        decision.reason = refusal + " [table=" + th.revision + ", allow_fallback=false]";
        return decision;
    }
    for (BackendKind candidate : FallbackCandidates(preferred)) {
        const CapabilityReport alt = GetBackend(candidate)->Supports(cfg, shape);
        if (!alt.supported) continue;
        decision.backend = candidate;
        if (!alt.tile.Empty()) decision.tile = alt.tile;
        decision.workspace_bytes = alt.workspace_bytes;
        decision.reason = std::string("fallback: ") + BackendName(preferred) + " unsupported (" + report.reason + ") => " +
                          BackendName(candidate) + "; " + head + " [table=" + th.revision + ", allow_fallback=true]";
        return decision;
    }
    decision.reason = refusal + "; no fallback backend supports shape " + ShapeSummary(shape);
    return decision;
}

std::string AttentionDispatcher::Explain(const AttentionConfig& cfg, const AttentionShape& shape) const {
    const DispatchDecision d = Select(cfg, shape);
    return std::string("backend=") + BackendName(d.backend) + "; tile={" + d.tile.ToString() + "}; workspace=" +
           std::to_string(d.workspace_bytes) + " B; reason=" + d.reason;
}

sci::Result<AttentionResult> AttentionDispatcher::Forward(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                                          const AttentionConfig& cfg) const {
    const sci::Result<AttentionShape> shape = InferShape(q, k, v, cfg.layout);
    if (!shape.ok()) return sci::MakeUnexpected<AttentionResult>(shape.error());
    const DispatchDecision decision = Select(cfg, *shape);
    if (decision.backend == BackendKind::kAuto) {
        return sci::MakeUnexpected<AttentionResult>(MakeStatus(AttnStatusCode::kShapeMismatch, decision.reason));
    }
    const IAttentionBackend* backend = GetBackend(decision.backend);
    const CapabilityReport report = backend->Supports(cfg, *shape);
    if (!report.supported) {
        return sci::MakeUnexpected<AttentionResult>(MakeStatus(AttnStatusCode::kDeviceCapability, report.reason));
    }
    return backend->Forward(q, k, v, cfg);
}

sci::Result<AttentionResult> AttentionDispatcher::Forward(const sci::Tensor& q, const sci::Tensor& k,
                                                          const sci::Tensor& v) const {
    return Forward(q, k, v, default_cfg_);
}

sci::Status AttentionDispatcher::ReloadDispatchTable(const char* path) {
    if (path == nullptr) return sci::Status::Ok();
    return sci::Status::NotImplemented(
        std::string("runtime dispatch-table reload requires the threshold sweep tool; compiled-in table \"") +
        tables::kDispatch.revision + "\" is in use");
}

// ---- top-level entry points -----------------------------------------------------------------------------
sci::Result<AttentionResult> attention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                       const AttentionConfig& cfg) {
    return AttentionDispatcher(cfg).Forward(q, k, v, cfg);
}

sci::Result<AttentionResult> decode(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v,
                                    const AttentionConfig& cfg) {
    AttentionConfig c = cfg;
    c.backend = BackendKind::kDecode;
    return attention(q, k, v, c);
}

sci::Result<AttentionResult> paged(const sci::Tensor& q, const PagedKVCache& kv, const AttentionConfig& cfg) {
    AttentionConfig c = cfg;
    c.backend = BackendKind::kPaged;
    return paged_attention(q, kv, PagedAttentionParams{}, c);
}

std::string ExplainAttention(const sci::Tensor& q, const sci::Tensor& k, const sci::Tensor& v, const AttentionConfig& cfg) {
    const sci::Result<AttentionShape> shape = InferShape(q, k, v, cfg.layout);
    if (!shape.ok()) return "invalid: " + shape.message();
    return AttentionDispatcher(cfg).Explain(cfg, *shape);
}

}  // namespace sca
