// Tests of the public C++ API (namespace sca), written against include/scicompute_attention/ only.
// They follow the reference's own suites - tests/unit (config, status, dispatch, tile, capability),
// tests/kernel (flash / decode / paged / naive / tiled correctness, numerics) and tests/kv - with the
// same seeds, shapes and assertions where the behaviour is shared, and the Blackwell tile / split
// tables where it deliberately differs. Expected outputs come from the FP64 oracle (oracle/liboracle.so,
// a checker that is linked into this test binary only).
#include <algorithm>
#include <cstdlib>
#include <memory>
#include <numeric>

#include <cuda_runtime_api.h>

#include "device/cuda_device.hpp"
#include "device/stream.hpp"
#include "mini_test.hpp"
#include "scicompute_attention/attention.hpp"

extern "C" {
void oracle_random_floats(float* out, size_t count, uint32_t seed, float low, float high);
void oracle_encode(const float* values, size_t count, int dtype, uint16_t* bits_out, float* dequant_out);
int oracle_attention_f64(const float* q, const float* k, const float* v, int64_t batch, int64_t heads_q, int64_t heads_kv,
                         int64_t seq_q, int64_t seq_kv, int64_t head_dim, int causal, double scale, double* out,
                         double* lse, int threads);
float oracle_half_bits_to_float(uint16_t);
float oracle_bf16_bits_to_float(uint16_t);
}

namespace {

using sci::DType;

std::shared_ptr<sci::Device> Gpu() {
    if (!sca::DeviceCapability::CudaAvailable()) return nullptr;
    return sci::DeviceManager::Instance().get_device(sci::DeviceType::kCUDA, 0);
}

int OracleDtype(DType dt) { return dt == DType::kFloat32 ? 0 : dt == DType::kFloat16 ? 1 : 2; }

struct Encoded {
    std::vector<uint8_t> bytes;
    std::vector<float> dequantized;
};

Encoded Encode(const std::vector<float>& values, DType dt) {
    Encoded e;
    e.dequantized.resize(values.size());
    if (dt == DType::kFloat32) {
        e.bytes.resize(values.size() * 4);
        std::memcpy(e.bytes.data(), values.data(), e.bytes.size());
        e.dequantized = values;
    } else {
        e.bytes.resize(values.size() * 2);
        oracle_encode(values.data(), values.size(), OracleDtype(dt), reinterpret_cast<uint16_t*>(e.bytes.data()),
                      e.dequantized.data());
    }
    return e;
}

std::vector<float> RandomFloats(size_t n, uint32_t seed, float lo = -1.0f, float hi = 1.0f) {
    std::vector<float> v(n);
    oracle_random_floats(v.data(), n, seed, lo, hi);
    return v;
}

sci::Tensor ToDevice(const std::vector<sci::index_t>& dims, DType dt, const std::vector<uint8_t>& bytes, sci::Device& dev) {
    sci::Tensor t(sci::TensorShape(dims), dt, dev);
    t.copy_from(bytes.data(), bytes.size());
    return t;
}
sci::Tensor ToDeviceI32(const std::vector<int32_t>& v, sci::Device& dev) {
    sci::Tensor t(sci::TensorShape({static_cast<sci::index_t>(v.size())}), DType::kInt32, dev);
    t.copy_from(v.data(), v.size() * 4);
    return t;
}

std::vector<float> ReadFloats(const sci::Tensor& t) {
    sci::Tensor host(t.shape(), t.dtype(), sci::HostDevice());
    host.copy_from(t);
    const size_t n = static_cast<size_t>(t.num_elements());
    std::vector<float> out(n);
    if (t.dtype() == DType::kFloat32) {
        std::memcpy(out.data(), host.data(), n * 4);
    } else {
        const uint16_t* src = static_cast<const uint16_t*>(host.data());
        for (size_t i = 0; i < n; ++i) {
            out[i] = t.dtype() == DType::kFloat16 ? oracle_half_bits_to_float(src[i]) : oracle_bf16_bits_to_float(src[i]);
        }
    }
    return out;
}

struct Err {
    double max_abs = 0, mean_abs = 0;
};
Err Compare(const std::vector<float>& got, const std::vector<double>& expect) {
    Err e;
    double sum = 0;
    for (size_t i = 0; i < got.size(); ++i) {
        const double d = std::fabs(double(got[i]) - expect[i]);
        e.max_abs = std::max(e.max_abs, d);
        sum += d;
    }
    e.mean_abs = got.empty() ? 0 : sum / double(got.size());
    return e;
}
// the reference's own bounds (tests/common/test_utils.hpp:293-299)
Err Tolerance(DType dt) {
    if (dt == DType::kFloat32) return {1e-4, 1e-6};
    if (dt == DType::kFloat16) return {5e-3, 5e-4};
    return {2e-2, 2e-3};
}

struct AttnCase {
    DType dtype = DType::kFloat16;
    bool causal = false;
    int64_t batch = 1, hq = 8, hkv = 8, sq = 128, skv = 128, d = 128;
    uint32_t seed = 1;
    sca::AttnLayout layout = sca::AttnLayout::kBHSD;
    float magnitude = 1.0f;
};

using Runner = sci::Result<sca::AttentionResult> (*)(const sci::Tensor&, const sci::Tensor&, const sci::Tensor&,
                                                     const sca::AttentionConfig&);

// Runs `fn` on seeded inputs and compares with the oracle; returns the result for further checks.
bool RunCase(const char* what, Runner fn, const AttnCase& c, sca::AttentionConfig cfg, sca::AttentionRuntimeStats* stats_out = nullptr,
             bool check_lse = false) {
    auto dev = Gpu();
    const size_t qn = size_t(c.batch * c.hq * c.sq * c.d), kn = size_t(c.batch * c.hkv * c.skv * c.d);
    const Encoded q = Encode(RandomFloats(qn, c.seed, -c.magnitude, c.magnitude), c.dtype);
    const Encoded k = Encode(RandomFloats(kn, c.seed + 101, -c.magnitude, c.magnitude), c.dtype);
    const Encoded v = Encode(RandomFloats(kn, c.seed + 202), c.dtype);
    sci::Tensor qt = ToDevice({c.batch, c.hq, c.sq, c.d}, c.dtype, q.bytes, *dev);
    sci::Tensor kt = ToDevice({c.batch, c.hkv, c.skv, c.d}, c.dtype, k.bytes, *dev);
    sci::Tensor vt = ToDevice({c.batch, c.hkv, c.skv, c.d}, c.dtype, v.bytes, *dev);
    cfg.causal = c.causal;
    cfg.return_lse = check_lse;
    const auto result = fn(qt, kt, vt, cfg);
    const std::string tag = std::string(what) + " dtype=" + sci::kDTypeName(c.dtype) + " causal=" + (c.causal ? "1" : "0") +
                            " B=" + std::to_string(c.batch) + " Hq=" + std::to_string(c.hq) + " Hkv=" + std::to_string(c.hkv) +
                            " Sq=" + std::to_string(c.sq) + " Skv=" + std::to_string(c.skv) + " D=" + std::to_string(c.d) +
                            " seed=" + std::to_string(c.seed);
    if (!result.ok()) {
        mini::Fail(__FILE__, __LINE__, tag + ": " + result.error().ToString());
        return false;
    }
    dev->synchronize();
    std::vector<double> expect(qn), lse(size_t(c.batch * c.hq * c.sq));
    oracle_attention_f64(q.dequantized.data(), k.dequantized.data(), v.dequantized.data(), c.batch, c.hq, c.hkv, c.sq, c.skv,
                         c.d, c.causal ? 1 : 0, 0.0, expect.data(), check_lse ? lse.data() : nullptr, 8);
    const Err e = Compare(ReadFloats(result->out), expect), tol = Tolerance(c.dtype);
    bool ok = true;
    if (!(e.max_abs <= tol.max_abs) || !(e.mean_abs <= tol.mean_abs)) {
        mini::Fail(__FILE__, __LINE__, tag + ": max_abs=" + std::to_string(e.max_abs) + " mean_abs=" + std::to_string(e.mean_abs));
        ok = false;
    }
    if (check_lse) {
        const std::vector<float> got = ReadFloats(result->lse);
        double worst = 0;
        for (size_t i = 0; i < got.size(); ++i) worst = std::max(worst, std::fabs(double(got[i]) - lse[i]));
        if (got.size() != lse.size() || worst > 1e-2) {
            mini::Fail(__FILE__, __LINE__, tag + ": LSE max abs error " + std::to_string(worst));
            ok = false;
        }
    }
    if (stats_out != nullptr) *stats_out = result->stats;
    return ok;
}

sca::AttentionShape Shape(int64_t sq, int64_t skv, int64_t d = 128, int64_t b = 1, int64_t hq = 8, int64_t hkv = 8) {
    sca::AttentionShape s;
    s.batch = b;
    s.seq_q = sq;
    s.seq_kv = skv;
    s.num_heads = hq;
    s.num_kv_heads = hkv;
    s.head_dim = d;
    return s;
}

}  // namespace

// ================================================================================================
// unit level (no GPU needed)
// ================================================================================================
TEST(Config, AcceptsEverySupportedHeadDimAndNamesRejectedValues) {
    for (int64_t i = 0; i < sca::kNumSupportedHeadDims; ++i) {
        EXPECT_TRUE(sca::Validate(sca::AttentionConfig{}, Shape(64, 64, sca::kSupportedHeadDims[i])).ok());
    }
    std::string detail;
    const sci::Status bad = sca::Validate(sca::AttentionConfig{}, Shape(64, 64, 48), &detail);
    EXPECT_EQ(sca::ExtractCode(bad), sca::AttnStatusCode::kUnsupportedHeadDim);
    EXPECT_HAS(detail, "head_dim=48");
    EXPECT_HAS(detail, "128");
    sca::AttentionConfig causal;
    causal.causal = true;
    EXPECT_FALSE(sca::Validate(causal, Shape(256, 128), &detail).ok());
    EXPECT_HAS(detail, "seq_kv(128)");
    EXPECT_HAS(detail, "seq_q(256)");
    const sci::Status gqa = sca::Validate(sca::AttentionConfig{}, Shape(64, 64, 128, 1, 32, 6));
    EXPECT_EQ(sca::ExtractCode(gqa), sca::AttnStatusCode::kShapeMismatch);
    EXPECT_HAS(gqa.message(), "num_kv_heads=6");
    sca::AttentionConfig window;
    window.sliding_window = 512;
    EXPECT_EQ(sca::ExtractCode(sca::Validate(window, Shape(64, 64))), sca::AttnStatusCode::kUnsupportedFeature);
    sca::AttentionConfig softcap;
    softcap.softcap = 50.0f;
    softcap.backend = sca::BackendKind::kNaive;
    EXPECT_FALSE(sca::Validate(softcap, Shape(64, 64)).ok());
    softcap.backend = sca::BackendKind::kFlash;
    EXPECT_TRUE(sca::Validate(softcap, Shape(64, 64)).ok());
}

TEST(Config, DefaultScaleAndVarlenMetadata) {
    sca::AttentionConfig cfg;
    EXPECT_NEAR(sca::EffectiveScale(cfg, Shape(64, 64, 128)), 1.0f / std::sqrt(128.0f), 1e-7);
    cfg.scale = 0.5f;
    EXPECT_EQ(sca::EffectiveScale(cfg, Shape(64, 64, 128)), 0.5f);
    cfg.scale = 0.0f;
    EXPECT_NEAR(sca::EffectiveScale(cfg, Shape(64, 64, 64)), 0.125f, 1e-7);
    const int32_t good[] = {0, 5, 9, 20};
    int64_t longest = 0;
    EXPECT_TRUE(sca::ValidateVarlenHost(good, 3, &longest).ok());
    EXPECT_EQ(longest, 11);
    const int32_t flat[] = {0, 5, 5};
    EXPECT_EQ(sca::ExtractCode(sca::ValidateVarlenHost(flat, 2)), sca::AttnStatusCode::kShapeMismatch);
    EXPECT_FALSE(sca::ValidateVarlenHost(nullptr, 2).ok());
}

TEST(Status, CodesNamesAndVersion) {
    const sci::Status s = sca::MakeStatus(sca::AttnStatusCode::kKVCapacityExceeded, "requested 40 blocks, free 8");
    EXPECT_EQ(s.code(), sci::StatusCode::kResourceExhausted);
    EXPECT_EQ(sca::ExtractCode(s), sca::AttnStatusCode::kKVCapacityExceeded);
    EXPECT_HAS(s.message(), "[SCA-2007]");
    EXPECT_EQ(sca::ToSciCode(sca::AttnStatusCode::kUnsupportedFeature), sci::StatusCode::kNotImplemented);
    EXPECT_EQ(sca::ToSciCode(sca::AttnStatusCode::kDeviceCapability), sci::StatusCode::kInvalidOperation);
    EXPECT_EQ(sca::ExtractCode(sci::Status::Ok()), sca::AttnStatusCode::kOk);
    EXPECT_STREQ(sca::ToString(sca::AttnStatusCode::kKVCapacityExceeded), "KVCapacityExceeded");
    EXPECT_STREQ(sca::BackendName(sca::BackendKind::kFlash), "flash");
    EXPECT_STREQ(sca::LayoutName(sca::AttnLayout::kBSHD), "bshd");
    EXPECT_STREQ(sca::VersionString(), SCI_ATTENTION_VERSION_STRING);
    EXPECT_EQ(sca::SupportedHeadDimIndex(128), 3);
    EXPECT_EQ(sca::SupportedHeadDimIndex(48), -1);
    EXPECT_TRUE(sca::IsSupportedComputeDtype(DType::kFloat32));
    EXPECT_FALSE(sca::IsSupportedComputeDtype(DType::kInt8));
    sca::BackendKind kind;
    EXPECT_TRUE(sca::ParseBackendName("paged", &kind));
    EXPECT_EQ(int(kind), int(sca::BackendKind::kPaged));
    EXPECT_FALSE(sca::ParseBackendName("nope", &kind));
}

TEST(Dispatch, RulesAndReasons) {
    const sca::AttentionDispatcher d;
    sca::DispatchDecision dec = d.Select(sca::AttentionConfig{}, Shape(1, 2048));
    EXPECT_EQ(int(dec.backend), int(sca::BackendKind::kDecode));
    EXPECT_HAS(dec.reason, "auto");
    EXPECT_HAS(dec.reason, "table=b200-r1");
    dec = d.Select(sca::AttentionConfig{}, Shape(16, 4096));
    EXPECT_EQ(int(dec.backend), int(sca::BackendKind::kFlash));
    EXPECT_HAS(dec.reason, "grouped small-q");
    dec = d.Select(sca::AttentionConfig{}, Shape(1024, 1024));
    EXPECT_EQ(int(dec.backend), int(sca::BackendKind::kFlash));
    EXPECT_HAS(dec.reason, "online softmax");
    dec = d.Select(sca::AttentionConfig{}, Shape(64, 64));
    EXPECT_EQ(int(dec.backend), int(sca::BackendKind::kTiled));
    EXPECT_HAS(dec.reason, "short sequence");
    sca::AttentionConfig naive;
    naive.backend = sca::BackendKind::kNaive;
    dec = d.Select(naive, Shape(1024, 1024));
    EXPECT_EQ(int(dec.backend), int(sca::BackendKind::kNaive));
    EXPECT_HAS(dec.reason, "explicit");
    dec = d.Select(sca::AttentionConfig{}, Shape(1024, 64, 48));
    EXPECT_EQ(int(dec.backend), int(sca::BackendKind::kAuto));
    EXPECT_HAS(dec.reason, "head_dim=48");
    const std::string text = d.Explain(sca::AttentionConfig{}, Shape(1024, 1024));
    EXPECT_HAS(text, "backend=");
    EXPECT_HAS(text, "tile={bm=");
    EXPECT_HAS(text, "workspace=");
    EXPECT_HAS(text, "reason=");
    // Blackwell tile table: 128-row query tiles everywhere, 12 warps, TMA on
    EXPECT_EQ(d.Select(sca::AttentionConfig{}, Shape(1024, 1024, 128)).tile.block_m, 128);
    EXPECT_EQ(d.Select(sca::AttentionConfig{}, Shape(1024, 1024, 256)).tile.block_n, 64);
    EXPECT_EQ(d.Select(sca::AttentionConfig{}, Shape(1024, 1024, 64)).tile.warps, 12);
    EXPECT_FALSE(sca::AttentionDispatcher::ReloadDispatchTable("x.json").ok());
    EXPECT_TRUE(sca::AttentionDispatcher::ReloadDispatchTable(nullptr).ok());
}

TEST(Tile, FootprintFormulaAndStrings) {
    EXPECT_EQ(sca::TileConfig::SmemBytesFlash(128, 2, 64, 64, 4, 2), 87040);
    EXPECT_LT(sca::TileConfig::SmemBytesFlash(0, 2, 64, 64, 4, 2), 0);
    EXPECT_LT(sca::TileConfig::SmemBytesFlash(128, 2, 64, 64, 4, 0), 0);
    sca::TileConfig t;
    t.block_m = 64;
    t.block_n = 64;
    t.warps = 4;
    t.stages = 2;
    EXPECT_EQ(t.ToString(), std::string("bm=64,bn=64,warps=4,stages=2,tma=off"));
    EXPECT_EQ(t.Threads(), 128);
    EXPECT_TRUE(sca::TileConfig{}.Empty());
    const sca::detail::Strides s = sca::detail::StridesFor(sca::AttnLayout::kBSHD, 10, 4, 64);
    EXPECT_EQ(s.s_b, 10 * 4 * 64);
    EXPECT_EQ(s.s_s, 4 * 64);
    EXPECT_EQ(s.s_h, 64);
    EXPECT_EQ(sca::detail::CeilDiv<int64_t>(17, 16), 2);
}

TEST(Workspace, SlicesAreBoundsAndOverlapChecked) {
    auto ws = sca::Workspace::Create(4096, sci::HostDevice());
    ASSERT_TRUE(ws.ok());
    EXPECT_TRUE(ws->Slice(0, 1024).ok());
    EXPECT_TRUE(ws->Slice(0, 1024).ok());            // identical slice may be taken again
    EXPECT_FALSE(ws->Slice(512, 1024).ok());         // partial overlap
    EXPECT_FALSE(ws->Slice(100, 16).ok());           // misaligned
    EXPECT_FALSE(ws->Slice(3840, 512).ok());         // out of range
    EXPECT_TRUE(ws->Slice(1024, 2048).ok());
    EXPECT_EQ(ws->AllocatedSlices(), 2u);
    EXPECT_EQ(ws->PeakBytes(), 3072u);
    EXPECT_TRUE(ws->Reset().ok());
    EXPECT_TRUE(ws->Slice(512, 1024, 512).ok());
    EXPECT_FALSE(sca::Workspace::Create(0, sci::HostDevice()).ok());
}

TEST(BlockManager, LifoOrderCountersAndTableRows) {
    auto r = sca::BlockManager::Create(16, 3, 4, sci::HostDevice());
    ASSERT_TRUE(r.ok());
    sca::BlockManager m = std::move(*r);
    const auto a = m.Allocate(2), b = m.Allocate(2);
    ASSERT_TRUE(a.ok() && b.ok());
    EXPECT_EQ((*a)[0], 0);
    EXPECT_EQ((*b)[1], 3);
    ASSERT_TRUE(m.AppendToTable(0, a->data(), 2).ok());
    ASSERT_TRUE(m.AppendToTable(1, b->data(), 2).ok());
    const sca::BlockTable& t = m.Table();
    EXPECT_EQ(t.host[0], 0);
    EXPECT_EQ(t.host[2], -1);
    EXPECT_EQ(t.host[4], 2);
    const uint64_t before = t.revision;
    ASSERT_TRUE(m.ResetSeq(0).ok());
    EXPECT_EQ(t.host[0], -1);
    EXPECT_GT(t.revision, before);
    EXPECT_EQ(m.NumFreeBlocks(), 14);
    EXPECT_TRUE(m.SyncTableToDevice(nullptr).ok());
    EXPECT_TRUE(m.SyncTableToDevice(nullptr).ok());
    EXPECT_FALSE(m.Allocate(0).ok());
    EXPECT_FALSE(m.AppendToTable(7, nullptr, 1).ok());
    const auto too_many = m.Allocate(15);
    ASSERT_FALSE(too_many.ok());
    EXPECT_HAS(too_many.error().message(), "only 14 of 16");
    EXPECT_EQ(m.AllocationFailures(), 1);
    m.Free(b->data(), 2);
    m.Free(b->data(), 2);
    EXPECT_EQ(m.DoubleFreeEvents(), 2);
}

TEST(KvCache, BudgetSlotMappingAndInvalidConfigs) {
    sca::KVCacheConfig cfg;
    cfg.num_layers = 32;
    cfg.num_kv_heads = 8;
    cfg.head_dim = 128;
    cfg.block_size = 16;
    cfg.num_blocks = 1536;
    cfg.max_num_seqs = 4;
    const auto bytes = sca::KvCacheBytes(cfg);
    ASSERT_TRUE(bytes.ok());
    EXPECT_EQ(*bytes, 3221225472ull);
    EXPECT_EQ(sca::MaxBlocksForBudget(cfg, *bytes), 1536);
    EXPECT_EQ(sca::MaxBlocksForBudget(cfg, *bytes / 2), 768);
    cfg.block_size = 7;
    EXPECT_FALSE(sca::KvCacheBytes(cfg).ok());
    const int32_t table[] = {3, 1, 0, -1};
    const auto slots = sca::ComputeSlotMapping(table, 17, 5, 16, 4);
    ASSERT_TRUE(slots.ok());
    EXPECT_EQ((*slots)[0], 17);
    EXPECT_EQ((*slots)[4], 21);
    const auto empty = sca::ComputeSlotMapping(table, 48, 1, 16, 4);
    ASSERT_FALSE(empty.ok());
    EXPECT_HAS(empty.error().message(), "empty");
}

// ================================================================================================
// device level
// ================================================================================================
TEST(Capability, ProbeReportsBlackwellFeatures) {
    if (!Gpu()) SKIP_TEST("no CUDA device");
    const sca::DeviceCapability& cap = sca::DeviceCapability::ForDevice(0);
    EXPECT_FALSE(cap.device_name.empty());
    EXPECT_GE(cap.sm_count, 1);
    EXPECT_GT(cap.smem_per_sm, 0u);
    EXPECT_TRUE(cap.has_mma_m16n8k16);
    EXPECT_TRUE(cap.has_cp_async);
    EXPECT_TRUE(cap.has_tma_bulk);
    EXPECT_FALSE(cap.has_wgmma);
    EXPECT_FALSE(cap.has_fp8_mma);
    if (cap.major == 10) {
        EXPECT_TRUE(cap.has_tcgen05);
        EXPECT_EQ(cap.tmem_columns, 512);
    }
    const size_t natural = sca::DeviceCapability::SmemLimitPerBlock(cap);
    setenv("SCI_ATTENTION_MAX_SMEM_BYTES", "49152", 1);
    EXPECT_EQ(sca::DeviceCapability::SmemLimitPerBlock(cap), 49152u);
    unsetenv("SCI_ATTENTION_MAX_SMEM_BYTES");
    EXPECT_EQ(sca::DeviceCapability::SmemLimitPerBlock(cap), natural);
    EXPECT_TRUE(sca::DeviceCapability::Refresh(0).ok());
}

TEST(Flash, DtypesCausalAndEveryHeadDim) {
    if (!Gpu()) SKIP_TEST("no CUDA device");
    uint32_t seed = 40000;
    for (DType dt : {DType::kFloat16, DType::kBFloat16}) {
        for (bool causal : {false, true}) {
            for (int64_t d : {32, 64, 96, 128, 160, 192, 256}) {
                AttnCase c;
                c.dtype = dt;
                c.causal = causal;
                c.hq = c.hkv = 4;
                c.d = d;
                c.seed = seed++;
                sca::AttentionRuntimeStats st;
                if (!RunCase("flash", sca::flash_attention, c, {}, &st)) return;
                EXPECT_EQ(st.workspace_bytes, 0u);
                EXPECT_EQ(st.materialized_score_bytes, 0);
            }
        }
    }
}

TEST(Flash, SequenceLengthsAroundTileEdges) {
    if (!Gpu()) SKIP_TEST("no CUDA device");
    uint32_t seed = 41000;
    for (int64_t s : {1, 7, 63, 64, 65, 127, 128, 129, 1024}) {
        for (bool causal : {false, true}) {
            AttnCase c;
            c.causal = causal;
            c.hq = c.hkv = 2;
            c.sq = c.skv = s;
            c.seed = seed++;
            if (!RunCase("flash", sca::flash_attention, c, {})) return;
        }
    }
}

TEST(Flash, GqaWithDifferentLengthsLseAndFp32Rejection) {
    auto dev = Gpu();
    if (!dev) SKIP_TEST("no CUDA device");
    uint32_t seed = 42000;
    for (int64_t group : {1, 2, 4, 8}) {
        AttnCase c;
        c.causal = true;
        c.hkv = 2;
        c.hq = 2 * group;
        c.sq = 96;
        c.skv = 160;
        c.d = 64;
        c.seed = seed++;
        if (!RunCase("flash", sca::flash_attention, c, {})) return;
    }
    AttnCase l;
    l.causal = true;
    l.hq = 4;
    l.hkv = 2;
    l.sq = 100;
    l.skv = 200;
    l.seed = 42100;
    RunCase("flash", sca::flash_attention, l, {}, nullptr, /*check_lse=*/true);
    sci::Tensor q(sci::TensorShape({1, 2, 16, 64}), DType::kFloat32, *dev);
    const auto rejected = sca::flash_attention(q, q, q, {});
    ASSERT_FALSE(rejected.ok());
    EXPECT_EQ(sca::ExtractCode(rejected.error()), sca::AttnStatusCode::kUnsupportedDtype);
    EXPECT_HAS(rejected.error().message(), "naive");
}

// A cudaStreamNonBlocking stream does not synchronise with the legacy default stream. Outputs are allocated (and
// zero-filled) per call and freed when the result goes out of scope, so repeated calls recycle the same pool blocks:
// if allocation, fill or release were ordered on another stream than the kernel, some repetition would read zeros
// or stale data.
TEST(Streams, FlashAndDecodeOnANonBlockingStream) {
    if (!Gpu()) SKIP_TEST("no CUDA device");
    cudaStream_t raw = nullptr;
    ASSERT_TRUE(cudaStreamCreateWithFlags(&raw, cudaStreamNonBlocking) == cudaSuccess);
    sci::Stream stream(raw);
    uint32_t seed = 47000;
    for (int rep = 0; rep < 12; ++rep) {
        sca::AttentionConfig cfg;
        cfg.stream = &stream;
        AttnCase f;
        f.causal = true;
        f.hq = 8;
        f.hkv = 2;
        f.sq = f.skv = 512;
        f.seed = seed++;
        if (!RunCase("flash(non-blocking stream)", sca::flash_attention, f, cfg)) break;
        AttnCase d;
        d.dtype = DType::kBFloat16;
        d.batch = 4;
        d.hq = 8;
        d.hkv = 2;
        d.sq = 1;
        d.skv = 1500;
        d.seed = seed++;
        if (!RunCase("decode(non-blocking stream)", static_cast<Runner>(sca::decode_attention), d, cfg)) break;
    }
    cudaStreamSynchronize(raw);
    cudaStreamDestroy(raw);
}

TEST(Flash, VarlenPackedBatches) {
    auto dev = Gpu();
    if (!dev) SKIP_TEST("no CUDA device");
    const int64_t hq = 4, hkv = 2, d = 64;
    const int32_t cu[] = {0, 37, 37 + 128, 37 + 128 + 5};
    const int64_t total = cu[3];
    const DType dt = DType::kFloat16;
    const Encoded q = Encode(RandomFloats(size_t(total * hq * d), 43000), dt);
    const Encoded k = Encode(RandomFloats(size_t(total * hkv * d), 43001), dt);
    const Encoded v = Encode(RandomFloats(size_t(total * hkv * d), 43002), dt);
    sci::Tensor qt = ToDevice({total, hq, d}, dt, q.bytes, *dev), kt = ToDevice({total, hkv, d}, dt, k.bytes, *dev),
                vt = ToDevice({total, hkv, d}, dt, v.bytes, *dev);
    sca::AttentionConfig cfg;
    cfg.causal = true;
    const auto r = sca::flash_attention_varlen(qt, kt, vt, 3, cu, cu, 128, 128, cfg);
    ASSERT_TRUE(r.ok());
    dev->synchronize();
    const std::vector<float> got = ReadFloats(r->out);
    for (int s = 0; s < 3; ++s) {
        const int64_t n = cu[s + 1] - cu[s];
        // packed [T,H,D] -> [1,H,n,D] for the oracle
        std::vector<float> qs(size_t(hq * n * d)), ks(size_t(hkv * n * d)), vs(size_t(hkv * n * d));
        for (int64_t t = 0; t < n; ++t) {
            for (int64_t h = 0; h < hq; ++h)
                std::copy_n(&q.dequantized[size_t(((cu[s] + t) * hq + h) * d)], d, &qs[size_t((h * n + t) * d)]);
            for (int64_t h = 0; h < hkv; ++h) {
                std::copy_n(&k.dequantized[size_t(((cu[s] + t) * hkv + h) * d)], d, &ks[size_t((h * n + t) * d)]);
                std::copy_n(&v.dequantized[size_t(((cu[s] + t) * hkv + h) * d)], d, &vs[size_t((h * n + t) * d)]);
            }
        }
        std::vector<double> expect(size_t(hq * n * d));
        oracle_attention_f64(qs.data(), ks.data(), vs.data(), 1, hq, hkv, n, n, d, 1, 0.0, expect.data(), nullptr, 4);
        double worst = 0;
        for (int64_t t = 0; t < n; ++t)
            for (int64_t h = 0; h < hq; ++h)
                for (int64_t e = 0; e < d; ++e)
                    worst = std::max(worst, std::fabs(double(got[size_t(((cu[s] + t) * hq + h) * d + e)]) - expect[size_t((h * n + t) * d + e)]));
        EXPECT_LE(worst, 5e-3);
    }
    cfg.return_lse = true;
    EXPECT_FALSE(sca::flash_attention_varlen(qt, kt, vt, 3, cu, cu, 128, 128, cfg).ok());
}

TEST(Decode, SplitCountsLengthsGroupsAndHeadDims) {
    if (!Gpu()) SKIP_TEST("no CUDA device");
    uint32_t seed = 70000;
    for (int64_t splits : {1, 2, 3, 4, 8, 16}) {
        for (int64_t skv : {1, 127, 1024, 4096}) {
            AttnCase c;
            c.causal = true;
            c.sq = 1;
            c.skv = skv;
            c.seed = seed++;
            sca::AttentionConfig cfg;
            cfg.backend = sca::BackendKind::kDecode;
            cfg.num_splits = splits;
            sca::AttentionRuntimeStats st;
            if (!RunCase("decode", sca::decode_attention, c, cfg, &st)) return;
            EXPECT_EQ(st.num_splits, splits);
            EXPECT_GT(st.workspace_bytes, 0u);
        }
    }
    seed = 71000;
    for (int64_t group : {1, 2, 4, 8}) {
        for (int64_t splits : {1, 4, 16}) {
            AttnCase c;
            c.causal = true;
            c.sq = 1;
            c.skv = 2048;
            c.hq = 8 * group;
            c.seed = seed++;
            sca::AttentionConfig cfg;
            cfg.num_splits = splits;
            if (!RunCase("decode", sca::decode_attention, c, cfg)) return;
        }
    }
    seed = 72000;
    for (int64_t d : {32, 64, 96, 128, 160, 192, 256}) {
        AttnCase c;
        c.dtype = DType::kBFloat16;
        c.causal = true;
        c.sq = 1;
        c.skv = 512;
        c.hq = 4;
        c.hkv = 2;
        c.d = d;
        c.seed = seed++;
        sca::AttentionConfig cfg;
        cfg.num_splits = 4;
        if (!RunCase("decode", sca::decode_attention, c, cfg)) return;
    }
}

TEST(Decode, RejectsMultiTokenQueriesAndAutoDispatchPicksIt) {
    auto dev = Gpu();
    if (!dev) SKIP_TEST("no CUDA device");
    sci::Tensor q(sci::TensorShape({1, 2, 4, 64}), DType::kFloat16, *dev), k(sci::TensorShape({1, 2, 64, 64}), DType::kFloat16, *dev);
    sca::AttentionConfig cfg;
    cfg.causal = true;
    const auto r = sca::decode_attention(q, k, k, cfg);
    ASSERT_FALSE(r.ok());
    EXPECT_EQ(sca::ExtractCode(r.error()), sca::AttnStatusCode::kUnsupportedFeature);
    EXPECT_HAS(r.error().message(), "flash");
    // sca::attention with backend=auto: S_q = 1 and S_kv >= 256 -> decode; prefill -> flash; short -> tiled
    AttnCase c;
    c.causal = true;
    c.sq = 1;
    c.skv = 1024;
    c.seed = 73000;
    sca::AttentionRuntimeStats st;
    RunCase("auto", sca::attention, c, {}, &st);
    EXPECT_EQ(int(st.used_backend), int(sca::BackendKind::kDecode));
    c.sq = c.skv = 512;
    RunCase("auto", sca::attention, c, {}, &st);
    EXPECT_EQ(int(st.used_backend), int(sca::BackendKind::kFlash));
    c.sq = c.skv = 64;
    RunCase("auto", sca::attention, c, {}, &st);
    EXPECT_EQ(int(st.used_backend), int(sca::BackendKind::kTiled));
    const std::string why = sca::ExplainAttention(q, k, k, cfg);
    EXPECT_HAS(why, "backend=");
}

TEST(ReferenceBackends, NaiveAndTiledIncludingFp32) {
    if (!Gpu()) SKIP_TEST("no CUDA device");
    uint32_t seed = 74000;
    for (DType dt : {DType::kFloat32, DType::kFloat16, DType::kBFloat16}) {
        for (bool causal : {false, true}) {
            AttnCase c;
            c.dtype = dt;
            c.causal = causal;
            c.hq = 4;
            c.hkv = 2;
            c.sq = 33;
            c.skv = 65;
            c.d = 64;
            c.seed = seed++;
            if (!RunCase("naive", sca::naive_attention, c, {})) return;
            if (!RunCase("tiled", sca::tiled_attention, c, {})) return;
        }
    }
    AttnCase big;
    big.d = 256;
    big.sq = big.skv = 16;
    auto dev = Gpu();
    sci::Tensor q(sci::TensorShape({1, 2, 16, 256}), DType::kFloat16, *dev);
    const auto r = sca::tiled_attention(q, q, q, {});
    ASSERT_FALSE(r.ok());
    EXPECT_EQ(sca::ExtractCode(r.error()), sca::AttnStatusCode::kDeviceCapability);
}

TEST(Numerics, LogitMagnitudesAndDegenerateRows) {
    if (!Gpu()) SKIP_TEST("no CUDA device");
    uint32_t seed = 75000;
    for (float mag : {0.0f, 1.0f, 10.0f, 100.0f}) {
        AttnCase c;
        c.dtype = DType::kFloat16;
        c.hq = c.hkv = 2;
        c.sq = c.skv = 256;
        c.magnitude = mag;
        c.seed = seed++;
        if (!RunCase("flash", sca::flash_attention, c, {})) return;
    }
    AttnCase one;   // S_q = 1 under the causal mask through flash and through decode
    one.causal = true;
    one.sq = 1;
    one.skv = 700;
    one.hq = 4;
    one.hkv = 2;
    one.seed = seed++;
    RunCase("flash", sca::flash_attention, one, {});
    RunCase("decode", sca::decode_attention, one, {});
    AttnCase wide;  // long keys, short queries
    wide.causal = true;
    wide.sq = 512;
    wide.skv = 8192;
    wide.hq = wide.hkv = 1;
    wide.seed = seed++;
    RunCase("flash", sca::flash_attention, wide, {});
}

TEST(KvCacheDevice, AppendGatherResetRoundTripAndOverBudget) {
    auto dev = Gpu();
    if (!dev) SKIP_TEST("no CUDA device");
    for (int64_t bs : {1, 8, 16, 32, 64}) {
        sca::KVCacheConfig cfg;
        cfg.num_layers = 1;
        cfg.num_kv_heads = 2;
        cfg.head_dim = 64;
        cfg.block_size = bs;
        cfg.num_blocks = 8;
        cfg.max_num_seqs = 4;
        const auto cache = sca::KVCache::Create(cfg, *dev);
        ASSERT_TRUE(cache.ok());
        EXPECT_EQ(cache->MemoryBytes(), size_t(2ull * 1 * 8 * bs * 2 * 64 * 2));
        EXPECT_EQ(cache->K(0).dim(1), bs);
    }
    sca::KVCacheConfig cfg;
    cfg.num_layers = 1;
    cfg.num_kv_heads = 2;
    cfg.head_dim = 32;
    cfg.block_size = 8;
    cfg.num_blocks = 4;
    cfg.max_num_seqs = 4;
    auto created = sca::KVCache::Create(cfg, *dev);
    ASSERT_TRUE(created.ok());
    sca::KVCache cache = std::move(*created);
    std::vector<float> kv(size_t(3 * 2 * 32)), vv(kv.size());
    for (size_t i = 0; i < kv.size(); ++i) {
        kv[i] = 10.0f + float(i);
        vv[i] = -1.0f - float(i);
    }
    const Encoded ke = Encode(kv, cfg.dtype), ve = Encode(vv, cfg.dtype);
    sci::Tensor k = ToDevice({3, 2, 32}, cfg.dtype, ke.bytes, *dev), v = ToDevice({3, 2, 32}, cfg.dtype, ve.bytes, *dev);
    sci::Tensor slots = ToDeviceI32({0, 9, 17}, *dev);
    ASSERT_TRUE(cache.Append(0, k, v, static_cast<const int32_t*>(slots.data()), 3, nullptr).ok());
    EXPECT_EQ(cache.Stats().num_appends, 1);
    sci::Tensor ids = ToDeviceI32({1, 0}, *dev);
    const auto g = cache.GatherK(0, static_cast<const int32_t*>(ids.data()), 2, nullptr);
    ASSERT_TRUE(g.ok());
    dev->synchronize();
    const std::vector<float> got = ReadFloats(*g);
    const size_t row = 2 * 32;
    EXPECT_EQ(got[0], 0.0f);
    EXPECT_NEAR(got[1 * row], ke.dequantized[row], 1e-3);
    EXPECT_NEAR(got[8 * row], ke.dequantized[0], 1e-3);
    sci::Tensor reset_ids = ToDeviceI32({2}, *dev);
    ASSERT_TRUE(cache.Reset(static_cast<const int32_t*>(reset_ids.data()), 1, nullptr).ok());
    sci::Tensor check = ToDeviceI32({2, 0}, *dev);
    const auto after = cache.GatherK(0, static_cast<const int32_t*>(check.data()), 2, nullptr);
    ASSERT_TRUE(after.ok());
    dev->synchronize();
    const std::vector<float> a = ReadFloats(*after);
    EXPECT_EQ(a[1 * row], 0.0f);
    EXPECT_NEAR(a[8 * row], ke.dequantized[0], 1e-3);
    EXPECT_EQ(cache.Stats().num_resets, 1);

    sca::KVCacheConfig huge = cfg;
    huge.num_layers = 32;
    huge.num_kv_heads = 8;
    huge.head_dim = 128;
    huge.block_size = 16;
    huge.num_blocks = 1000000;
    const auto refused = sca::KVCache::Create(huge, *dev);
    ASSERT_FALSE(refused.ok());
    EXPECT_EQ(sca::ExtractCode(refused.error()), sca::AttnStatusCode::kKVCapacityExceeded);
    EXPECT_HAS(refused.error().message(), "num_blocks <=");
}

TEST(PagedKv, IsolationExhaustionResetAndAttention) {
    auto dev = Gpu();
    if (!dev) SKIP_TEST("no CUDA device");
    sca::KVCacheConfig cfg;
    cfg.num_layers = 1;
    cfg.num_kv_heads = 1;
    cfg.head_dim = 32;
    cfg.block_size = 8;
    cfg.num_blocks = 8;
    cfg.max_num_seqs = 2;
    auto created = sca::PagedKVCache::Create(cfg, *dev);
    ASSERT_TRUE(created.ok());
    sca::PagedKVCache cache = std::move(*created);
    auto tokens = [&](int64_t n, float base) {
        std::vector<float> vals(size_t(n * 32));
        for (size_t i = 0; i < vals.size(); ++i) vals[i] = base + 0.01f * float(i);
        return ToDevice({n, 1, 32}, cfg.dtype, Encode(vals, cfg.dtype).bytes, *dev);
    };
    sci::Tensor a3 = tokens(3, 1.0f), b3 = tokens(3, 100.0f), a6 = tokens(6, 2.0f);
    ASSERT_TRUE(cache.AppendTokens(0, 0, a3, a3, nullptr).ok());
    ASSERT_TRUE(cache.AppendTokens(1, 0, b3, b3, nullptr).ok());
    ASSERT_TRUE(cache.AppendTokens(0, 0, a6, a6, nullptr).ok());
    EXPECT_EQ(cache.SeqLength(0), 9);
    EXPECT_EQ(cache.SeqLength(1), 3);
    EXPECT_EQ(cache.LogicalBlockCount(0), 2);
    EXPECT_EQ(cache.Stats().used_blocks, 3);
    EXPECT_EQ(cache.Stats().free_blocks, 5);
    EXPECT_EQ(cache.Stats().num_appends, 3);
    sci::Tensor big = tokens(48, 5.0f);
    const sci::Status overflow = cache.AppendTokens(1, 0, big, big, nullptr);
    ASSERT_FALSE(overflow.ok());
    EXPECT_EQ(sca::ExtractCode(overflow), sca::AttnStatusCode::kKVCapacityExceeded);
    EXPECT_EQ(cache.SeqLength(1), 3);
    EXPECT_EQ(cache.Stats().free_blocks, 5);
    ASSERT_TRUE(cache.SyncPageTable(nullptr).ok());
    // attention over both sequences with the cache's own table
    sci::Tensor q = ToDevice({2, 2, 1, 32}, cfg.dtype, Encode(RandomFloats(2 * 2 * 32, 9), cfg.dtype).bytes, *dev);
    sca::PagedAttentionParams params;
    params.page_table = cache.PageTableDevicePtr();
    params.seq_lens = cache.SeqLensDevicePtr();
    params.num_seqs = 2;
    params.block_size = cache.BlockSize();
    params.max_blocks_per_seq = cache.MaxBlocksPerSeq();
    const auto out = sca::paged_attention(q, cache, params, {});
    ASSERT_TRUE(out.ok());
    EXPECT_EQ(int(out->stats.used_backend), int(sca::BackendKind::kPaged));
    EXPECT_GT(out->stats.kv_bytes, 0u);
    ASSERT_TRUE(cache.ResetSeq(0, nullptr).ok());
    EXPECT_EQ(cache.SeqLength(0), 0);
    EXPECT_EQ(cache.Stats().free_blocks, 7);
    EXPECT_EQ(cache.Stats().num_resets, 1);
    ASSERT_TRUE(cache.AppendTokens(0, 0, a3, a3, nullptr).ok());
    EXPECT_EQ(cache.Stats().free_blocks, 6);
    sci::Tensor wrong(sci::TensorShape({2, 2, 4, 32}), cfg.dtype, *dev);
    EXPECT_FALSE(sca::paged_attention(wrong, cache, params, {}).ok());
}

// The short form sca::paged_attention(q, kv, cfg) takes table and lengths from the cache. With a length that is not
// a multiple of block_size the zero-filled rest of the last block must carry no weight: the result equals the
// explicit form with the cache's lengths.
TEST(PagedKv, ShortFormUsesTheCachesOwnLengths) {
    auto dev = Gpu();
    if (!dev) SKIP_TEST("no CUDA device");
    sca::KVCacheConfig cfg;
    cfg.num_layers = 1;
    cfg.num_kv_heads = 1;
    cfg.head_dim = 32;
    cfg.block_size = 8;
    cfg.num_blocks = 8;
    cfg.max_num_seqs = 2;
    auto created = sca::PagedKVCache::Create(cfg, *dev);
    ASSERT_TRUE(created.ok());
    sca::PagedKVCache cache = std::move(*created);
    auto tokens = [&](int64_t n, uint32_t seed) {
        return ToDevice({n, 1, 32}, cfg.dtype, Encode(RandomFloats(size_t(n * 32), seed, 0.5f, 2.0f), cfg.dtype).bytes, *dev);
    };
    sci::Tensor t11 = tokens(11, 31), t5 = tokens(5, 32);
    ASSERT_TRUE(cache.AppendTokens(0, 0, t11, t11, nullptr).ok());
    ASSERT_TRUE(cache.AppendTokens(1, 0, t5, t5, nullptr).ok());
    ASSERT_TRUE(cache.SyncPageTable(nullptr).ok());
    sci::Tensor q = ToDevice({2, 2, 1, 32}, cfg.dtype, Encode(RandomFloats(2 * 2 * 32, 33), cfg.dtype).bytes, *dev);
    sca::PagedAttentionParams params;
    params.seq_lens = cache.SeqLensDevicePtr();
    params.num_seqs = 2;
    params.block_size = cache.BlockSize();  // the struct's default is 16, as in the reference
    const auto explicit_form = sca::paged_attention(q, cache, params, {});
    const auto short_form = sca::paged_attention(q, cache, sca::AttentionConfig{});
    ASSERT_TRUE(explicit_form.ok());
    ASSERT_TRUE(short_form.ok());
    dev->synchronize();
    const std::vector<float> a = ReadFloats(explicit_form->out), b = ReadFloats(short_form->out);
    ASSERT_EQ(a.size(), b.size());
    for (size_t i = 0; i < a.size(); ++i) EXPECT_EQ(a[i], b[i]);
    // all values are >= 0.5, so an output row is >= 0.5 too unless zero rows were averaged in
    for (float x : b) EXPECT_GE(x, 0.49f);
}

TEST(PagedKv, LaunchOrderIsLongestFirstAndOnlyOfferedWhenItIsAPermutation) {
    auto dev = Gpu();
    if (!dev) SKIP_TEST("no CUDA device");
    sca::KVCacheConfig cfg;
    cfg.num_layers = 1;
    cfg.num_kv_heads = 1;
    cfg.head_dim = 32;
    cfg.block_size = 8;
    cfg.num_blocks = 16;
    cfg.max_num_seqs = 4;
    auto created = sca::PagedKVCache::Create(cfg, *dev);
    ASSERT_TRUE(created.ok());
    sca::PagedKVCache cache = std::move(*created);
    EXPECT_TRUE(cache.SeqOrderDevicePtr(4) == nullptr);  // nothing synced yet
    auto tokens = [&](int64_t n) {
        return ToDevice({n, 1, 32}, cfg.dtype, Encode(RandomFloats(size_t(n * 32), 21), cfg.dtype).bytes, *dev);
    };
    sci::Tensor t3 = tokens(3), t17 = tokens(17), t9 = tokens(9);
    ASSERT_TRUE(cache.AppendTokens(0, 0, t3, t3, nullptr).ok());
    ASSERT_TRUE(cache.AppendTokens(1, 0, t17, t17, nullptr).ok());
    ASSERT_TRUE(cache.AppendTokens(2, 0, t9, t9, nullptr).ok());
    ASSERT_TRUE(cache.SyncPageTable(nullptr).ok());
    const int32_t* order_dev = cache.SeqOrderDevicePtr(4);
    ASSERT_TRUE(order_dev != nullptr);
    int32_t order[4] = {-1, -1, -1, -1};
    dev->copy_to_host(order, order_dev, sizeof(order));
    EXPECT_EQ(order[0], 1);
    EXPECT_EQ(order[1], 2);
    EXPECT_EQ(order[2], 0);
    EXPECT_EQ(order[3], 3);
    EXPECT_TRUE(cache.SeqOrderDevicePtr(3) == order_dev);  // slot 3 is empty: the first three entries permute [0, 3)
    EXPECT_TRUE(cache.SeqOrderDevicePtr(2) == nullptr);   // slot 2 is live: no permutation of [0, 2) in there
    EXPECT_TRUE(cache.SeqOrderDevicePtr(5) == nullptr);
    // the order is a scheduling hint: attention over three sequences equals attention over each one alone
    const std::vector<float> qvals = RandomFloats(3 * 2 * 32, 5);
    sci::Tensor q = ToDevice({3, 2, 1, 32}, cfg.dtype, Encode(qvals, cfg.dtype).bytes, *dev);
    sci::Tensor q0 = ToDevice({1, 2, 1, 32}, cfg.dtype,
                              Encode(std::vector<float>(qvals.begin(), qvals.begin() + 2 * 32), cfg.dtype).bytes, *dev);
    sca::PagedAttentionParams params;
    params.seq_lens = cache.SeqLensDevicePtr();
    params.num_seqs = 3;
    params.block_size = cache.BlockSize();
    const auto all = sca::paged_attention(q, cache, params, {});
    ASSERT_TRUE(all.ok());
    const std::vector<float> got = ReadFloats(all->out);
    ASSERT_TRUE(cache.ResetSeq(1, nullptr).ok());
    ASSERT_TRUE(cache.ResetSeq(2, nullptr).ok());
    ASSERT_TRUE(cache.SyncPageTable(nullptr).ok());
    params.num_seqs = 1;
    const auto first = sca::paged_attention(q0, cache, params, {});  // q row 0 against sequence 0 alone
    ASSERT_TRUE(first.ok());
    const std::vector<float> alone = ReadFloats(first->out);
    ASSERT_EQ(alone.size(), size_t(2 * 32));
    for (size_t i = 0; i < alone.size(); ++i) EXPECT_TRUE(std::fabs(got[i] - alone[i]) <= 1e-3f);
}

int main(int argc, char** argv) { return mini::RunAll(argc, argv); }
