// Support services on every call path: cached device capability, the grow-only scratch pool, the
// Workspace slice allocator, and the glue between the C ABI's integer codes and sci::Status.
// Behaviour follows src/runtime/capability.cpp, scratch_pool.cpp and workspace.cpp of the reference.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <utility>

#include "device/stream.hpp"
#include "internal.hpp"

namespace sca {
namespace runtime {

sci::Status FromAbi(int rc) {
    if (rc == 0) return sci::Status::Ok();
    return sci::Status(static_cast<sci::StatusCode>(rc), sca_last_error());
}

void* StreamHandle(sci::Stream* stream) {
    return stream != nullptr ? stream->handle() : sci::Stream::GetCurrent().handle();
}

// ---- scratch pool -----------------------------------------------------------------------------------------
namespace {
struct ScratchEntry {
    sci::Tensor buffer;
    size_t elements{0};
};
std::mutex& ScratchMutex() {
    static std::mutex m;
    return m;
}
// Leaked on purpose: freeing device memory from a static destructor runs after the CUDA runtime is gone.
std::unordered_map<int, ScratchEntry>& ScratchMap() {
    static auto* map = new std::unordered_map<int, ScratchEntry>();
    return *map;
}
size_t g_scratch_peak_bytes = 0;
}  // namespace

sci::Result<float*> AcquireScratchFp32(ScratchKind kind, size_t elements, sci::Device& device) {
    if (elements == 0) {
        return sci::MakeUnexpected<float*>(MakeStatus(AttnStatusCode::kWorkspaceExceeded, "scratch request with 0 elements"));
    }
    std::lock_guard<std::mutex> lock(ScratchMutex());
    ScratchEntry& entry = ScratchMap()[device.id() * 16 + static_cast<int>(kind)];
    if (entry.buffer.data() == nullptr || entry.elements < elements) {
        const size_t grown = static_cast<size_t>(static_cast<double>(elements) * 1.25) + 1024;
        entry.buffer = sci::Tensor(sci::TensorShape({static_cast<sci::index_t>(grown)}), sci::DType::kFloat32, device);
        if (entry.buffer.data() == nullptr) {
            entry.elements = 0;
            return sci::MakeUnexpected<float*>(MakeStatus(
                AttnStatusCode::kWorkspaceExceeded, "scratch allocation of " + std::to_string(grown * sizeof(float)) + " B failed"));
        }
        entry.elements = grown;
        g_scratch_peak_bytes = std::max(g_scratch_peak_bytes, grown * sizeof(float));
    }
    return sci::Ok(static_cast<float*>(entry.buffer.data()));
}

sci::Status ReleaseScratch() {
    std::lock_guard<std::mutex> lock(ScratchMutex());
    ScratchMap().clear();
    return sci::Status::Ok();
}

size_t ScratchHighWaterMarkBytes() {
    std::lock_guard<std::mutex> lock(ScratchMutex());
    return g_scratch_peak_bytes;
}

}  // namespace runtime

// ---- device capability ----------------------------------------------------------------------------------------
namespace {

std::mutex& CapMutex() {
    static std::mutex m;
    return m;
}
std::unordered_map<int, DeviceCapability>& CapCache() {
    static auto* cache = new std::unordered_map<int, DeviceCapability>();
    return *cache;
}
// CudaAvailable() is asked on every Supports() / Forward(); the answer cannot change while the process
// lives, so it is probed once (the reference re-probes the device on every call).
int g_cuda_available = -1;

DeviceCapability ProbeDevice(int device_id) {
    DeviceCapability cap;
    ScaDeviceProbeB200 ext{};
    if (sca_probe_device_b200(device_id, &ext) != 0 || ext.base.cuda_available == 0) {
        cap.device_name = "cuda-unavailable";
        return cap;
    }
    const ScaDeviceProbe& raw = ext.base;
    cap.device_name = raw.name;
    cap.major = raw.major;
    cap.minor = raw.minor;
    cap.sm_count = raw.sm_count;
    cap.smem_per_sm = raw.smem_per_sm;
    cap.smem_per_block_default = raw.smem_per_block_default;
    cap.smem_per_block_optin = raw.smem_per_block_optin;
    cap.regs_per_sm = raw.regs_per_sm;
    cap.max_threads_per_sm = raw.max_threads_per_sm;
    cap.l2_bytes = raw.l2_bytes;
    cap.total_mem_bytes = raw.total_mem_bytes;
    cap.free_mem_bytes = raw.free_mem_bytes;
    const int cc = cap.major * 10 + cap.minor;
    cap.has_mma_m16n8k16 = cc >= 80 && raw.binary_has_sm80 != 0;
    cap.has_cp_async = cc >= 80 && raw.binary_has_sm80 != 0;
    cap.has_tma_bulk = cc >= 90 && raw.binary_has_sm90 != 0;
    cap.has_wgmma = false;
    cap.has_fp8_mma = false;
    cap.has_tcgen05 = cap.major == 10 && ext.binary_has_sm100a != 0;
    cap.tmem_columns = ext.tmem_columns;
    cap.max_cluster_size = ext.max_cluster_size;
    return cap;
}

}  // namespace

const DeviceCapability& DeviceCapability::ForDevice(int device_id) {
    std::lock_guard<std::mutex> lock(CapMutex());
    auto& cache = CapCache();
    auto it = cache.find(device_id);
    if (it == cache.end()) it = cache.emplace(device_id, ProbeDevice(device_id)).first;
    return it->second;
}

sci::Status DeviceCapability::Refresh(int device_id) {
    DeviceCapability fresh = ProbeDevice(device_id);
    std::lock_guard<std::mutex> lock(CapMutex());
    CapCache()[device_id] = std::move(fresh);
    g_cuda_available = -1;
    return sci::Status::Ok();
}

size_t DeviceCapability::SmemLimitPerBlock(const DeviceCapability& cap) noexcept {
    size_t limit = cap.smem_per_block_optin != 0 ? cap.smem_per_block_optin : cap.smem_per_block_default;
    if (const char* env = std::getenv("SCI_ATTENTION_MAX_SMEM_BYTES")) {
        const long long parsed = std::strtoll(env, nullptr, 10);
        if (parsed > 0 && static_cast<size_t>(parsed) < limit) limit = static_cast<size_t>(parsed);
    }
    if (cap.smem_per_sm != 0 && limit > cap.smem_per_sm) limit = cap.smem_per_sm;
    return limit;
}

bool DeviceCapability::CudaAvailable() noexcept {
    std::lock_guard<std::mutex> lock(CapMutex());
    if (g_cuda_available < 0) {
        ScaDeviceProbe raw{};
        g_cuda_available = (sca_probe_device(0, &raw) == 0 && raw.cuda_available != 0) ? 1 : 0;
    }
    return g_cuda_available == 1;
}

// ---- workspace ----------------------------------------------------------------------------------------------------
struct Workspace::Impl {
    sci::Tensor buffer;
    size_t bytes{0};
    size_t peak{0};
    std::vector<std::pair<size_t, size_t>> spans;  // [begin, end)
};

Workspace::Workspace() : impl_(std::make_shared<Impl>()) {}
Workspace::~Workspace() = default;

sci::Result<Workspace> Workspace::Create(size_t bytes, sci::Device& device) {
    if (bytes == 0) return sci::MakeUnexpected<Workspace>(MakeStatus(AttnStatusCode::kWorkspaceExceeded, "workspace bytes=0"));
    Workspace ws;
    ws.impl_->buffer = sci::Tensor(sci::TensorShape({static_cast<sci::index_t>(bytes)}), sci::DType::kUInt8, device);
    if (ws.impl_->buffer.data() == nullptr) {
        return sci::MakeUnexpected<Workspace>(
            MakeStatus(AttnStatusCode::kWorkspaceExceeded, "allocation of " + std::to_string(bytes) + " B failed"));
    }
    ws.impl_->bytes = bytes;
    return sci::Ok(std::move(ws));
}

void* Workspace::Data() noexcept { return impl_->buffer.data(); }
const void* Workspace::Data() const noexcept { return impl_->buffer.data(); }
size_t Workspace::Bytes() const noexcept { return impl_->bytes; }
bool Workspace::Valid() const noexcept { return impl_ != nullptr && impl_->buffer.data() != nullptr; }
size_t Workspace::PeakBytes() const noexcept { return impl_->peak; }
size_t Workspace::AllocatedSlices() const noexcept { return impl_->spans.size(); }

sci::Result<void*> Workspace::Slice(size_t offset, size_t bytes, size_t align) {
    auto refuse = [](const std::string& text) {
        return sci::MakeUnexpected<void*>(MakeStatus(AttnStatusCode::kWorkspaceExceeded, text));
    };
    if (!Valid()) return refuse("workspace is not initialised");
    if (bytes == 0) return refuse("slice bytes=0");
    if (align == 0 || offset % align != 0) {
        return refuse("slice offset=" + std::to_string(offset) + " is not " + std::to_string(align) + " B aligned");
    }
    if (offset > impl_->bytes || bytes > impl_->bytes - offset) {
        return refuse("slice [" + std::to_string(offset) + ", " + std::to_string(offset + bytes) +
                      ") exceeds workspace bytes=" + std::to_string(impl_->bytes));
    }
    const size_t begin = offset, end = offset + bytes;
    bool same = false, clash = false;
    for (const auto& span : impl_->spans) {
        if (span.first == begin && span.second == end) same = true;
        else if (begin < span.second && span.first < end) clash = true;
    }
    if (clash && !same) {
        return refuse("slice [" + std::to_string(begin) + ", " + std::to_string(end) +
                      ") partially overlaps an existing slice (either reuse it exactly or Reset())");
    }
    if (!same) impl_->spans.emplace_back(begin, end);
    impl_->peak = std::max(impl_->peak, end);
    return sci::Ok(static_cast<void*>(static_cast<unsigned char*>(impl_->buffer.data()) + offset));
}

sci::Status Workspace::Reset() {
    if (!Valid()) return MakeStatus(AttnStatusCode::kWorkspaceExceeded, "workspace is not initialised");
    impl_->spans.clear();
    return sci::Status::Ok();
}

}  // namespace sca

// ---- NVTX ranges around the public entry points ----------------------------------------------------------
#include <nvtx3/nvToolsExt.h>

namespace sca {
namespace {
nvtxDomainHandle_t ApiDomain() {
    static nvtxDomainHandle_t domain = nvtxDomainCreateA("sci_attention");
    return domain;
}
}  // namespace

ApiRange::ApiRange(const char* name) {
    nvtxEventAttributes_t attr{};
    attr.version = NVTX_VERSION;
    attr.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
    attr.messageType = NVTX_MESSAGE_TYPE_ASCII;
    attr.message.ascii = name;
    nvtxDomainRangePushEx(ApiDomain(), &attr);
}
ApiRange::~ApiRange() { nvtxDomainRangePop(ApiDomain()); }
}  // namespace sca
