// API-level latency benchmark of the public C++ entry points, with the record format of the reference's
// benchmark suite (benchmarks/common/bench_utils.hpp:103-135 CaseResult / RunHeader, :261-330 JSON and CSV writers;
// protocol of docs/benchmarking.md: 20 warm-up calls, 100 timed calls, mean / median / std / P50 / P90 / P95 / P99).
//
// What is timed is ONE CALL of the public API - sca::flash_attention, sca::decode_attention, sca::paged_attention -
// between two CUDA events on the call's stream: shape inference, validation, the allocation of the freshly returned
// output tensor, scratch acquisition and the kernels. That is the number a caller of the library sees; the kernel-only
// number (output pre-allocated, C ABI called directly) is what bench.py reports, and the two should differ by a few
// per cent at most.
//
// FLOPs are counted for the pairs the mask leaves visible: causal rows see S_kv - S_q + i + 1 keys, i.e.
// 4 * B * H_q * D * (S_q * (S_kv - S_q) + S_q (S_q + 1) / 2). (The reference's own causal path multiplies the pair
// count by B * H_q a second time, benchmarks/common/bench_utils.hpp; that is not reproduced here.)
//
//   bench_attention [--runs N] [--warmup W] [--out-dir DIR] [--small]
// --small runs reduced shapes (a smoke test of the tool itself). Exit codes: 0 ok, 2 no GPU, 4 a call failed.
#include <cuda_runtime_api.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <fstream>
#include <functional>
#include <numeric>
#include <string>
#include <vector>

#include "device/cuda_device.hpp"
#include "scicompute_attention/attention.hpp"
#include "scicompute_attention/paged_attention.hpp"
#include "scicompute_attention/paged_kv_cache.hpp"

namespace {

struct Latency {
    double mean{0}, median{0}, stddev{0}, p50{0}, p90{0}, p95{0}, p99{0};
};

struct Record {
    std::string case_id, impl, params_json, note;
    Latency ms;
    double flops_effective{0}, tflops{0}, effective_bw_gbps{0}, workspace_mb{0};
    int64_t bytes_moved_modeled{0};
};

Latency Summarise(std::vector<float> v) {
    Latency l;
    if (v.empty()) return l;
    std::sort(v.begin(), v.end());
    auto pct = [&](double p) {
        const double pos = p * (v.size() - 1);
        const size_t lo = static_cast<size_t>(pos);
        const size_t hi = std::min(lo + 1, v.size() - 1);
        return v[lo] + (v[hi] - v[lo]) * (pos - lo);
    };
    l.mean = std::accumulate(v.begin(), v.end(), 0.0) / v.size();
    double var = 0;
    for (float x : v) var += (x - l.mean) * (x - l.mean);
    l.stddev = std::sqrt(var / v.size());
    l.median = l.p50 = pct(0.50);
    l.p90 = pct(0.90);
    l.p95 = pct(0.95);
    l.p99 = pct(0.99);
    return l;
}

// Device fp16 / bf16 tensor with a seeded pattern in [-1, 1] (bit patterns built on the host).
sci::Tensor Filled(std::initializer_list<int64_t> dims, sci::DType dtype, sci::Device& dev, uint32_t seed) {
    sci::Tensor t(sci::TensorShape(dims), dtype, dev);
    std::vector<uint16_t> host(static_cast<size_t>(t.num_elements()));
    uint32_t s = seed * 2654435761u + 12345u;
    for (uint16_t& h : host) {
        s = s * 1664525u + 1013904223u;
        const float f = static_cast<float>(s >> 8) * (2.0f / 16777216.0f) - 1.0f;
        uint32_t bits;
        std::memcpy(&bits, &f, 4);
        if (dtype == sci::DType::kBFloat16) {
            h = static_cast<uint16_t>((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
        } else {
            const uint32_t sign = (bits >> 16) & 0x8000u;
            const int32_t exp = static_cast<int32_t>((bits >> 23) & 0xff) - 127 + 15;
            h = exp <= 0 ? static_cast<uint16_t>(sign)
                         : static_cast<uint16_t>(sign | (static_cast<uint32_t>(exp) << 10) | ((bits & 0x7fffffu) >> 13));
        }
    }
    t.copy_from(host.data(), host.size() * sizeof(uint16_t));
    return t;
}

struct Runner {
    int warmup{20}, runs{100};
    cudaEvent_t start{}, stop{};
    // Times `call` (one public API call; returns false on failure). The result tensor of every call is dropped at the
    // end of the call's scope, as a caller that consumes the output would.
    bool Time(const std::function<bool()>& call, Latency* out) {
        for (int i = 0; i < warmup; ++i) {
            if (!call()) return false;
        }
        cudaDeviceSynchronize();
        std::vector<float> ms(static_cast<size_t>(runs));
        for (int i = 0; i < runs; ++i) {
            cudaEventRecord(start, nullptr);
            if (!call()) return false;
            cudaEventRecord(stop, nullptr);
            cudaEventSynchronize(stop);
            cudaEventElapsedTime(&ms[static_cast<size_t>(i)], start, stop);
        }
        *out = Summarise(ms);
        return true;
    }
};

std::string Escape(const std::string& s) {
    std::string o;
    for (char c : s) {
        if (c == '"' || c == '\\') o += '\\';
        o += c;
    }
    return o;
}

void WriteJson(const std::string& path, const std::string& gpu, const std::string& cc, int warmup, int runs,
               const std::vector<Record>& cases) {
    std::ofstream out(path);
    if (!out) return;
    char stamp[64];
    const std::time_t now = std::time(nullptr);
    std::strftime(stamp, sizeof(stamp), "%Y-%m-%dT%H:%M:%SZ", std::gmtime(&now));
    int driver = 0, runtime = 0;
    cudaDriverGetVersion(&driver);
    cudaRuntimeGetVersion(&runtime);
    out.setf(std::ios::fixed);
    out.precision(6);
    out << "{\n  \"benchmark_name\": \"bench_attention (public API, per call)\",\n  \"git_sha\": \"\",\n"
        << "  \"build_type\": \"Release\",\n  \"gpu\": \"" << Escape(gpu) << "\",\n  \"compute_cap\": \"" << cc << "\",\n"
        << "  \"driver\": \"" << driver << "\",\n  \"cuda\": \"" << runtime << "\",\n  \"sm_clock_mhz\": 0,\n"
        << "  \"timestamp\": \"" << stamp << "\",\n  \"warmup\": " << warmup << ",\n  \"runs\": " << runs
        << ",\n  \"seed\": 1234,\n  \"cases\": [\n";
    for (size_t i = 0; i < cases.size(); ++i) {
        const Record& c = cases[i];
        out << "    {\n      \"case_id\": \"" << Escape(c.case_id) << "\",\n      \"impl\": \"" << Escape(c.impl) << "\",\n"
            << "      \"params\": " << c.params_json << ",\n"
            << "      \"latency_ms\": {\"mean\": " << c.ms.mean << ", \"median\": " << c.ms.median << ", \"std\": " << c.ms.stddev
            << ", \"p50\": " << c.ms.p50 << ", \"p90\": " << c.ms.p90 << ", \"p95\": " << c.ms.p95 << ", \"p99\": " << c.ms.p99 << "},\n"
            << "      \"flops_effective\": " << c.flops_effective << ",\n      \"tflops\": " << c.tflops << ",\n"
            << "      \"bytes_moved_modeled\": " << c.bytes_moved_modeled << ",\n      \"effective_bw_gbps\": " << c.effective_bw_gbps << ",\n"
            << "      \"peak_mem_mb\": 0.000000,\n      \"workspace_mb\": " << c.workspace_mb << ",\n"
            << "      \"registers_per_thread\": -1,\n      \"smem_bytes\": 0,\n      \"achieved_occupancy_pct\": -1.000000,\n"
            << "      \"reference_max_abs_err\": -1.000000,\n      \"note\": \"" << Escape(c.note) << "\"\n    }"
            << (i + 1 == cases.size() ? "" : ",") << "\n";
    }
    out << "  ]\n}\n";
    std::printf("[bench] json written: %s\n", path.c_str());
}

void WriteCsv(const std::string& path, int warmup, int runs, const std::vector<Record>& cases) {
    std::ofstream out(path);
    if (!out) return;
    out << "name,case_id,warmup,runs,mean_ms,median_ms,std_ms,p50_ms,p90_ms,p95_ms,p99_ms,tflops,effective_bw_gbps,peak_mem_mb,unit\n";
    out.setf(std::ios::fixed);
    out.precision(6);
    for (const Record& c : cases) {
        out << c.impl << "," << c.case_id << "," << warmup << "," << runs << "," << c.ms.mean << "," << c.ms.median << ","
            << c.ms.stddev << "," << c.ms.p50 << "," << c.ms.p90 << "," << c.ms.p95 << "," << c.ms.p99 << "," << c.tflops << ","
            << c.effective_bw_gbps << ",0.000000,ms\n";
    }
    std::printf("[bench] csv written: %s\n", path.c_str());
}

std::string Params(int64_t b, int64_t hq, int64_t hkv, int64_t sq, int64_t skv, int64_t d, const char* dtype, bool causal) {
    char buf[256];
    std::snprintf(buf, sizeof(buf), "{\"B\":%lld,\"H\":%lld,\"H_kv\":%lld,\"S_q\":%lld,\"S_kv\":%lld,\"D\":%lld,\"dtype\":\"%s\",\"causal\":%s}",
                  static_cast<long long>(b), static_cast<long long>(hq), static_cast<long long>(hkv), static_cast<long long>(sq),
                  static_cast<long long>(skv), static_cast<long long>(d), dtype, causal ? "true" : "false");
    return buf;
}

}  // namespace

int main(int argc, char** argv) {
    Runner run;
    std::string out_dir = ".";
    bool small = false;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--runs" && i + 1 < argc) run.runs = std::max(1, std::atoi(argv[++i]));
        else if (a == "--warmup" && i + 1 < argc) run.warmup = std::max(0, std::atoi(argv[++i]));
        else if (a == "--out-dir" && i + 1 < argc) out_dir = argv[++i];
        else if (a == "--small") small = true;
        else {
            std::fprintf(stderr, "bad argument: %s\n", a.c_str());
            return 1;
        }
    }
    std::shared_ptr<sci::Device> device = sci::DeviceManager::Instance().get_device(sci::DeviceType::kCUDA, 0);
    if (device == nullptr) {
        std::printf("[bench] no CUDA device\n");
        return 2;
    }
    cudaEventCreate(&run.start);
    cudaEventCreate(&run.stop);
    const sca::DeviceCapability& cap = sca::DeviceCapability::ForDevice(0);
    std::vector<Record> cases;
    const int64_t hq = 32, hkv = 8, d = 128;

    // ---- prefill (config C2: B=4, S=4096, causal), fp16 and bf16 ------------------------------------------
    for (sci::DType dtype : {sci::DType::kBFloat16, sci::DType::kFloat16}) {
        const int64_t b = small ? 1 : 4, s = small ? 512 : 4096;
        sci::Tensor q = Filled({b, hq, s, d}, dtype, *device, 1), k = Filled({b, hkv, s, d}, dtype, *device, 2),
                    v = Filled({b, hkv, s, d}, dtype, *device, 3);
        sca::AttentionConfig cfg;
        cfg.backend = sca::BackendKind::kFlash;
        cfg.causal = true;
        Record r;
        r.impl = "sca::flash_attention";
        r.case_id = std::string("prefill_causal_B") + std::to_string(b) + "_S" + std::to_string(s) + (dtype == sci::DType::kBFloat16 ? "_bf16" : "_fp16");
        r.params_json = Params(b, hq, hkv, s, s, d, dtype == sci::DType::kBFloat16 ? "bf16" : "fp16", true);
        if (!run.Time([&] { return sca::flash_attention(q, k, v, cfg).ok(); }, &r.ms)) return 4;
        r.flops_effective = 4.0 * b * hq * d * (static_cast<double>(s) * (s + 1) / 2.0);
        r.tflops = r.flops_effective / (r.ms.p50 * 1e-3) / 1e12;
        r.bytes_moved_modeled = (2 * b * hq + 2 * b * hkv) * s * d * 2;
        r.effective_bw_gbps = static_cast<double>(r.bytes_moved_modeled) / (r.ms.p50 * 1e-3) / 1e9;
        r.note = "one API call incl. allocation of the returned output; tflops from P50";
        cases.push_back(r);
    }
    // ---- split-K decode (config C3: B=128, S_kv=4096, bf16) ------------------------------------------------
    {
        const int64_t b = small ? 8 : 128, s = small ? 1024 : 4096;
        sci::Tensor q = Filled({b, hq, 1, d}, sci::DType::kBFloat16, *device, 4), k = Filled({b, hkv, s, d}, sci::DType::kBFloat16, *device, 5),
                    v = Filled({b, hkv, s, d}, sci::DType::kBFloat16, *device, 6);
        sca::AttentionConfig cfg;
        cfg.backend = sca::BackendKind::kDecode;
        cfg.causal = true;
        Record r;
        r.impl = "sca::decode_attention";
        r.case_id = "decode_B" + std::to_string(b) + "_Skv" + std::to_string(s) + "_bf16";
        r.params_json = Params(b, hq, hkv, 1, s, d, "bf16", true);
        double ws = 0;
        if (!run.Time([&] {
                auto out = sca::decode_attention(q, k, v, cfg);
                if (out.ok()) ws = static_cast<double>(out->stats.workspace_bytes) / 1e6;
                return out.ok();
            }, &r.ms)) return 4;
        r.workspace_mb = ws;
        r.flops_effective = 4.0 * b * hq * d * s;
        r.tflops = r.flops_effective / (r.ms.p50 * 1e-3) / 1e12;
        r.bytes_moved_modeled = 2 * b * hkv * s * d * 2 + 2 * b * hq * d * 2;
        r.effective_bw_gbps = static_cast<double>(r.bytes_moved_modeled) / (r.ms.p50 * 1e-3) / 1e9;
        r.note = "one API call incl. output allocation and pooled split-K scratch; GB/s from P50";
        cases.push_back(r);
    }
    // ---- paged decode (config C4 shape: ragged lengths, 16-token pages) through PagedKVCache ---------------
    {
        const int64_t nseq = small ? 16 : 256, lo = 512, hi = small ? 1024 : 8192, bs = 16;
        std::vector<int64_t> lens(static_cast<size_t>(nseq));
        int64_t total = 0;
        uint32_t s = 99;
        for (int64_t& n : lens) {
            s = s * 1664525u + 1013904223u;
            n = lo + static_cast<int64_t>(s >> 8) % (hi - lo + 1);
            total += n;
        }
        sca::KVCacheConfig kc;
        kc.num_layers = 1;
        kc.num_kv_heads = hkv;
        kc.head_dim = d;
        kc.block_size = bs;
        kc.max_num_seqs = nseq;
        kc.dtype = sci::DType::kBFloat16;
        kc.num_blocks = total / bs + 2 * nseq;
        auto made = sca::PagedKVCache::Create(kc, *device);
        if (!made.ok()) {
            std::printf("[bench] PagedKVCache::Create failed: %s\n", made.error().ToString().c_str());
            return 4;
        }
        sca::PagedKVCache cache = std::move(*made);
        for (int64_t r = 0; r < nseq; ++r) {
            const int64_t n = lens[static_cast<size_t>(r)];
            sci::Tensor kt = Filled({n, hkv, d}, kc.dtype, *device, 100 + static_cast<uint32_t>(r));
            if (!cache.AppendTokens(r, 0, kt, kt, nullptr).ok()) return 4;
        }
        if (!cache.SyncPageTable(nullptr).ok()) return 4;
        sci::Tensor q = Filled({nseq, hq, 1, d}, kc.dtype, *device, 7);
        sca::PagedAttentionParams params;
        params.page_table = cache.PageTableDevicePtr();
        params.seq_lens = cache.SeqLensDevicePtr();
        params.num_seqs = nseq;
        params.block_size = bs;
        params.max_blocks_per_seq = cache.MaxBlocksPerSeq();
        sca::AttentionConfig cfg;
        cfg.backend = sca::BackendKind::kPaged;
        cfg.causal = true;
        Record r;
        r.impl = "sca::paged_attention";
        r.case_id = "paged_decode_" + std::to_string(nseq) + "seq_len" + std::to_string(lo) + "-" + std::to_string(hi) + "_bs16_bf16";
        r.params_json = Params(nseq, hq, hkv, 1, total / nseq, d, "bf16", true);
        if (!run.Time([&] { return sca::paged_attention(q, cache, params, cfg).ok(); }, &r.ms)) return 4;
        r.flops_effective = 4.0 * hq * d * static_cast<double>(total);
        r.tflops = r.flops_effective / (r.ms.p50 * 1e-3) / 1e12;
        r.bytes_moved_modeled = total * (2 * hkv * d * 2) + 2 * nseq * hq * d * 2;
        r.effective_bw_gbps = static_cast<double>(r.bytes_moved_modeled) / (r.ms.p50 * 1e-3) / 1e9;
        r.note = "one API call over a PagedKVCache (attention only, no append); GB/s from P50";
        cases.push_back(r);
    }

    for (const Record& c : cases) {
        std::printf("[bench] %-48s %-26s p50 %.4f ms  p90 %.4f  p99 %.4f  %.1f TFLOP/s  %.0f GB/s\n", c.case_id.c_str(), c.impl.c_str(),
                    c.ms.p50, c.ms.p90, c.ms.p99, c.tflops, c.effective_bw_gbps);
    }
    char cc[16];
    std::snprintf(cc, sizeof(cc), "%d.%d", cap.major, cap.minor);
    WriteJson(out_dir + "/bench_attention.json", cap.device_name, cc, run.warmup, run.runs, cases);
    WriteCsv(out_dir + "/bench_attention.csv", run.warmup, run.runs, cases);
    cudaEventDestroy(run.start);
    cudaEventDestroy(run.stop);
    return 0;
}
