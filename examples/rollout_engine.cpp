// A serving loop on the public C++ API, end to end on one GPU: prefill of uneven prompts through the
// flash backend, KV written into paged caches, then batched decode steps (one batched append and one
// paged-attention call per layer and step). It plays the role of the reference's
// examples/rollout_engine_stub.cpp (same stages: prefill on token-major views -> append -> page-table
// sync -> paged decode), extended to several layers (one PagedKVCache per layer, because a cache
// advances a sequence on every append), to the batched append, to follow-up prompts (a chunk of new tokens per
// request that attends over the paged cache in ONE chunked-prefill launch per layer) and to several GPUs.
//
//   rollout_engine [--requests N] [--layers L] [--new-tokens T] [--prompt-min A] [--prompt-max B]
//                  [--followup F] [--gpus G] [--verify]
//
// --gpus G serves G times the requests: the process starts one copy of itself per GPU (CUDA_VISIBLE_DEVICES = g),
// every copy serves its own requests on its own caches - requests are independent, nothing crosses GPUs - and the
// parent adds up the rates. --followup 0 skips the follow-up stage.
// --verify re-computes the last decode step of layer 0 for every request with the split-K decode backend
// on the request's gathered (contiguous) cache, and the follow-up outputs of the first requests with the flash
// backend on the gathered cache, and fails if the backends differ by more than 2e-3.
// Exit codes: 0 ok, 2 no GPU, 3 KV budget, 4 a call failed, 5 verification failed.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "device/cuda_device.hpp"
#include "scicompute_attention/attention.hpp"
#include "scicompute_attention/paged_attention.hpp"
#include "scicompute_attention/paged_kv_cache.hpp"

namespace {

constexpr int64_t kHeadsQ = 32, kHeadsKv = 8, kHeadDim = 128, kBlockSize = 16;

struct Args {
    int64_t requests{32}, layers{4}, new_tokens{16}, prompt_min{64}, prompt_max{1024}, followup{64}, gpus{1};
    int64_t shard{-1};  // >= 0: this process is copy `shard` of a multi-GPU run
    bool verify{false};
};

bool Parse(int argc, char** argv, Args* a) {
    for (int i = 1; i < argc; ++i) {
        const std::string s = argv[i];
        auto next = [&](int64_t* dst) {
            if (i + 1 >= argc) return false;
            *dst = std::atoll(argv[++i]);
            return *dst > 0;
        };
        bool ok = true;
        if (s == "--requests") ok = next(&a->requests);
        else if (s == "--layers") ok = next(&a->layers);
        else if (s == "--new-tokens") ok = next(&a->new_tokens);
        else if (s == "--prompt-min") ok = next(&a->prompt_min);
        else if (s == "--prompt-max") ok = next(&a->prompt_max);
        else if (s == "--gpus") ok = next(&a->gpus);
        else if (s == "--followup") {
            ok = i + 1 < argc;
            if (ok) a->followup = std::atoll(argv[++i]);
            ok = ok && a->followup >= 0;
        } else if (s == "--shard") {
            ok = i + 1 < argc;
            if (ok) a->shard = std::atoll(argv[++i]);
        }
        else if (s == "--verify") a->verify = true;
        else ok = false;
        if (!ok) {
            std::fprintf(stderr, "bad argument: %s\n", s.c_str());
            return false;
        }
    }
    return a->prompt_min <= a->prompt_max;
}

// float -> IEEE half, round to nearest even (values here are small and finite)
uint16_t ToHalf(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t exp = static_cast<int32_t>((x >> 23) & 0xff) - 127 + 15;
    uint32_t man = x & 0x7fffffu;
    if (exp <= 0) return static_cast<uint16_t>(sign);  // flush tiny values
    if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
    uint32_t half = sign | (static_cast<uint32_t>(exp) << 10) | (man >> 13);
    const uint32_t rest = man & 0x1fffu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1u))) ++half;
    return static_cast<uint16_t>(half);
}
float FromHalf(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
    if (exp == 0) return 0.0f * (sign ? -1.0f : 1.0f);
    const uint32_t x = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

// Device fp16 tensor filled with a seeded pattern in [-amp, amp].
sci::Tensor Filled(std::initializer_list<int64_t> dims, sci::Device& dev, uint32_t seed, float amp) {
    sci::Tensor t(sci::TensorShape(dims), sci::DType::kFloat16, dev);
    std::vector<uint16_t> host(static_cast<size_t>(t.num_elements()));
    uint32_t s = seed * 2654435761u + 12345u;
    for (uint16_t& h : host) {
        s = s * 1664525u + 1013904223u;
        h = ToHalf(amp * (static_cast<float>(s >> 8) * (2.0f / 16777216.0f) - 1.0f));
    }
    t.copy_from(host.data(), host.size() * sizeof(uint16_t));
    return t;
}

sci::Tensor View(sci::Tensor& base, std::initializer_list<int64_t> dims) {
    return sci::Tensor(sci::TensorShape(dims), base.dtype(), base.device(), base.data(), false);
}

double Ms(std::chrono::steady_clock::time_point a, std::chrono::steady_clock::time_point b) {
    return std::chrono::duration<double, std::milli>(b - a).count();
}

// One copy of this program per GPU; the parent adds up the "[rollout-rates]" lines of the copies.
int RunOnSeveralGpus(const Args& args, const char* self) {
    std::vector<FILE*> pipes;
    for (int64_t g = 0; g < args.gpus; ++g) {
        std::string cmd = "CUDA_VISIBLE_DEVICES=" + std::to_string(g) + " '" + self + "' --shard " + std::to_string(g) +
                          " --requests " + std::to_string(args.requests) + " --layers " + std::to_string(args.layers) +
                          " --new-tokens " + std::to_string(args.new_tokens) + " --prompt-min " + std::to_string(args.prompt_min) +
                          " --prompt-max " + std::to_string(args.prompt_max) + " --followup " + std::to_string(args.followup) +
                          (args.verify ? " --verify" : "") + " 2>&1";
        FILE* f = popen(cmd.c_str(), "r");  // all copies run at the same time; they are read one after the other
        if (f == nullptr) {
            std::printf("[rollout] cannot start the copy for GPU %lld\n", static_cast<long long>(g));
            return 4;
        }
        pipes.push_back(f);
    }
    double prefill = 0.0, decode = 0.0, followup = 0.0;
    int worst = 0;
    for (size_t g = 0; g < pipes.size(); ++g) {
        char line[512];
        while (std::fgets(line, sizeof(line), pipes[g]) != nullptr) {
            double a = 0.0, b = 0.0, c = 0.0;
            if (std::sscanf(line, "[rollout-rates] prefill=%lf decode=%lf followup=%lf", &a, &b, &c) == 3) {
                prefill += a;
                decode += b;
                followup += c;
            } else {
                std::printf("[gpu %zu] %s", g, line);
            }
        }
        const int status = pclose(pipes[g]);
        const int code = (status >> 8) & 0xff;  // exit status of the shell = exit status of the copy
        if (code != 0) worst = code;
    }
    std::printf("[rollout] %lld GPUs together: %.0f prompt tokens/s per layer, %.0f generated tokens/s, %.0f follow-up tokens/s per layer\n",
                static_cast<long long>(args.gpus), prefill, decode, followup);
    return worst;
}

}  // namespace

int main(int argc, char** argv) {
    Args args;
    if (!Parse(argc, argv, &args)) return 1;
    if (args.gpus > 1 && args.shard < 0) return RunOnSeveralGpus(args, argv[0]);
    std::shared_ptr<sci::Device> device = sci::DeviceManager::Instance().get_device(sci::DeviceType::kCUDA, 0);
    if (device == nullptr) {
        std::printf("[rollout] no CUDA device\n");
        return 2;
    }
    std::vector<int64_t> prompt(static_cast<size_t>(args.requests));
    int64_t tokens_needed = 0;
    for (int64_t r = 0; r < args.requests; ++r) {
        const int64_t span = args.prompt_max - args.prompt_min + 1;
        prompt[static_cast<size_t>(r)] = args.prompt_min + (r * 7919 + 13) % span;
        tokens_needed += prompt[static_cast<size_t>(r)] + args.new_tokens + args.followup;
    }

    sca::KVCacheConfig kv_cfg;
    kv_cfg.num_layers = 1;
    kv_cfg.num_kv_heads = kHeadsKv;
    kv_cfg.head_dim = kHeadDim;
    kv_cfg.block_size = kBlockSize;
    kv_cfg.max_num_seqs = args.requests;
    kv_cfg.dtype = sci::DType::kFloat16;
    kv_cfg.num_blocks = (tokens_needed + kBlockSize - 1) / kBlockSize + args.requests;
    const auto bytes = sca::KvCacheBytes(kv_cfg);
    if (!bytes.ok()) {
        std::printf("[rollout] KV budget rejected: %s\n", bytes.error().ToString().c_str());
        return 3;
    }
    std::vector<sca::PagedKVCache> caches;
    for (int64_t l = 0; l < args.layers; ++l) {
        auto made = sca::PagedKVCache::Create(kv_cfg, *device);
        if (!made.ok()) {  // an error code with advice, never an out-of-memory crash
            std::printf("[rollout] PagedKVCache::Create (layer %lld) failed: %s\n", static_cast<long long>(l),
                        made.error().ToString().c_str());
            return 3;
        }
        caches.push_back(std::move(*made));
    }
    std::printf("[rollout] %lld requests, prompts %lld..%lld, %lld layers, %lld blocks x %lld tokens per layer (%.1f MiB)\n",
                static_cast<long long>(args.requests), static_cast<long long>(args.prompt_min),
                static_cast<long long>(args.prompt_max), static_cast<long long>(args.layers),
                static_cast<long long>(kv_cfg.num_blocks), static_cast<long long>(kBlockSize),
                static_cast<double>(*bytes) / (1024.0 * 1024.0));

    // ---- prefill -------------------------------------------------------------------------------------
    sca::AttentionConfig prefill_cfg;
    prefill_cfg.backend = sca::BackendKind::kFlash;
    prefill_cfg.causal = true;
    prefill_cfg.layout = sca::AttnLayout::kBSHD;  // packed [tokens, heads, dim] buffers are token-major
    int64_t prompt_tokens = 0;
    // the activations of one layer per request, made before the clock starts and fed to every layer
    std::vector<sci::Tensor> q_in, k_in, v_in;
    for (int64_t r = 0; r < args.requests; ++r) {
        const int64_t n = prompt[static_cast<size_t>(r)];
        const uint32_t seed = static_cast<uint32_t>(r * 131 + (args.shard > 0 ? args.shard * 7717 : 0));
        q_in.push_back(Filled({n, kHeadsQ, kHeadDim}, *device, 1000 + seed, 1.0f));
        k_in.push_back(Filled({n, kHeadsKv, kHeadDim}, *device, 2000 + seed, 1.0f));
        v_in.push_back(Filled({n, kHeadsKv, kHeadDim}, *device, 3000 + seed, 0.5f));
    }
    device->synchronize();
    const auto t0 = std::chrono::steady_clock::now();
    for (int64_t r = 0; r < args.requests; ++r) {
        const int64_t n = prompt[static_cast<size_t>(r)];
        prompt_tokens += n;
        sci::Tensor& q_packed = q_in[static_cast<size_t>(r)];
        sci::Tensor& k_packed = k_in[static_cast<size_t>(r)];
        sci::Tensor& v_packed = v_in[static_cast<size_t>(r)];
        for (int64_t l = 0; l < args.layers; ++l) {
            sci::Tensor q = View(q_packed, {1, n, kHeadsQ, kHeadDim});
            sci::Tensor k = View(k_packed, {1, n, kHeadsKv, kHeadDim});
            sci::Tensor v = View(v_packed, {1, n, kHeadsKv, kHeadDim});
            const auto out = sca::flash_attention(q, k, v, prefill_cfg);
            if (!out.ok()) {
                std::printf("[rollout] prefill failed: %s\n", out.error().ToString().c_str());
                return 4;
            }
            const sci::Status stored = caches[static_cast<size_t>(l)].AppendTokens(r, 0, k_packed, v_packed, nullptr);
            if (!stored.ok()) {
                std::printf("[rollout] KV append failed: %s\n", stored.ToString().c_str());
                return 4;
            }
        }
    }
    device->synchronize();
    const auto t1 = std::chrono::steady_clock::now();

    // ---- decode loop ---------------------------------------------------------------------------------
    sca::AttentionConfig decode_cfg;
    decode_cfg.backend = sca::BackendKind::kPaged;
    decode_cfg.causal = true;
    // one set of new-token activations per layer, made before the clock starts and reused by every step
    std::vector<sci::Tensor> q_steps, k_steps, v_steps;
    for (int64_t l = 0; l < args.layers; ++l) {
        const uint32_t seed = static_cast<uint32_t>(l * 17);
        k_steps.push_back(Filled({args.requests, kHeadsKv, kHeadDim}, *device, 6000 + seed, 1.0f));
        v_steps.push_back(Filled({args.requests, kHeadsKv, kHeadDim}, *device, 7000 + seed, 0.5f));
        q_steps.push_back(Filled({args.requests, kHeadsQ, 1, kHeadDim}, *device, 5000 + seed, 1.0f));
    }
    device->synchronize();
    const auto t1b = std::chrono::steady_clock::now();
    sci::Tensor last_out;
    for (int64_t step = 0; step < args.new_tokens; ++step) {
        for (int64_t l = 0; l < args.layers; ++l) {
            sci::Tensor& k_step = k_steps[static_cast<size_t>(l)];
            sci::Tensor& v_step = v_steps[static_cast<size_t>(l)];
            sci::Tensor& q_step = q_steps[static_cast<size_t>(l)];
            sca::PagedKVCache& cache = caches[static_cast<size_t>(l)];
            const sci::Status appended = cache.AppendTokenBatch(args.requests, 0, k_step, v_step, nullptr);
            if (!appended.ok()) {
                std::printf("[rollout] batched append failed: %s\n", appended.ToString().c_str());
                return 4;
            }
            sca::PagedAttentionParams params;
            params.page_table = cache.PageTableDevicePtr();
            params.seq_lens = cache.SeqLensDevicePtr();
            params.num_seqs = args.requests;
            params.block_size = kBlockSize;
            params.max_blocks_per_seq = cache.MaxBlocksPerSeq();
            params.layer = 0;
            auto decoded = sca::paged_attention(q_step, cache, params, decode_cfg);
            if (!decoded.ok()) {
                std::printf("[rollout] paged decode failed: %s\n", decoded.error().ToString().c_str());
                return 4;
            }
            if (l == 0 && step == args.new_tokens - 1) last_out = std::move(decoded->out);
        }
    }
    device->synchronize();
    const auto t2 = std::chrono::steady_clock::now();

    std::vector<int64_t> decode_len(static_cast<size_t>(args.requests));  // cache lengths the last decode step saw
    for (int64_t r = 0; r < args.requests; ++r) decode_len[static_cast<size_t>(r)] = caches[0].SeqLength(r);

    // ---- follow-up prompts: a chunk of new tokens per request over the paged cache -----------------------
    // The chunk's K/V go into the cache first (as for any prompt), then ONE chunked-prefill launch per layer serves
    // all requests: every new token attends over its request's whole cached history, causally within the chunk.
    double followup_ms = 0.0;
    sci::Tensor followup_out;
    std::vector<sci::Tensor> fq, fk, fv;
    std::vector<int32_t> cu_follow(static_cast<size_t>(args.requests) + 1, 0);
    if (args.followup > 0) {
        const int64_t f = args.followup;
        for (int64_t r = 0; r < args.requests; ++r) cu_follow[static_cast<size_t>(r) + 1] = static_cast<int32_t>((r + 1) * f);
        for (int64_t l = 0; l < args.layers; ++l) {
            const uint32_t seed = static_cast<uint32_t>(l * 29);
            fq.push_back(Filled({args.requests * f, kHeadsQ, kHeadDim}, *device, 8000 + seed, 1.0f));
            fk.push_back(Filled({args.requests * f, kHeadsKv, kHeadDim}, *device, 8100 + seed, 1.0f));
            fv.push_back(Filled({args.requests * f, kHeadsKv, kHeadDim}, *device, 8200 + seed, 0.5f));
        }
        device->synchronize();
        const auto f0 = std::chrono::steady_clock::now();
        sca::AttentionConfig follow_cfg;
        follow_cfg.causal = true;
        for (int64_t l = 0; l < args.layers; ++l) {
            sca::PagedKVCache& cache = caches[static_cast<size_t>(l)];
            for (int64_t r = 0; r < args.requests; ++r) {
                const int64_t row = kHeadsKv * kHeadDim;
                sci::Tensor kr(sci::TensorShape({f, kHeadsKv, kHeadDim}), sci::DType::kFloat16, *device,
                               static_cast<uint16_t*>(fk[static_cast<size_t>(l)].data()) + r * f * row, false);
                sci::Tensor vr(sci::TensorShape({f, kHeadsKv, kHeadDim}), sci::DType::kFloat16, *device,
                               static_cast<uint16_t*>(fv[static_cast<size_t>(l)].data()) + r * f * row, false);
                const sci::Status stored = cache.AppendTokens(r, 0, kr, vr, nullptr);
                if (!stored.ok()) {
                    std::printf("[rollout] follow-up append failed: %s\n", stored.ToString().c_str());
                    return 4;
                }
            }
            if (const sci::Status synced = cache.SyncPageTable(nullptr); !synced.ok()) return 4;
            auto served = sca::paged_prefill(fq[static_cast<size_t>(l)], cache, args.requests, cu_follow.data(), 0, follow_cfg);
            if (!served.ok()) {
                std::printf("[rollout] chunked prefill over the paged cache failed: %s\n", served.error().ToString().c_str());
                return 4;
            }
            if (l == 0) followup_out = std::move(served->out);
        }
        device->synchronize();
        followup_ms = Ms(f0, std::chrono::steady_clock::now());
    }

    const double prefill_ms = Ms(t0, t1), decode_ms = Ms(t1b, t2);
    sci::Tensor& last_q = q_steps[0];
    const int64_t generated = args.requests * args.new_tokens;
    std::printf("[rollout] prefill: %lld prompt tokens x %lld layers in %.2f ms -> %.0f prompt tokens/s per layer\n",
                static_cast<long long>(prompt_tokens), static_cast<long long>(args.layers), prefill_ms,
                1000.0 * static_cast<double>(prompt_tokens * args.layers) / prefill_ms);
    std::printf("[rollout] decode : %lld steps x %lld layers in %.2f ms -> %.0f generated tokens/s (%.3f ms per step)\n",
                static_cast<long long>(args.new_tokens), static_cast<long long>(args.layers), decode_ms,
                1000.0 * static_cast<double>(generated) / decode_ms, decode_ms / static_cast<double>(args.new_tokens));
    const double followup_rate =
        followup_ms > 0.0 ? 1000.0 * static_cast<double>(args.requests * args.followup * args.layers) / followup_ms : 0.0;
    if (args.followup > 0) {
        std::printf("[rollout] follow-up: %lld requests x %lld new tokens x %lld layers over the paged cache in %.2f ms -> %.0f tokens/s per layer\n",
                    static_cast<long long>(args.requests), static_cast<long long>(args.followup),
                    static_cast<long long>(args.layers), followup_ms, followup_rate);
    }
    if (args.shard >= 0) {
        std::printf("[rollout-rates] prefill=%.1f decode=%.1f followup=%.1f\n",
                    1000.0 * static_cast<double>(prompt_tokens * args.layers) / prefill_ms,
                    1000.0 * static_cast<double>(generated) / decode_ms, followup_rate);
    }
    const sca::KVCacheStats stats = caches[0].Stats();
    std::printf("[rollout] layer 0 cache: %lld of %lld blocks used, %lld appends\n", static_cast<long long>(stats.used_blocks),
                static_cast<long long>(stats.num_blocks), static_cast<long long>(stats.num_appends));

    if (args.verify) {
        // paged output of the last step vs. the split-K decode backend on the gathered, contiguous cache
        sca::PagedKVCache& cache = caches[0];
        std::vector<uint16_t> paged(static_cast<size_t>(args.requests * kHeadsQ * kHeadDim));
        device->copy_to_host(paged.data(), last_out.data(), paged.size() * sizeof(uint16_t));
        sca::AttentionConfig dense_cfg;
        dense_cfg.backend = sca::BackendKind::kDecode;
        dense_cfg.causal = true;
        dense_cfg.layout = sca::AttnLayout::kBSHD;
        double worst = 0.0;
        for (int64_t r = 0; r < args.requests; ++r) {
            const int64_t len = decode_len[static_cast<size_t>(r)];
            const int64_t nblk = (len + kBlockSize - 1) / kBlockSize;
            const int32_t* ids = cache.PageTableDevicePtr() + r * cache.MaxBlocksPerSeq();
            auto gk = cache.Storage().GatherK(0, ids, nblk, nullptr);
            auto gv = cache.Storage().GatherV(0, ids, nblk, nullptr);
            if (!gk.ok() || !gv.ok()) return 4;
            sci::Tensor kc = View(*gk, {1, len, kHeadsKv, kHeadDim});
            sci::Tensor vc = View(*gv, {1, len, kHeadsKv, kHeadDim});
            sci::Tensor q1(sci::TensorShape({1, 1, kHeadsQ, kHeadDim}), sci::DType::kFloat16, *device,
                           static_cast<uint16_t*>(last_q.data()) + r * kHeadsQ * kHeadDim, false);
            const auto dense = sca::decode_attention(q1, kc, vc, dense_cfg);
            if (!dense.ok()) {
                std::printf("[rollout] verification decode failed: %s\n", dense.error().ToString().c_str());
                return 4;
            }
            std::vector<uint16_t> ref(static_cast<size_t>(kHeadsQ * kHeadDim));
            device->copy_to_host(ref.data(), dense->out.data(), ref.size() * sizeof(uint16_t));
            for (size_t i = 0; i < ref.size(); ++i) {
                const double d = std::fabs(static_cast<double>(FromHalf(ref[i])) -
                                           static_cast<double>(FromHalf(paged[static_cast<size_t>(r) * ref.size() + i])));
                worst = std::max(worst, d);
            }
        }
        std::printf("[rollout] verify: paged vs contiguous decode, max abs difference %.3e over %lld requests\n", worst,
                    static_cast<long long>(args.requests));
        if (!(worst <= 2e-3)) return 5;
        if (args.followup > 0) {
            // follow-up outputs of the first requests vs. the flash backend on the gathered cache (S_q < S_kv, causal)
            const int64_t f = args.followup, checked = std::min<int64_t>(args.requests, 4);
            sca::AttentionConfig flash_cfg;
            flash_cfg.backend = sca::BackendKind::kFlash;
            flash_cfg.causal = true;
            flash_cfg.layout = sca::AttnLayout::kBSHD;
            std::vector<uint16_t> got(static_cast<size_t>(checked * f * kHeadsQ * kHeadDim));
            device->copy_to_host(got.data(), followup_out.data(), got.size() * sizeof(uint16_t));
            double worst_follow = 0.0;
            for (int64_t r = 0; r < checked; ++r) {
                const int64_t len = cache.SeqLength(r);
                const int64_t nblk = cache.LogicalBlockCount(r);
                const int32_t* ids = cache.PageTableDevicePtr() + r * cache.MaxBlocksPerSeq();
                auto gk = cache.Storage().GatherK(0, ids, nblk, nullptr);
                auto gv = cache.Storage().GatherV(0, ids, nblk, nullptr);
                if (!gk.ok() || !gv.ok()) return 4;
                sci::Tensor kc = View(*gk, {1, len, kHeadsKv, kHeadDim});
                sci::Tensor vc = View(*gv, {1, len, kHeadsKv, kHeadDim});
                sci::Tensor qc(sci::TensorShape({1, f, kHeadsQ, kHeadDim}), sci::DType::kFloat16, *device,
                               static_cast<uint16_t*>(fq[0].data()) + r * f * kHeadsQ * kHeadDim, false);
                const auto dense = sca::flash_attention(qc, kc, vc, flash_cfg);
                if (!dense.ok()) {
                    std::printf("[rollout] verification prefill failed: %s\n", dense.error().ToString().c_str());
                    return 4;
                }
                // flash returns BHSD [1, H, f, D]; the follow-up output is token-major [f, H, D]
                std::vector<uint16_t> ref(static_cast<size_t>(f * kHeadsQ * kHeadDim));
                device->copy_to_host(ref.data(), dense->out.data(), ref.size() * sizeof(uint16_t));
                for (int64_t t = 0; t < f; ++t) {
                    for (int64_t h = 0; h < kHeadsQ; ++h) {
                        for (int64_t e = 0; e < kHeadDim; ++e) {
                            const float a = FromHalf(ref[static_cast<size_t>((h * f + t) * kHeadDim + e)]);
                            const float b = FromHalf(got[static_cast<size_t>(((r * f + t) * kHeadsQ + h) * kHeadDim + e)]);
                            worst_follow = std::max(worst_follow, std::fabs(static_cast<double>(a) - static_cast<double>(b)));
                        }
                    }
                }
            }
            std::printf("[rollout] verify: chunked prefill over the paged cache vs flash on the gathered cache, max abs difference %.3e over %lld requests\n",
                        worst_follow, static_cast<long long>(checked));
            if (!(worst_follow <= 2e-3)) return 5;
        }
    }
    return 0;
}
