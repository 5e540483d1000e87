// Plain SIMT attention: the functional (not tuned) path behind the reference-level backends.
//
// It serves three reference entry points with one kernel:
//   LaunchNaiveForward  (src/backends/naive/attention_naive.cuh:60)  - any dtype incl. fp32
//   LaunchTiledForward  (src/backends/tiled/attention_tiled.cuh:57)  - same contract
//   the fp32 instantiation of the split-K decode partial kernel
//   (src/backends/decode/decode_splitk.cu:66-140), including page-table addressing.
// One warp owns one (batch, head, query row[, split]); lane L holds head-dim elements
// L, L+32, ... (coalesced 64/128-byte row reads), scores are reduced with warp shuffles and the
// softmax is the usual running-max form in fp32. The score matrix is never materialised.
#include <algorithm>

#include "common.cuh"

namespace sca_b200 {
namespace {

struct SimtParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;           // normalised output (T) or nullptr when writing partials
    float* lse;          // optional, natural log
    float* partial_m;    // split mode: [rows * splits]
    float* partial_l;
    float* partial_o;    // [rows * splits, D]
    int64_t batch, heads, kv_heads, seq_q, seq_kv, head_dim, splits;
    int64_t q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss;
    float scale;
    int causal;
    int64_t diagonal;
    const int32_t* page_table;
    int64_t block_size, max_blocks_per_seq, num_kv_blocks;
    const int32_t* seq_lens;
};

constexpr int kMaxPerLane = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128) simt_attention_kernel(const SimtParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t total = p.batch * p.heads * p.seq_q * p.splits;
    if (warp_global >= total) return;
    int64_t rest = warp_global;
    const int64_t split = rest % p.splits;
    rest /= p.splits;
    const int64_t i = rest % p.seq_q;
    rest /= p.seq_q;
    const int64_t h = rest % p.heads;
    const int64_t b = rest / p.heads;
    const int64_t h_kv = h / (p.heads / p.kv_heads);
    const int per_lane = static_cast<int>(p.head_dim / 32);

    const T* q_row = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh + i * p.q_ss;
    const bool paged = p.page_table != nullptr;
    const T* k_base = reinterpret_cast<const T*>(p.k) + (paged ? 0 : b * p.k_sb) + h_kv * p.k_sh;
    const T* v_base = reinterpret_cast<const T*>(p.v) + (paged ? 0 : b * p.v_sb) + h_kv * p.v_sh;

    float qv[kMaxPerLane], acc[kMaxPerLane];
#pragma unroll
    for (int e = 0; e < kMaxPerLane; ++e) {
        qv[e] = e < per_lane ? ToFloat(q_row[lane + 32 * e]) : 0.0f;
        acc[e] = 0.0f;
    }

    int64_t visible = p.seq_lens != nullptr ? static_cast<int64_t>(p.seq_lens[b]) : p.seq_kv;
    if (p.causal) visible = min(visible, i + p.diagonal + 1);
    if (visible < 0) visible = 0;
    const int64_t chunk = (visible + p.splits - 1) / p.splits;
    const int64_t j_begin = split * chunk;
    const int64_t j_end = min(j_begin + chunk, visible);

    float m = -CUDART_INF_F, l = 0.0f;
    const float scale_log2 = p.scale * kLog2e;
    for (int64_t j = j_begin; j < j_end; ++j) {
        int64_t row = j;
        if (paged) {
            const int64_t logical = j / p.block_size;
            if (logical >= p.max_blocks_per_seq) continue;
            const int32_t phys = __ldg(p.page_table + b * p.max_blocks_per_seq + logical);
            if (phys < 0 || phys >= p.num_kv_blocks) continue;
            row = static_cast<int64_t>(phys) * p.block_size + j % p.block_size;
        }
        const T* k_row = k_base + row * p.k_ss;
        const T* v_row = v_base + row * p.v_ss;
        float dot = 0.0f;
#pragma unroll
        for (int e = 0; e < kMaxPerLane; ++e) {
            if (e < per_lane) dot += qv[e] * ToFloat(k_row[lane + 32 * e]);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float s = dot * scale_log2;
        const float m_new = fmaxf(m, s);
        const float alpha = Exp2(m - m_new);  // m = -inf -> 0
        const float w = Exp2(s - m_new);
        l = l * alpha + w;
#pragma unroll
        for (int e = 0; e < kMaxPerLane; ++e) {
            if (e < per_lane) acc[e] = acc[e] * alpha + w * ToFloat(v_row[lane + 32 * e]);
        }
        m = m_new;
    }

    if (p.partial_o != nullptr) {
        const int64_t flat = (b * p.heads + h) * p.splits + split;  // seq_q == 1 in split mode
        if (lane == 0) {
            p.partial_m[flat] = m * kLn2;
            p.partial_l[flat] = l;
        }
#pragma unroll
        for (int e = 0; e < kMaxPerLane; ++e) {
            if (e < per_lane) p.partial_o[flat * p.head_dim + lane + 32 * e] = acc[e];
        }
        return;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    T* o_row = reinterpret_cast<T*>(p.out) + b * p.o_sb + h * p.o_sh + i * p.o_ss;
#pragma unroll
    for (int e = 0; e < kMaxPerLane; ++e) {
        if (e < per_lane) o_row[lane + 32 * e] = FromFloat<T>(acc[e] * inv);
    }
    if (p.lse != nullptr && lane == 0) {
        p.lse[(b * p.heads + h) * p.seq_q + i] = l > 0.0f ? m * kLn2 + logf(l) : -CUDART_INF_F;
    }
}

int LaunchSimt(const SimtParams& p, int dtype, cudaStream_t stream) {
    const int64_t warps = p.batch * p.heads * p.seq_q * p.splits;
    const int64_t blocks = (warps + 3) / 4;
    if (blocks <= 0 || blocks > 0x7fffffffLL) {
        return Fail(SCA_INVALID_ARGUMENT, "simt attention: grid of " + std::to_string(blocks) + " blocks is out of range");
    }
    const unsigned grid = static_cast<unsigned>(blocks);
    switch (dtype) {
        case SCA_DTYPE_F32: simt_attention_kernel<float><<<grid, 128, 0, stream>>>(p); break;
        case SCA_DTYPE_F16: simt_attention_kernel<__half><<<grid, 128, 0, stream>>>(p); break;
        case SCA_DTYPE_BF16: simt_attention_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(p); break;
        default: return Fail(SCA_INVALID_ARGUMENT, "simt attention: unsupported dtype id " + std::to_string(dtype));
    }
    return CheckLaunch("simt_attention_kernel", stream);
}

}  // namespace

int LaunchDecodePartialF32(const ScaDecodeFwdParams& d, cudaStream_t stream) {
    if (d.head_dim % 32 != 0 || d.head_dim > 256) {
        return Fail(SCA_INVALID_ARGUMENT, "decode: head_dim=" + std::to_string(d.head_dim) + " is not instantiated");
    }
    SimtParams p{};
    p.q = d.q; p.k = d.k; p.v = d.v;
    p.partial_m = d.partial_m; p.partial_l = d.partial_l; p.partial_o = d.partial_o;
    p.batch = d.batch; p.heads = d.num_heads; p.kv_heads = d.num_kv_heads;
    p.seq_q = 1; p.seq_kv = d.seq_kv; p.head_dim = d.head_dim; p.splits = d.num_splits;
    p.q_sb = d.q_stride.s_b; p.q_sh = d.q_stride.s_h; p.q_ss = d.q_stride.s_s;
    p.k_sb = d.k_stride.s_b; p.k_sh = d.k_stride.s_h; p.k_ss = d.k_stride.s_s;
    p.v_sb = d.v_stride.s_b; p.v_sh = d.v_stride.s_h; p.v_ss = d.v_stride.s_s;
    p.scale = d.scale;
    p.page_table = d.page_table; p.block_size = d.block_size;
    p.max_blocks_per_seq = d.max_blocks_per_seq; p.num_kv_blocks = d.num_kv_blocks;
    p.seq_lens = d.seq_lens;
    return LaunchSimt(p, SCA_DTYPE_F32, stream);
}

}  // namespace sca_b200

using namespace sca_b200;

extern "C" int sca_launch_simt_forward(const ScaFlashFwdParams* params, void* stream) {
    ClearError();
    if (params == nullptr) return Fail(SCA_INVALID_ARGUMENT, "attention: null parameter block");
    const ScaFlashFwdParams& f = *params;
    if (f.q == nullptr || f.k == nullptr || f.v == nullptr || f.out == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "attention: null tensor pointer");
    }
    if (f.head_dim % 32 != 0 || f.head_dim < 32 || f.head_dim > 256) {
        return Fail(SCA_INVALID_ARGUMENT, "attention: head_dim=" + std::to_string(f.head_dim) + " is not instantiated");
    }
    if (f.batch < 1 || f.num_heads < 1 || f.num_kv_heads < 1 || f.seq_q < 1 || f.seq_kv < 1 ||
        f.num_heads % f.num_kv_heads != 0) {
        return Fail(SCA_INVALID_ARGUMENT, "attention: invalid geometry");
    }
    SimtParams p{};
    p.q = f.q; p.k = f.k; p.v = f.v; p.out = f.out;
    p.lse = f.return_lse ? f.lse : nullptr;
    p.batch = f.batch; p.heads = f.num_heads; p.kv_heads = f.num_kv_heads;
    p.seq_q = f.seq_q; p.seq_kv = f.seq_kv; p.head_dim = f.head_dim; p.splits = 1;
    p.q_sb = f.q_sb; p.q_sh = f.q_sh; p.q_ss = f.q_ss;
    p.k_sb = f.k_sb; p.k_sh = f.k_sh; p.k_ss = f.k_ss;
    p.v_sb = f.v_sb; p.v_sh = f.v_sh; p.v_ss = f.v_ss;
    p.o_sb = f.o_sb; p.o_sh = f.o_sh; p.o_ss = f.o_ss;
    p.scale = f.scale; p.causal = f.causal; p.diagonal = f.diagonal;
    return LaunchSimt(p, f.dtype_id, static_cast<cudaStream_t>(stream));
}
