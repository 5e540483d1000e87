// Level-1 "naive" attention: the score matrix is materialised in an fp32 workspace, exactly the behaviour
// the reference documents and tests for its naive backend (stats.materialized_score_bytes > 0). Stands in
// for LaunchNaiveForward and its three kernels (src/backends/naive/attention_naive.cuh:28-60): scores,
// row softmax in place, P.V. It exists as the readable ground truth next to the tcgen05 kernel and as the
// fp32 path; nothing here is tuned - every thread works on one element.
//
//   scores  S[b,h,i,j] = scale * q_i . k_j            (-inf where the bottom-right causal mask hides j)
//   softmax P = exp(S - rowmax) / rowsum in place      (a fully masked row becomes zeros), optional LSE
//   output  O[b,h,i,:] = sum_j P[i,j] v_j
#include <algorithm>

#include "common.cuh"

namespace sca_b200 {
namespace {

struct NaiveParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    float* lse;
    float* scores;  // [batch, heads, seq_q, seq_kv] fp32
    int64_t batch, heads, kv_heads, seq_q, seq_kv, head_dim;
    int64_t q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss;
    float scale;
    int causal;
    int64_t diagonal;
};

template <typename T>
__global__ void __launch_bounds__(256) naive_scores_kernel(const NaiveParams p) {
    const int64_t total = p.batch * p.heads * p.seq_q * p.seq_kv;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t rest = idx;
        const int64_t j = rest % p.seq_kv;
        rest /= p.seq_kv;
        const int64_t i = rest % p.seq_q;
        rest /= p.seq_q;
        const int64_t h = rest % p.heads;
        const int64_t b = rest / p.heads;
        float s = -CUDART_INF_F;
        if (!p.causal || j <= i + p.diagonal) {
            const T* q_row = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh + i * p.q_ss;
            const T* k_row = reinterpret_cast<const T*>(p.k) + b * p.k_sb + (h / (p.heads / p.kv_heads)) * p.k_sh + j * p.k_ss;
            float dot = 0.0f;
            for (int64_t d = 0; d < p.head_dim; ++d) dot = fmaf(ToFloat(q_row[d]), ToFloat(k_row[d]), dot);
            s = dot * p.scale;
        }
        p.scores[idx] = s;
    }
}

// one warp per score row
__global__ void __launch_bounds__(128) naive_softmax_kernel(const NaiveParams p) {
    const int lane = threadIdx.x & 31;
    const int64_t rows = p.batch * p.heads * p.seq_q;
    const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    for (int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
        float* s = p.scores + row * p.seq_kv;
        float m = -CUDART_INF_F;
        for (int64_t j = lane; j < p.seq_kv; j += 32) m = fmaxf(m, s[j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.0f;
        if (m != -CUDART_INF_F) {
            for (int64_t j = lane; j < p.seq_kv; j += 32) l += __expf(s[j] - m);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        for (int64_t j = lane; j < p.seq_kv; j += 32) s[j] = l > 0.0f ? __expf(s[j] - m) * inv : 0.0f;
        if (p.lse != nullptr && lane == 0) p.lse[row] = l > 0.0f ? m + logf(l) : -CUDART_INF_F;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) naive_pv_kernel(const NaiveParams p) {
    const int64_t total = p.batch * p.heads * p.seq_q * p.head_dim;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t rest = idx;
        const int64_t d = rest % p.head_dim;
        rest /= p.head_dim;
        const int64_t row = rest;  // (b, h, i) flattened
        const int64_t i = rest % p.seq_q;
        rest /= p.seq_q;
        const int64_t h = rest % p.heads;
        const int64_t b = rest / p.heads;
        const float* prob = p.scores + row * p.seq_kv;
        const T* v_col = reinterpret_cast<const T*>(p.v) + b * p.v_sb + (h / (p.heads / p.kv_heads)) * p.v_sh + d;
        int64_t visible = p.seq_kv;
        if (p.causal) {
            const int64_t upto = i + p.diagonal + 1;
            visible = upto < 0 ? 0 : (upto < p.seq_kv ? upto : p.seq_kv);
        }
        float acc = 0.0f;
        for (int64_t j = 0; j < visible; ++j) acc = fmaf(prob[j], ToFloat(v_col[j * p.v_ss]), acc);
        reinterpret_cast<T*>(p.out)[b * p.o_sb + h * p.o_sh + i * p.o_ss + d] = FromFloat<T>(acc);
    }
}

unsigned GridFor(int64_t items, int threads) {
    const int64_t want = (items + threads - 1) / threads;
    return static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(SmCount()) * 64)));
}

template <typename T>
int LaunchNaive(const NaiveParams& p, cudaStream_t stream) {
    const int64_t rows = p.batch * p.heads * p.seq_q;
    naive_scores_kernel<T><<<GridFor(rows * p.seq_kv, 256), 256, 0, stream>>>(p);
    if (int rc = CheckLaunch("naive_scores_kernel", stream)) return rc;
    naive_softmax_kernel<<<GridFor(rows * 32, 128), 128, 0, stream>>>(p);
    if (int rc = CheckLaunch("naive_softmax_kernel", stream)) return rc;
    naive_pv_kernel<T><<<GridFor(rows * p.head_dim, 256), 256, 0, stream>>>(p);
    return CheckLaunch("naive_pv_kernel", stream);
}

}  // namespace
}  // namespace sca_b200

using namespace sca_b200;

extern "C" long long sca_naive_score_bytes(int64_t batch, int64_t heads, int64_t seq_q, int64_t seq_kv) {
    if (batch < 1 || heads < 1 || seq_q < 1 || seq_kv < 1) return -1;
    return static_cast<long long>(batch) * heads * seq_q * seq_kv * static_cast<long long>(sizeof(float));
}

extern "C" int sca_launch_naive_forward(const ScaFlashFwdParams* params, float* scores, void* stream) {
    ClearError();
    if (params == nullptr) return Fail(SCA_INVALID_ARGUMENT, "naive attention: null parameter block");
    const ScaFlashFwdParams& f = *params;
    if (f.q == nullptr || f.k == nullptr || f.v == nullptr || f.out == nullptr || scores == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "naive attention: null tensor pointer");
    }
    if (f.batch < 1 || f.num_heads < 1 || f.num_kv_heads < 1 || f.seq_q < 1 || f.seq_kv < 1 || f.head_dim < 1 ||
        f.num_heads % f.num_kv_heads != 0) {
        return Fail(SCA_INVALID_ARGUMENT, "naive attention: invalid geometry");
    }
    NaiveParams p{};
    p.q = f.q; p.k = f.k; p.v = f.v; p.out = f.out;
    p.lse = f.return_lse ? f.lse : nullptr;
    p.scores = scores;
    p.batch = f.batch; p.heads = f.num_heads; p.kv_heads = f.num_kv_heads;
    p.seq_q = f.seq_q; p.seq_kv = f.seq_kv; p.head_dim = f.head_dim;
    p.q_sb = f.q_sb; p.q_sh = f.q_sh; p.q_ss = f.q_ss;
    p.k_sb = f.k_sb; p.k_sh = f.k_sh; p.k_ss = f.k_ss;
    p.v_sb = f.v_sb; p.v_sh = f.v_sh; p.v_ss = f.v_ss;
    p.o_sb = f.o_sb; p.o_sh = f.o_sh; p.o_ss = f.o_ss;
    p.scale = f.scale; p.causal = f.causal; p.diagonal = f.diagonal;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (f.dtype_id) {
        case SCA_DTYPE_F32: return LaunchNaive<float>(p, s);
        case SCA_DTYPE_F16: return LaunchNaive<__half>(p, s);
        case SCA_DTYPE_BF16: return LaunchNaive<__nv_bfloat16>(p, s);
        default: break;
    }
    return Fail(SCA_INVALID_ARGUMENT, "naive attention: unsupported dtype id " + std::to_string(f.dtype_id));
}
