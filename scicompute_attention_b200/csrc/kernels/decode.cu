// Split-K decode attention (one query token per head) over a contiguous or a paged KV cache.
//
// Stands in for the reference's decode_partial_kernel / decode_reduce_kernel
// (src/backends/decode/decode_splitk.cu:66-182) and the page-table variant
// (src/backends/paged/page_table.cuh:18-36). The arithmetic contract is the same - per split an
// online softmax producing (m, l, O) in fp32, then a max-rescaled merge - the execution plan is
// new and built for an HBM-bound problem:
//
//   * one CTA per (sequence, kv head, 16-query-head chunk, split): the whole GQA group shares one
//     pass over K and V, so every K/V byte is fetched from HBM once (the reference fetches it once
//     per query head);
//   * each of the 4 warps streams its own interleaved 16-token tiles through a private 3-stage
//     shared-memory ring filled with 16-byte cp.async copies (zero-filled for masked tokens), so
//     two tiles per warp are always in flight and no CTA-wide barrier sits in the main loop;
//   * the tiny matrix products run on the warp-level tensor-core path (m16n8k16, fp32 accumulate)
//     with operand fragments read straight from the ring by 128-bit loads: the head dimension is
//     consumed in a permuted order that both operands agree on, which is why no ldmatrix and no
//     transposition of V is needed; XOR swizzles keep those loads bank-conflict free;
//   * page tables are resolved once per token row by 16 lanes (one table read per row, broadcast
//     by shuffle), never per element.
//
// Algorithmic HBM traffic per token and kv head: 2 * D * sizeof(T) bytes (K row + V row), read once.
#include <algorithm>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace sca_b200 {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kTile = 16;   // tokens per warp step (k extent of the P.V product)
constexpr int kStages = 3;  // ring depth per warp

template <int D>
struct DecodeGeom {
    static constexpr int kRowBytes = D * 2;
    static constexpr int kChunksPerRow = kRowBytes / 16;
    static constexpr bool kSwizzle = (kChunksPerRow % 8) == 0;
    static constexpr int kTileBytes = kTile * kRowBytes;
    static constexpr int kStageBytes = 2 * kTileBytes;  // K tile then V tile
    static constexpr int kWarpBytes = kStages * kStageBytes;
    static constexpr int kSmemBytes = kWarps * kWarpBytes;
    static constexpr int kKRounds = D / 32;         // 16-byte K loads per lane and token tile half
    static constexpr int kVRounds = (D + 63) / 64;  // groups of eight n8 output tiles
    static_assert(D % 32 == 0, "head_dim must be a multiple of 32");
    static_assert(kWarpBytes >= (32 + 16 * D) * 4, "merge staging must fit in the warp's ring");
};

__device__ __forceinline__ float2 Unpack2Bf16(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

// K fragments: a phase of 8 lanes reads rows {r, r+1} x 4 adjacent chunks -> flip bit 2 on odd rows.
template <bool kSwizzle>
__device__ __forceinline__ int SwizzleK(int row, int chunk) {
    return kSwizzle ? (chunk ^ ((row & 1) << 2)) : chunk;
}
// V fragments: a phase of 8 lanes reads rows {r, r+2, r+4, r+6} x 2 adjacent chunks.
template <bool kSwizzle>
__device__ __forceinline__ int SwizzleV(int row, int chunk) {
    return kSwizzle ? (chunk ^ (((row >> 1) & 3) << 1)) : chunk;
}

// Tokens one CTA consumes per step: every warp takes one 16-token tile.
constexpr int kSpan = kWarps * kTile;

// Length of sequence b as the kernel sees it (never past the K/V extent / the page table) and the number of
// kSpan-token steps it takes. An empty sequence still counts one (empty) step so that somebody writes its partial.
template <bool kPaged>
__device__ __forceinline__ int64_t SeqLen(const ScaDecodeFwdParams& p, int64_t b) {
    int64_t len = p.seq_lens != nullptr ? static_cast<int64_t>(__ldg(p.seq_lens + b)) : p.seq_kv;
    if (len < 0) len = 0;
    const int64_t cap = kPaged ? p.max_blocks_per_seq * p.block_size : p.seq_kv;
    return len < cap ? len : cap;
}
__device__ __forceinline__ int64_t StepsFor(int64_t len) {
    const int64_t t = (len + kSpan - 1) / kSpan;
    return t > 0 ? t : 1;
}

// One segment = tokens [j_begin, j_end) of one (sequence, kv head, head chunk): streams K/V once, keeps the running
// softmax state of up to 16 query heads, and writes one (m, l, O) partial per head into `slot`.
template <typename T, int D, bool kPaged, bool kHi>
__device__ __forceinline__ void DecodeSegment(const ScaDecodeFwdParams& p, unsigned char* smem, const int64_t b,
                                              const int hk, const int hc, const int64_t j_begin, const int64_t j_end,
                                              const int slot) {
    using G = DecodeGeom<D>;
    constexpr int CPR = G::kChunksPerRow;
    // bf16 keeps 8 bits of a probability: rounding P alone would cost about 1e-3 of relative L2 error in the output.
    // The kernel is bound by HBM, not by the tensor pipe, so P goes into the P V product as two bf16 terms.
    constexpr bool kSplitP = std::is_same<T, __nv_bfloat16>::value;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;  // fragment row / token slot
    const int c = lane & 3;   // fragment column pair
    const int group = static_cast<int>(p.num_heads / p.num_kv_heads);
    const int head0 = hk * group + hc * 16;
    const int nheads = min(16, group - hc * 16);

    const int ntiles = j_end > j_begin ? static_cast<int>((j_end - j_begin + kTile - 1) / kTile) : 0;
    const int my_tiles = ntiles > warp ? (ntiles - warp + kWarps - 1) / kWarps : 0;

    // ---- query fragments (A operand), rows = heads of this chunk -----------------------------
    uint32_t qa[G::kKRounds][2][4];
    {
        const T* q_base = reinterpret_cast<const T*>(p.q) + b * p.q_stride.s_b;
#pragma unroll
        for (int i = 0; i < G::kKRounds; ++i) {
            uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
            if (g < nheads) {
                lo = *reinterpret_cast<const uint4*>(q_base + (head0 + g) * p.q_stride.s_h + 32 * i + 8 * c);
            }
            if (kHi && g + 8 < nheads) {
                hi = *reinterpret_cast<const uint4*>(q_base + (head0 + g + 8) * p.q_stride.s_h + 32 * i + 8 * c);
            }
            qa[i][0][0] = lo.x; qa[i][0][2] = lo.y; qa[i][1][0] = lo.z; qa[i][1][2] = lo.w;
            qa[i][0][1] = hi.x; qa[i][0][3] = hi.y; qa[i][1][1] = hi.z; qa[i][1][3] = hi.w;
        }
    }

    const unsigned char* k_base = reinterpret_cast<const unsigned char*>(p.k) +
                                  ((kPaged ? 0 : b * p.k_stride.s_b) + hk * p.k_stride.s_h) * 2;
    const unsigned char* v_base = reinterpret_cast<const unsigned char*>(p.v) +
                                  ((kPaged ? 0 : b * p.v_stride.s_b) + hk * p.v_stride.s_h) * 2;
    const int64_t k_row_bytes = p.k_stride.s_s * 2;
    const int64_t v_row_bytes = p.v_stride.s_s * 2;
    const int32_t* table_row =
        kPaged ? p.page_table + b * p.max_blocks_per_seq : nullptr;

    unsigned char* ring = smem + warp * G::kWarpBytes;
    const uint32_t ring_addr = SmemAddr(ring);

    // Issues the copies of this warp's `tl`-th tile into `stage`; returns the 16-bit token validity.
    auto issue = [&](int tl, int stage) -> uint32_t {
        const int64_t jt0 = j_begin + static_cast<int64_t>(warp + tl * kWarps) * kTile;
        int prow = -1;  // row of the pool / the K/V slab; pools stay below 2^31 rows
        if (lane < kTile) {
            const int64_t jt = jt0 + lane;
            if (jt < j_end) {
                if (kPaged) {
                    const int64_t logical = jt / p.block_size;
                    if (logical < p.max_blocks_per_seq) {
                        const int32_t phys = __ldg(table_row + logical);
                        if (phys >= 0 && phys < p.num_kv_blocks) {
                            prow = static_cast<int>(phys * p.block_size + jt % p.block_size);
                        }
                    }
                } else {
                    prow = static_cast<int>(jt);
                }
            }
        }
        const uint32_t mask = __ballot_sync(0xffffffffu, prow >= 0) & 0xffffu;
        const uint32_t k_stage = ring_addr + stage * G::kStageBytes;
        const uint32_t v_stage = k_stage + G::kTileBytes;
#pragma unroll
        for (int n = 0; n < (kTile * CPR) / 32; ++n) {
            const int item = lane + 32 * n;
            const int row = item / CPR;
            const int ch = item % CPR;
            const int pr = __shfl_sync(0xffffffffu, prow, row);
            const int bytes = pr >= 0 ? 16 : 0;
            const int64_t r = pr >= 0 ? pr : 0;
            CpAsync16(k_stage + row * G::kRowBytes + SwizzleK<G::kSwizzle>(row, ch) * 16,
                      k_base + r * k_row_bytes + ch * 16, bytes);
            CpAsync16(v_stage + row * G::kRowBytes + SwizzleV<G::kSwizzle>(row, ch) * 16,
                      v_base + r * v_row_bytes + ch * 16, bytes);
        }
        CpAsyncCommit();
        return mask;
    };

    // ---- running state: rows g (index 0) and g + 8 (index 1); scores live in the log2 domain ----
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
    float l_run[2] = {0.0f, 0.0f};
    float o[G::kVRounds][8][4];
#pragma unroll
    for (int r = 0; r < G::kVRounds; ++r)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[r][j][e] = 0.0f;
    const float scale_log2 = p.scale * kLog2e;

    uint32_t mask_queue = 0;
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        uint32_t mk = 0;
        if (s < my_tiles) mk = issue(s, s);
        else CpAsyncCommit();
        mask_queue |= mk << (16 * s);
    }

    int stage = 0;
    for (int tl = 0; tl < my_tiles; ++tl) {
        CpAsyncWait<kStages - 2>();
        __syncwarp();
        {
            const int nt = tl + kStages - 1;
            int nstage = stage + kStages - 1;
            if (nstage >= kStages) nstage -= kStages;
            uint32_t mk = 0;
            if (nt < my_tiles) mk = issue(nt, nstage);
            else CpAsyncCommit();
            const uint32_t cur = mask_queue & 0xffffu;
            mask_queue = (mask_queue >> 16) | (mk << 16);
            if (cur != 0) {
                const uint32_t k_stage = ring_addr + stage * G::kStageBytes;
                const uint32_t v_stage = k_stage + G::kTileBytes;

                // S = Q K^T for 16 tokens: two n8 tiles
                float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int i = 0; i < G::kKRounds; ++i) {
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const int row = 8 * t + g;
                        const uint4 kr = LdsV4(k_stage + row * G::kRowBytes +
                                               SwizzleK<G::kSwizzle>(row, 4 * i + c) * 16);
                        MmaM16N8K16<T>(s[t], qa[i][0][0], qa[i][0][1], qa[i][0][2], qa[i][0][3], kr.x, kr.y);
                        MmaM16N8K16<T>(s[t], qa[i][1][0], qa[i][1][1], qa[i][1][2], qa[i][1][3], kr.z, kr.w);
                    }
                }
                // scale, mask, online softmax
#pragma unroll
                for (int t = 0; t < 2; ++t) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const bool ok = (cur >> (8 * t + 2 * c + (e & 1))) & 1u;
                        s[t][e] = ok ? s[t][e] * scale_log2 : -CUDART_INF_F;
                    }
                }
                uint32_t pa[4], pb[4];
                float alpha[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h == 1 && !kHi) {
                        alpha[1] = 1.0f;
                        pa[1] = 0u;
                        pa[3] = 0u;
                        pb[1] = 0u;
                        pb[3] = 0u;
                        continue;
                    }
                    float mx = fmaxf(fmaxf(s[0][2 * h], s[0][2 * h + 1]), fmaxf(s[1][2 * h], s[1][2 * h + 1]));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                    const float m_new = fmaxf(m_run[h], mx);
                    const float m_safe = (m_new == -CUDART_INF_F) ? 0.0f : m_new;
                    alpha[h] = Exp2(m_run[h] - m_safe);
                    const float p00 = Exp2(s[0][2 * h] - m_safe);
                    const float p01 = Exp2(s[0][2 * h + 1] - m_safe);
                    const float p10 = Exp2(s[1][2 * h] - m_safe);
                    const float p11 = Exp2(s[1][2 * h + 1] - m_safe);
                    l_run[h] = l_run[h] * alpha[h] + (p00 + p01) + (p10 + p11);
                    m_run[h] = m_new;
                    pa[h] = Pack2<T>(p00, p01);      // rows g / g+8, tokens 2c, 2c+1
                    pa[2 + h] = Pack2<T>(p10, p11);  // tokens 8+2c, 8+2c+1
                    if (kSplitP) {
                        // what the 8-bit mantissa dropped, as a second bf16 operand: P = P_hi + P_lo to 2^-16
                        const float2 h0 = Unpack2Bf16(pa[h]), h1 = Unpack2Bf16(pa[2 + h]);
                        pb[h] = Pack2<T>(p00 - h0.x, p01 - h0.y);
                        pb[2 + h] = Pack2<T>(p10 - h1.x, p11 - h1.y);
                    }
                }
                // O = alpha * O + P V
#pragma unroll
                for (int r = 0; r < G::kVRounds; ++r) {
                    const int ch = 8 * r + g;
                    uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0, v2 = v0, v3 = v0;
                    if (ch < CPR) {
                        const int r0 = 2 * c;
                        v0 = LdsV4(v_stage + r0 * G::kRowBytes + SwizzleV<G::kSwizzle>(r0, ch) * 16);
                        v1 = LdsV4(v_stage + (r0 + 1) * G::kRowBytes + SwizzleV<G::kSwizzle>(r0 + 1, ch) * 16);
                        v2 = LdsV4(v_stage + (r0 + 8) * G::kRowBytes + SwizzleV<G::kSwizzle>(r0 + 8, ch) * 16);
                        v3 = LdsV4(v_stage + (r0 + 9) * G::kRowBytes + SwizzleV<G::kSwizzle>(r0 + 9, ch) * 16);
                    }
                    const uint32_t a0[4] = {v0.x, v0.y, v0.z, v0.w};
                    const uint32_t a1[4] = {v1.x, v1.y, v1.z, v1.w};
                    const uint32_t a2[4] = {v2.x, v2.y, v2.z, v2.w};
                    const uint32_t a3[4] = {v3.x, v3.y, v3.z, v3.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                        const uint32_t b0 = __byte_perm(a0[j >> 1], a1[j >> 1], sel);
                        const uint32_t b1 = __byte_perm(a2[j >> 1], a3[j >> 1], sel);
                        o[r][j][0] *= alpha[0];
                        o[r][j][1] *= alpha[0];
                        if (kHi) {
                            o[r][j][2] *= alpha[1];
                            o[r][j][3] *= alpha[1];
                        }
                        MmaM16N8K16<T>(o[r][j], pa[0], pa[1], pa[2], pa[3], b0, b1);
                        if (kSplitP) MmaM16N8K16<T>(o[r][j], pb[0], pb[1], pb[2], pb[3], b0, b1);
                    }
                }
            }
        }
        __syncwarp();
        if (++stage == kStages) stage = 0;
    }
    CpAsyncWait<0>();
    __syncwarp();

    // ---- per-warp results -> this warp's (now idle) ring, then a CTA-wide merge ----------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float* stage_m = reinterpret_cast<float*>(ring);  // [16]
    float* stage_l = stage_m + 16;                    // [16]
    float* stage_o = stage_m + 32;                    // [16][D]
    if (c == 0) {
        stage_m[g] = m_run[0];
        stage_l[g] = l_run[0];
        stage_m[g + 8] = kHi ? m_run[1] : -CUDART_INF_F;
        stage_l[g + 8] = kHi ? l_run[1] : 0.0f;
    }
#pragma unroll
    for (int r = 0; r < G::kVRounds; ++r) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d0 = 64 * r + 16 * c + j;
            const int d1 = d0 + 8;
            if (d0 < D) {
                stage_o[g * D + d0] = o[r][j][0];
                if (kHi) stage_o[(g + 8) * D + d0] = o[r][j][2];
            }
            if (d1 < D) {
                stage_o[g * D + d1] = o[r][j][1];
                if (kHi) stage_o[(g + 8) * D + d1] = o[r][j][3];
            }
        }
    }
    __syncthreads();

    for (int item = threadIdx.x; item < nheads * D; item += kThreads) {
        const int row = item / D;
        const int d = item % D;
        float m_all = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            m_all = fmaxf(m_all, reinterpret_cast<const float*>(smem + w * G::kWarpBytes)[row]);
        }
        float acc = 0.0f, l_all = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float* wm = reinterpret_cast<const float*>(smem + w * G::kWarpBytes);
            const float mw = wm[row];
            if (mw == -CUDART_INF_F) continue;
            const float wgt = Exp2(mw - m_all);
            acc += wm[32 + row * D + d] * wgt;
            l_all += wm[16 + row] * wgt;
        }
        const int64_t flat = (b * p.num_heads + head0 + row) * p.num_splits + slot;
        p.partial_o[flat * D + d] = acc;
        if (d == 0) {
            p.partial_m[flat] = m_all * kLn2;  // stored in natural units like the reference workspace
            p.partial_l[flat] = l_all;
        }
    }
    __syncthreads();  // the rings double as merge staging: nobody refills them before everyone has read
}

// Marks slots [first, num_splits) of every head of one (sequence, kv head, head chunk) as empty (m = -inf; the merge
// skips such entries without reading l or O).
__device__ __forceinline__ void MarkUnusedSlots(const ScaDecodeFwdParams& p, int64_t b, int hk, int hc, int first) {
    const int group = static_cast<int>(p.num_heads / p.num_kv_heads);
    const int head0 = hk * group + hc * 16;
    const int nheads = min(16, group - hc * 16);
    const int unused = static_cast<int>(p.num_splits) - first;
    for (int item = threadIdx.x; item < nheads * unused; item += kThreads) {
        const int row = item / unused;
        const int slot = first + item % unused;
        p.partial_m[(b * p.num_heads + head0 + row) * p.num_splits + slot] = -CUDART_INF_F;
    }
}

// The split-K partial kernel, scheduled for an equal share of the K/V stream per CTA.
//
// The grid is one wave of resident CTAs, a multiple of the number of (kv head, head chunk) columns. CTA c works on
// column c % columns for its whole life; the CTAs of one column split that column's list of kSpan-token steps
// (sequence after sequence) into equal contiguous shares. Neighbouring CTAs therefore read the same tokens of
// neighbouring kv heads at about the same time - in a paged pool those are adjacent 2*D-byte pieces of one token row.
// A share may start and end in the middle of a sequence and may cover several short ones; every piece of a sequence
// a CTA holds is one "segment" and yields one partial. The pieces of one sequence sit in consecutive CTAs of the
// column, so a segment's slot in the [rows, num_splits] partial arrays is the distance to the first CTA that touches
// the sequence. A share is never smaller than longest_sequence / (num_splits - 1) steps, which bounds the pieces of
// any sequence by num_splits (with num_splits == 1 shares are made of whole sequences); slots that stay unused are
// marked empty by the CTA that holds the sequence's first step.
// Sequence lengths are read on the device (seq_lens), so the schedule needs no host knowledge of a ragged batch.
template <typename T, int D, bool kPaged, bool kHi>
__global__ void __launch_bounds__(kThreads)
decode_partial_kernel(const ScaDecodeFwdParams p, const int head_chunks) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int64_t s_part[kWarps][2];
    __shared__ int64_t s_found[2];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int columns = static_cast<int>(p.num_kv_heads) * head_chunks;
    // grids smaller than the number of columns let every CTA walk several columns, each as its only CTA
    const int sharers = gridDim.x >= static_cast<unsigned>(columns) ? static_cast<int>(gridDim.x) / columns : 1;
    const int share = gridDim.x >= static_cast<unsigned>(columns) ? static_cast<int>(blockIdx.x) / columns : 0;
    const int first_column = gridDim.x >= static_cast<unsigned>(columns) ? static_cast<int>(blockIdx.x) % columns
                                                                         : static_cast<int>(blockIdx.x);
    const int column_stride = gridDim.x >= static_cast<unsigned>(columns) ? columns : static_cast<int>(gridDim.x);
    if (share >= sharers) return;  // a grid that is no multiple of the column count

    // ---- this CTA's share [begin, end) of a column's step list, and the sequence that holds `begin` ----------
    int64_t b, before, len, steps, per_cta, begin, end;
    if (p.seq_lens == nullptr) {
        // every sequence has the same length: the list is regular and needs no look at device memory
        len = SeqLen<kPaged>(p, 0);
        steps = StepsFor(len);
        const int64_t total = p.batch * steps;
        per_cta = (total + sharers - 1) / sharers;
        const int64_t floor_steps = p.num_splits > 1 ? (steps + p.num_splits - 2) / (p.num_splits - 1) : total;
        if (per_cta < floor_steps) per_cta = floor_steps;
        if (p.num_splits == 1) per_cta = ((per_cta + steps - 1) / steps) * steps;  // whole sequences only
        begin = share * per_cta;
        if (begin >= total) return;
        end = begin + per_cta < total ? begin + per_cta : total;
        b = begin / steps;
        before = b * steps;
    } else {
        // pass 1: total steps and the longest sequence
        int64_t sum = 0, longest = 0;
        for (int64_t i = threadIdx.x; i < p.batch; i += kThreads) {
            const int64_t t = StepsFor(SeqLen<kPaged>(p, i));
            sum += t;
            longest = t > longest ? t : longest;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const int64_t other = __shfl_xor_sync(0xffffffffu, longest, o);
            longest = other > longest ? other : longest;
        }
        if (lane == 0) {
            s_part[warp][0] = sum;
            s_part[warp][1] = longest;
        }
        __syncthreads();
        sum = 0;
        longest = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            sum += s_part[w][0];
            longest = s_part[w][1] > longest ? s_part[w][1] : longest;
        }
        const int64_t total = sum;
        per_cta = (total + sharers - 1) / sharers;
        // with one slot a share must end where a sequence ends: the whole column then goes to its first CTA
        const int64_t floor_steps = p.num_splits > 1 ? (longest + p.num_splits - 2) / (p.num_splits - 1) : total;
        if (per_cta < floor_steps) per_cta = floor_steps;
        begin = share * per_cta;
        if (begin >= total) return;
        end = begin + per_cta < total ? begin + per_cta : total;

        // pass 2: find i with before[i] <= begin < before[i] + steps[i]
        int64_t running = 0;
        __syncthreads();
        for (int64_t base = 0; base < p.batch && running <= begin; base += kThreads) {
            const int64_t i = base + threadIdx.x;
            const int64_t t = i < p.batch ? StepsFor(SeqLen<kPaged>(p, i)) : 0;
            int64_t incl = t;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int64_t up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            if (lane == 31) s_part[warp][0] = incl;
            __syncthreads();
            int64_t mine = running + incl - t;
            int64_t chunk_total = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                if (w < warp) mine += s_part[w][0];
                chunk_total += s_part[w][0];
            }
            if (t > 0 && mine <= begin && begin < mine + t) {
                s_found[0] = i;
                s_found[1] = mine;
            }
            running += chunk_total;
            __syncthreads();
        }
        b = s_found[0];
        before = s_found[1];  // steps of this column before sequence b
        len = SeqLen<kPaged>(p, b);
        steps = StepsFor(len);
    }
    // the merge kernel that follows on the stream may be set up while this grid streams K/V
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // ---- walk the share segment by segment, in every column this CTA serves -----------------------------
    const int64_t b_first = b, before_first = before, len_first = len, steps_first = steps;
    for (int column = first_column; column < columns; column += column_stride) {
        const int hk = column / head_chunks, hc = column % head_chunks;
        b = b_first;
        before = before_first;
        len = len_first;
        steps = steps_first;
        int64_t pos = begin;
        while (pos < end) {
            const int64_t t0 = pos - before;
            int64_t t1 = t0 + (end - pos);
            if (t1 > steps) t1 = steps;
            const int slot = static_cast<int>(share - before / per_cta);
            if (t0 == 0) {
                const int used = static_cast<int>((before + steps - 1) / per_cta - before / per_cta) + 1;
                MarkUnusedSlots(p, b, hk, hc, used);
            }
            const int64_t j_end = t1 * kSpan < len ? t1 * kSpan : len;
            DecodeSegment<T, D, kPaged, kHi>(p, smem, b, hk, hc, t0 * kSpan, j_end, slot);
            pos += t1 - t0;
            if (t1 == steps && pos < end) {
                before += steps;
                ++b;
                len = SeqLen<kPaged>(p, b);
                steps = StepsFor(len);
            }
        }
    }
}

// Where the parts of one output row live: element (row, part) of m / l is at
// m[row * m_row_stride + part * m_part_stride]; its O vector starts at
// o[row * o_row_stride + part * o_part_stride].
struct MergeSource {
    const float* m;
    const float* l;
    const float* o;
    int64_t m_row_stride, m_part_stride, o_row_stride, o_part_stride;
};

// Max-rescaled merge of `parts` (m, l, O) triples per row (reference: decode_splitk.cu:143-182).
// kTriples == false: out[row] = O / l in T through (heads, o_sb, o_sh); true: writes the merged,
// still unnormalised triple {m, l, O[D]} per row as fp32.
template <typename T, bool kTriples>
__global__ void __launch_bounds__(256)
decode_merge_kernel(const MergeSource src, const int64_t rows, const int parts, const int head_dim,
                    void* __restrict__ out, const int64_t heads, const int64_t o_sb, const int64_t o_sh) {
    // launched with programmatic stream serialisation: the grid may start before the kernel that produces the parts
    // has finished; this returns once that kernel is complete and its writes are visible (a no-op otherwise)
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int64_t total = rows * head_dim;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; item < total;
         item += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = item / head_dim;
        const int d = static_cast<int>(item % head_dim);
        const float* m = src.m + row * src.m_row_stride;
        const float* l = src.l + row * src.m_row_stride;
        const float* o = src.o + row * src.o_row_stride + d;
        float m_all = -CUDART_INF_F;
        for (int s = 0; s < parts; ++s) m_all = fmaxf(m_all, m[s * src.m_part_stride]);
        float l_all = 0.0f, acc = 0.0f;
        for (int s = 0; s < parts; ++s) {
            const float ms = m[s * src.m_part_stride];
            if (ms == -CUDART_INF_F) continue;
            const float wgt = Exp2((ms - m_all) * kLog2e);
            l_all += l[s * src.m_part_stride] * wgt;
            acc += o[s * src.o_part_stride] * wgt;
        }
        if (kTriples) {
            float* t = reinterpret_cast<float*>(out) + row * (2 + head_dim);
            t[2 + d] = acc;
            if (d == 0) {
                t[0] = m_all;
                t[1] = l_all;
            }
        } else {
            const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
            const int64_t b = row / heads;
            const int64_t h = row % heads;
            reinterpret_cast<T*>(out)[b * o_sb + h * o_sh + d] = FromFloat<T>(acc * inv);
        }
    }
}

// Launches the merge kernel. `after_partial`: it directly follows the partial kernel on the same stream, so it is
// launched with programmatic stream serialisation - its blocks are set up while the partial kernel still runs and
// wait inside the kernel (griddepcontrol.wait) until that grid has completed.
template <typename T, bool kTriples>
void LaunchMerge(unsigned blocks, cudaStream_t stream, bool after_partial, const MergeSource& src, int64_t rows, int parts,
                 int head_dim, void* out, int64_t heads, int64_t o_sb, int64_t o_sh) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = after_partial ? 1 : 0;
    cudaLaunchKernelEx(&cfg, decode_merge_kernel<T, kTriples>, src, rows, parts, head_dim, out, heads, o_sb, o_sh);
}

template <typename T, int D, bool kPaged, bool kHi>
int LaunchPartial(const ScaDecodeFwdParams& p, int head_chunks, cudaStream_t stream) {
    using G = DecodeGeom<D>;
    const void* fn = reinterpret_cast<const void*>(&decode_partial_kernel<T, D, kPaged, kHi>);
    if (int rc = EnsureDynamicSmem(fn, G::kSmemBytes, "decode_partial_kernel")) return rc;
    // one wave: as many CTAs as stay resident together, fewer when there is less work than that
    static int resident_per_sm = 0;  // per instantiation; the same on every device of one model
    if (resident_per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_partial_kernel<T, D, kPaged, kHi>, kThreads,
                                                          G::kSmemBytes) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = 1;
        }
        resident_per_sm = n;
    }
    const int64_t columns = p.num_kv_heads * head_chunks;
    const int64_t resident = static_cast<int64_t>(SmCount()) * resident_per_sm;
    const int64_t upper = kPaged ? p.max_blocks_per_seq * p.block_size : p.seq_kv;
    const int64_t steps = std::max<int64_t>(1, (std::min(p.seq_kv, upper) + kSpan - 1) / kSpan);
    // CTAs per column: as many as stay resident, never more than the column has steps (or sequences, with one slot)
    const int64_t useful = p.num_splits == 1 ? p.batch : p.batch * steps;
    int64_t blocks;
    if (resident >= columns) {
        blocks = columns * std::max<int64_t>(1, std::min(resident / columns, useful));
    } else {
        blocks = resident;  // more columns than resident CTAs: every CTA walks several columns
    }
    decode_partial_kernel<T, D, kPaged, kHi>
        <<<static_cast<unsigned>(blocks), kThreads, G::kSmemBytes, stream>>>(p, head_chunks);
    return CheckLaunch("decode_partial_kernel", stream);
}

template <typename T, int D>
int LaunchPartialForDim(const ScaDecodeFwdParams& p, cudaStream_t stream) {
    const int group = static_cast<int>(p.num_heads / p.num_kv_heads);
    const int head_chunks = (group + 15) / 16;
    const bool paged = p.page_table != nullptr;
    const bool hi = group > 8;
    if (paged) {
        return hi ? LaunchPartial<T, D, true, true>(p, head_chunks, stream)
                  : LaunchPartial<T, D, true, false>(p, head_chunks, stream);
    }
    return hi ? LaunchPartial<T, D, false, true>(p, head_chunks, stream)
              : LaunchPartial<T, D, false, false>(p, head_chunks, stream);
}

template <typename T>
int LaunchPartialTyped(const ScaDecodeFwdParams& p, cudaStream_t stream) {
    switch (p.head_dim) {
        case 32: return LaunchPartialForDim<T, 32>(p, stream);
        case 64: return LaunchPartialForDim<T, 64>(p, stream);
        case 96: return LaunchPartialForDim<T, 96>(p, stream);
        case 128: return LaunchPartialForDim<T, 128>(p, stream);
        case 160: return LaunchPartialForDim<T, 160>(p, stream);
        case 192: return LaunchPartialForDim<T, 192>(p, stream);
        case 256: return LaunchPartialForDim<T, 256>(p, stream);
        default: break;
    }
    return Fail(SCA_INVALID_ARGUMENT,
                "decode: head_dim=" + std::to_string(p.head_dim) + " is not instantiated");
}

int ValidateDecode(const ScaDecodeFwdParams* params, bool need_out) {
    if (params == nullptr) return Fail(SCA_INVALID_ARGUMENT, "decode: null parameter block");
    const ScaDecodeFwdParams& p = *params;
    if (p.q == nullptr || p.k == nullptr || p.v == nullptr || (need_out && p.out == nullptr) ||
        p.partial_m == nullptr || p.partial_l == nullptr || p.partial_o == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "decode: null pointer");
    }
    if (p.num_splits < 1) return Fail(SCA_INVALID_ARGUMENT, "decode: num_splits must be >= 1");
    if (p.batch < 1 || p.num_heads < 1 || p.num_kv_heads < 1 || p.num_heads % p.num_kv_heads != 0) {
        return Fail(SCA_INVALID_ARGUMENT,
                    "decode: invalid geometry batch=" + std::to_string(p.batch) + " heads=" +
                        std::to_string(p.num_heads) + " kv_heads=" + std::to_string(p.num_kv_heads));
    }
    if (p.dtype != SCA_DTYPE_F16 && p.dtype != SCA_DTYPE_BF16 && p.dtype != SCA_DTYPE_F32) {
        return Fail(SCA_INVALID_ARGUMENT, "decode: unsupported dtype id");
    }
    if (p.dtype != SCA_DTYPE_F32) {
        // 128-bit loads: 16-byte aligned bases and row starts
        if (!Aligned16(p.q) || !Aligned16(p.k) || !Aligned16(p.v) || p.q_stride.s_b % 8 != 0 ||
            p.q_stride.s_h % 8 != 0 || p.k_stride.s_b % 8 != 0 || p.k_stride.s_h % 8 != 0 ||
            p.k_stride.s_s % 8 != 0 || p.v_stride.s_b % 8 != 0 || p.v_stride.s_h % 8 != 0 ||
            p.v_stride.s_s % 8 != 0) {
            return Fail(SCA_INVALID_ARGUMENT,
                        "decode: q/k/v must be 16-byte aligned with strides that are multiples of 8 elements");
        }
    }
    return SCA_OK;
}

int LaunchMergeOut(const ScaDecodeFwdParams& p, cudaStream_t stream) {
    MergeSource src;
    src.m = p.partial_m;
    src.l = p.partial_l;
    src.o = p.partial_o;
    src.m_row_stride = p.num_splits;
    src.m_part_stride = 1;
    src.o_row_stride = p.num_splits * p.head_dim;
    src.o_part_stride = p.head_dim;
    const int64_t rows = p.batch * p.num_heads;
    const int64_t total = rows * p.head_dim;
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 1 << 20));
    const int parts = static_cast<int>(p.num_splits);
    const int hd = static_cast<int>(p.head_dim);
    switch (p.dtype) {
        case SCA_DTYPE_F16:
            LaunchMerge<__half, false>(blocks, stream, true, src, rows, parts, hd, p.out, p.num_heads, p.o_stride.s_b, p.o_stride.s_h);
            break;
        case SCA_DTYPE_BF16:
            LaunchMerge<__nv_bfloat16, false>(blocks, stream, true, src, rows, parts, hd, p.out, p.num_heads, p.o_stride.s_b, p.o_stride.s_h);
            break;
        default:
            LaunchMerge<float, false>(blocks, stream, true, src, rows, parts, hd, p.out, p.num_heads, p.o_stride.s_b, p.o_stride.s_h);
            break;
    }
    return CheckLaunch("decode_merge_kernel", stream);
}

}  // namespace

// fp32 inputs take the SIMT partial kernel (simt.cu); declared here, defined there.
int LaunchDecodePartialF32(const ScaDecodeFwdParams& p, cudaStream_t stream);

int LaunchDecodePartials(const ScaDecodeFwdParams& p, cudaStream_t stream) {
    switch (p.dtype) {
        case SCA_DTYPE_F16: return LaunchPartialTyped<__half>(p, stream);
        case SCA_DTYPE_BF16: return LaunchPartialTyped<__nv_bfloat16>(p, stream);
        case SCA_DTYPE_F32: return LaunchDecodePartialF32(p, stream);
        default: break;
    }
    return Fail(SCA_INVALID_ARGUMENT, "decode: unsupported dtype id");
}

}  // namespace sca_b200

// ---- allocation-free variant ---------------------------------------------------------------------
// Split-K partials for callers that must not allocate device memory live in this fixed array. Every
// GPU that loads the library carries it until the process exits. In host code the name below is only
// a host-side stand-in for the symbol, never a device address: the address a kernel may use comes
// from cudaGetSymbolAddress, looked up once per device with that device current.
namespace sca_b200 {
namespace {

constexpr int64_t kStaticScratchFloats = int64_t{4} << 20;  // 4 Mi floats = 16 MiB per GPU
static __device__ __align__(256) float g_decode_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mutex;
float* g_static_scratch_ptr[kMaxDevices] = {};

// Device address of the static scratch on the current device (looked up on first use per device).
int StaticScratchFor(float** out) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return FailCuda(err, "decode (static scratch): cudaGetDevice");
    if (device < 0 || device >= kMaxDevices) {
        return Fail(SCA_INVALID_ARGUMENT, "decode (static scratch): device index " + std::to_string(device) + " is out of range");
    }
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[device] == nullptr) {
        float* ptr = nullptr;
        err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_decode_static_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return FailCuda(err, "decode (static scratch): cudaGetSymbolAddress");
        }
        g_static_scratch_ptr[device] = ptr;
    }
    *out = g_static_scratch_ptr[device];
    return SCA_OK;
}

}  // namespace
}  // namespace sca_b200

using namespace sca_b200;

extern "C" int sca_launch_decode_splitk(const ScaDecodeFwdParams* params, void* stream) {
    ClearError();
    if (int rc = ValidateDecode(params, true)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (int rc = LaunchDecodePartials(*params, s)) return rc;
    return LaunchMergeOut(*params, s);
}

extern "C" int sca_launch_decode_splitk_paged(const ScaDecodeFwdParams* params, void* stream) {
    ClearError();
    if (params == nullptr) return Fail(SCA_INVALID_ARGUMENT, "paged attention: null parameter block");
    if (params->page_table == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT,
                    "paged attention: page_table is null (use the contiguous entry point instead)");
    }
    if (params->block_size <= 0 || params->max_blocks_per_seq <= 0 || params->num_kv_blocks <= 0) {
        return Fail(SCA_INVALID_ARGUMENT,
                    "paged attention: block_size/max_blocks_per_seq/num_kv_blocks must be positive");
    }
    return sca_launch_decode_splitk(params, stream);
}

extern "C" int sca_launch_paged_attention_ordered(const ScaPagedDecodeParams* params,
                                                  const int32_t* seq_order, void* stream) {
    ClearError();
    if (params == nullptr || params->page_table == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "paged attention: null page table");
    }
    ScaDecodeFwdParams p = params->base;
    p.page_table = params->page_table;
    p.block_size = params->block_size;
    p.max_blocks_per_seq = params->max_blocks_per_seq;
    p.num_kv_blocks = params->num_kv_blocks;
    if (p.block_size <= 0 || p.max_blocks_per_seq <= 0 || p.num_kv_blocks <= 0) {
        return Fail(SCA_INVALID_ARGUMENT,
                    "paged attention: block_size/max_blocks_per_seq/num_kv_blocks must be positive");
    }
    if (int rc = ValidateDecode(&p, true)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    (void)seq_order;  // the kernel deals out equal shares of the K/V stream itself; the hint has nothing left to improve
    if (int rc = LaunchDecodePartials(p, s)) return rc;
    return LaunchMergeOut(p, s);
}

extern "C" int sca_launch_paged_attention(const ScaPagedDecodeParams* params, void* stream) {
    return sca_launch_paged_attention_ordered(params, nullptr, stream);
}

// Partial kernel only: fills partial_m / partial_l / partial_o; the caller merges (sca_launch_seqsplit_exchange).
extern "C" int sca_launch_decode_partials(const ScaDecodeFwdParams* params, void* stream) {
    ClearError();
    if (int rc = ValidateDecode(params, false)) return rc;
    return LaunchDecodePartials(*params, static_cast<cudaStream_t>(stream));
}

extern "C" int sca_launch_decode_triples(const ScaDecodeFwdParams* params, float* triples, void* stream) {
    ClearError();
    if (int rc = ValidateDecode(params, false)) return rc;
    if (triples == nullptr) return Fail(SCA_INVALID_ARGUMENT, "decode triples: null output");
    const ScaDecodeFwdParams& p = *params;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (int rc = LaunchDecodePartials(p, s)) return rc;
    MergeSource src;
    src.m = p.partial_m;
    src.l = p.partial_l;
    src.o = p.partial_o;
    src.m_row_stride = p.num_splits;
    src.m_part_stride = 1;
    src.o_row_stride = p.num_splits * p.head_dim;
    src.o_part_stride = p.head_dim;
    const int64_t rows = p.batch * p.num_heads;
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((rows * p.head_dim + 255) / 256, 1 << 20));
    LaunchMerge<float, true>(blocks, s, true, src, rows, static_cast<int>(p.num_splits), static_cast<int>(p.head_dim), triples, 1, 0, 0);
    return CheckLaunch("decode_merge_kernel(triples)", s);
}

extern "C" int sca_launch_merge_triples(const float* gathered, int64_t ranks, int64_t rows,
                                        int64_t head_dim, void* out, int32_t out_dtype, void* stream) {
    ClearError();
    if (gathered == nullptr || out == nullptr) return Fail(SCA_INVALID_ARGUMENT, "merge triples: null pointer");
    if (ranks < 1 || rows < 1 || head_dim < 1) {
        return Fail(SCA_INVALID_ARGUMENT, "merge triples: ranks/rows/head_dim must be positive");
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MergeSource src;
    src.m = gathered;
    src.l = gathered + 1;
    src.o = gathered + 2;
    src.m_row_stride = 2 + head_dim;
    src.m_part_stride = rows * (2 + head_dim);
    src.o_row_stride = 2 + head_dim;
    src.o_part_stride = rows * (2 + head_dim);
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((rows * head_dim + 255) / 256, 1 << 20));
    const int parts = static_cast<int>(ranks);
    const int hd = static_cast<int>(head_dim);
    // rows are written densely: [rows, head_dim]
    switch (out_dtype) {
        case SCA_DTYPE_F16:
            LaunchMerge<__half, false>(blocks, s, false, src, rows, parts, hd, out, 1, head_dim, 0);
            break;
        case SCA_DTYPE_BF16:
            LaunchMerge<__nv_bfloat16, false>(blocks, s, false, src, rows, parts, hd, out, 1, head_dim, 0);
            break;
        case SCA_DTYPE_F32:
            LaunchMerge<float, false>(blocks, s, false, src, rows, parts, hd, out, 1, head_dim, 0);
            break;
        default: return Fail(SCA_INVALID_ARGUMENT, "merge triples: unsupported dtype id");
    }
    return CheckLaunch("decode_merge_kernel(ranks)", s);
}

// Allocation-free split-K decode: same kernels and same result as sca_launch_decode_splitk, with the
// partials kept in the library's fixed 16 MiB device array instead of caller-provided scratch.
extern "C" int sca_launch_decode_splitk_static(const ScaDecodeFwdParams* params, void* stream) {
    ClearError();
    if (params == nullptr) return Fail(SCA_INVALID_ARGUMENT, "decode: null parameter block");
    ScaDecodeFwdParams p = *params;
    if (p.batch < 1 || p.num_heads < 1 || p.num_splits < 1 || p.head_dim < 1) {
        return Fail(SCA_INVALID_ARGUMENT, "decode (static scratch): batch/heads/num_splits/head_dim must be positive");
    }
    const int64_t base = p.batch * p.num_heads * p.num_splits;
    const int64_t need = base * (2 + p.head_dim);
    if (base > kStaticScratchFloats || need > kStaticScratchFloats) {
        return Fail(SCA_INVALID_ARGUMENT,
                    "decode (static scratch): batch*heads*num_splits*(2+head_dim) = " + std::to_string(need) +
                        " floats exceeds the built-in scratch of " + std::to_string(kStaticScratchFloats) +
                        " floats; use fewer splits or the entry point that takes caller scratch");
    }
    float* scratch = nullptr;
    if (int rc = StaticScratchFor(&scratch)) return rc;
    p.partial_m = scratch;
    p.partial_l = scratch + base;
    p.partial_o = scratch + 2 * base;
    if (int rc = ValidateDecode(&p, true)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (int rc = LaunchDecodePartials(p, s)) return rc;
    return LaunchMergeOut(p, s);
}
