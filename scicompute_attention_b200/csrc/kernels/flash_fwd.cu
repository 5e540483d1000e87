// Flash prefill for sm_100a: O = softmax(scale * Q K^T + mask) V with the score matrix kept on chip.
//
// Stands in for the reference's flash_fwd_kernel (src/backends/flash/flash_fwd_impl.cuh:45-279, an
// sm_80 mma.sync + ldmatrix + cp.async design with 64x64 tiles and one CTA-wide barrier pair per
// tile). Same arithmetic contract - fp16/bf16 inputs, fp32 accumulation, online softmax through
// exp2, bottom-right aligned causal mask, GQA, optional log-sum-exp - on a Blackwell execution plan:
//
//   * one persistent CTA per SM walks a list of work items; an item is 256 query rows of one
//     (batch, head): two 128-row tiles that ping-pong, so the tensor core works on one tile while
//     the other tile's softmax runs;
//   * warp 0 is the TMA producer: Q tiles once, then K_j, V_j, K_j+1, ... into a ring of 128-byte
//     swizzled shared-memory slots, each guarded by a full/empty mbarrier pair. Loads are plain
//     per-CTA tensor loads (one CTA, one destination); K/V reuse between the CTAs of a kv head comes
//     from L2. Rows past the end of a sequence are zero-filled by the TMA unit;
//   * warp 1 issues every tcgen05.mma from one thread: S_t = Q_t K_j^T (both operands in shared
//     memory, K-major) into tensor memory, and O_t += P_t V_j with P_t read from tensor memory and
//     V_j as an MN-major shared-memory operand (no transposition of V anywhere);
//   * warps 4-7 and 8-11 are the two softmax groups, one thread per query row: they read their S row
//     from tensor memory once, 64 columns at a time, exponentiate against the reference point the
//     row already has, keep the running sum in registers and write P back over S as packed 16-bit
//     values. The reference point moves (and O, the sum and the part of P already written are
//     rescaled) only when a half-row exceeds it by more than 2^8; the final division by the row sum
//     absorbs the stale reference point exactly;
//   * tensor memory: S_0 | S_1 | O_0 | O_1, 128 (or D) fp32 columns each, 512 columns in total;
//   * head dims above 128 leave room for one query tile only (O needs 256 columns). There the scores of
//     64-key tiles are double-buffered instead: S(j+1) is computed while the softmax of tile j runs, and
//     S(j+2) follows P(j) V_j into the buffer P(j) came from.
//
// Packed variable-length batches run on the same kernel: the work list then holds (sequence, query block)
// entries and every item carries its sequence's lengths and token offsets (see sca_launch_flash_varlen).
//
// Every wait on an mbarrier is bounded (sm100.cuh): on expiry the role raises a CTA-wide abort flag,
// the kernel records a code in a host-visible word, frees its tensor memory and returns.
//
// FLOPs per (query, key) pair that is visible: 4 * D. Algorithmic HBM bytes: Q + K + V + O once.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <type_traits>
#include <vector>

#include "common.cuh"
#include "sm100.cuh"

namespace sca_b200 {
namespace {

using namespace sm100;

constexpr int kBlockM = 128;

// Two fp32 lanes per instruction (sm_100 packed arithmetic): halves the issue slots of the scale-and-shift and of
// the row-sum accumulation in the softmax, which is issue-bound.
__device__ __forceinline__ float2 Fma2(float2 a, float2 b, float2 c) {
    uint64_t ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 Add2(float2 a, float2 b) {
    uint64_t ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

template <typename T>
__device__ __forceinline__ float2 Unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 Unpack2<__nv_bfloat16>(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 Unpack2<__half>(uint32_t v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
// bf16 inputs: the probabilities are handed to the P V product as fp16, not bf16. They lie in [0, 2^8], where fp16
// resolves 2^-11 relative against 2^-8 - with bf16 the rounding of P alone costs about 1e-3 of relative L2 error in
// the output. The tensor core wants both operands of one product in the same 16-bit format (a descriptor that mixes
// them raises "illegal instruction" on sm_100a), so for bf16 inputs a small kernel first rewrites V as fp16 into a
// stream-ordered temporary (values beyond the fp16 range saturate) and the prefill kernel reads V from there.
// (Rewriting the V tiles in shared memory by the two idle warps was measured too: 7 % slower than this, because
// the extra instructions land on two of the four schedulers the softmax warps run on.)
template <typename T>
struct PvFormat {
    using type = __half;
    static constexpr bool kConvertV = std::is_same<T, __nv_bfloat16>::value;
};
constexpr int kFlashThreads = 384;   // warp 0 TMA, 1 MMA, 2 TMEM owner, 3 idle, 4-7 / 8-11 softmax
constexpr int kTmemColumns = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 domain: P stays <= 2^8

// DP: padded head dim (64 / 128 / 256); QT: query tiles per CTA; BN: keys per KV tile.
// 64 and 128 run two query tiles against 128-key tiles; 256 needs 256 TMEM columns for O, so it runs one
// query tile against 64-key tiles (S 64 + O 256 columns).
template <int DP, int QT, int BN>
struct FlashGeom {
    static constexpr int kKBlocks = DP / 64;               // 64-element (128-byte) column blocks per row
    static constexpr int kQBlockBytes = kBlockM * 128;      // one column block of a query tile
    static constexpr int kKvBlockBytes = BN * 128;          // one column block of a K or V tile
    static constexpr int kQTileBytes = kKBlocks * kQBlockBytes;
    static constexpr int kKvTileBytes = kKBlocks * kKvBlockBytes;
    static constexpr int kSlots = (DP == 64) ? 8 : 5;  // K/V ring
    static constexpr int kBarrierBytes = 384;
    static constexpr int kSmemBytes = 1024 + QT * kQTileBytes + kSlots * kKvTileBytes + kBarrierBytes;
    static constexpr int kSCol = 0;                         // S_t at kSCol + t * 128
    static constexpr int kOCol = 256;                       // O_t at kOCol + t * DP
    static_assert((DP == 64 || DP == 128) ? (QT == 2 && BN == 128) : (DP == 256 && QT == 1 && BN == 64), "geometry");
    static_assert(kOCol + QT * DP <= kTmemColumns, "tensor memory budget");
    static_assert(kSmemBytes <= 232448, "exceeds the 227 KiB per-CTA limit");
};

struct FlashKernelParams {
    void* out;
    float* lse;
    int* error_word; // host-visible; non-zero after a wait expired
    int seq_q, seq_kv, heads, kv_heads, head_dim, batch;
    int64_t o_sb, o_sh, o_ss;
    float scale_log2;
    int causal;
    int diagonal;
    int m_blocks;
    // packed variable-length batches (null for dense [B, H, S, D] problems): seqs[s] = {first query token,
    // first key token, S_q, S_kv}; entries[e] = {sequence, query block}, heaviest first
    const int4* seqs;
    const int2* entries;
    int num_entries;
    // paged K/V (kPaged kernels): the K/V tensor maps cover one layer's pool viewed as [blocks * block_size, H_kv, D]
    // with a box of block_size rows; a KV tile is assembled page by page through the sequence's page-table row
    const int32_t* page_table;   // device [num_seqs, max_blocks_per_seq], -1 = unmapped
    int max_blocks_per_seq, num_kv_blocks;
    int block_size, block_shift;  // block_size = 1 << block_shift
};

// KV tiles a query tile starting at row m0 of its sequence has to visit.
template <int BN>
__device__ __forceinline__ int TilesFor(int m0, int seq_q, int seq_kv, int causal, int diagonal) {
    if (m0 >= seq_q) return 0;
    int64_t limit = seq_kv;
    if (causal) limit = min(limit, static_cast<int64_t>(m0) + kBlockM + diagonal);
    if (limit <= 0) return 0;
    return static_cast<int>((limit + BN - 1) / BN);
}

// kVarlen: the work list comes from the (sequence, query block) table of a packed ragged batch; otherwise it is
// computed from the dense [B, H, S, D] geometry and every per-sequence quantity is a launch constant.
// kPaged (only with kVarlen): K and V of a sequence are scattered over the pages of a KV pool.
template <typename T, int DP, int QT, int BN, bool kVarlen, bool kPaged = false>
__global__ void __launch_bounds__(kFlashThreads, 1)
flash_fwd_sm100_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const FlashKernelParams p) {
    using G = FlashGeom<DP, QT, BN>;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t smem_base = (SmemAddr(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (smem_base - SmemAddr(smem_raw));

    const uint32_t q_smem = smem_base;
    const uint32_t ring_smem = smem_base + QT * G::kQTileBytes;
    const uint32_t bar_base = ring_smem + G::kSlots * G::kKvTileBytes;
    auto bar = [&](int i) { return bar_base + 8u * i; };
    // barrier indices
    constexpr int kQFull = 0;                       // [2]
    constexpr int kKvFull = 2;                      // [kSlots]
    constexpr int kKvEmpty = kKvFull + G::kSlots;   // [kSlots]
    constexpr int kSFull = kKvEmpty + G::kSlots;    // [2]
    constexpr int kPFull = kSFull + 2;              // [2]
    constexpr int kODone = kPFull + 2;              // [2]
    constexpr int kQEmpty = kODone + 2;             // [2]
    constexpr int kOFree = kQEmpty + 2;             // [2]
    constexpr int kVReady = kOFree + 2;             // [kSlots] paged bf16: V tile rewritten as fp16 in place
    constexpr int kNumBars = kVReady + G::kSlots;
    // P and V enter the P V product as fp16 also for bf16 inputs (PvFormat). Contiguous V comes from an fp16 copy made
    // before the launch; the pages of a pool are rewritten tile by tile in shared memory by warps 2 and 3 instead
    // (a copy of the pool would cost more than the prefill), at the price of some issue slots of two schedulers.
    using PT = typename PvFormat<T>::type;
    constexpr bool kCvtInKernel = kPaged && PvFormat<T>::kConvertV;
    constexpr int kConverterThreads = 64;
    static_assert(!kPaged || kVarlen, "paged K/V runs on the packed work list");
    static_assert(kNumBars * 8 + 16 <= G::kBarrierBytes, "barrier area too small");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + (bar_base - smem_base) + kNumBars * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // paged K/V: which pages of a KV tile are mapped (bit i = i-th page of the tile), written by the producer when
    // it loads the K tile and read by the softmax groups; indexed by the CTA's running KV-tile count
    constexpr int kValidRing = 16;
    volatile uint32_t* valid_ring = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);
    static_assert(kNumBars * 8 + 8 + kValidRing * 4 <= G::kBarrierBytes, "barrier area too small");

    // One query tile per CTA (head dims above 128): no second tile to ping-pong with, so the scores are double-
    // buffered instead: S(j+1) is computed while the softmax of block j runs. The barriers s_full / p_full / o_done
    // are then indexed by the score buffer j & 1 instead of by the query tile.
    constexpr bool kDoubleS = (QT == 1);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // ---- work items: (query block, batch*head), heaviest causal blocks first. The list is dealt to the
    // CTAs in rounds of gridDim.x items, every other round in reverse CTA order, so that the CTA that got
    // the heaviest item of one round gets the lightest of the next (the static schedule then ends within
    // about one KV tile of each other on all SMs). Every role of a CTA walks the same sequence. ----------
    const int bh_count = p.batch * p.heads;
    const int total_items = kVarlen ? p.num_entries * p.heads : p.m_blocks * bh_count;
    struct Item {
        int b, h, h_kv;
        int seq;                      // index of the sequence (row of the page table); 0 for dense problems
        int q_tok0, kv_tok0;          // first row of the sequence in the packed tensors (0 for dense problems)
        int seq_q, seq_kv, diagonal;  // of this item's sequence
        int m0[2];                    // first query row of each tile, relative to the sequence
        int ntiles[2];
        int n_max;
    };
    auto decode_item = [&](int idx) {
        Item w;
        int mb;
        if constexpr (kVarlen) {
            const int2 entry = __ldg(p.entries + idx / p.heads);
            const int4 seq = __ldg(p.seqs + entry.x);
            mb = entry.y;
            w.seq = entry.x;
            w.b = 0;
            w.h = idx % p.heads;
            w.q_tok0 = seq.x;
            w.kv_tok0 = seq.y;
            w.seq_q = seq.z;
            w.seq_kv = seq.w;
            w.diagonal = p.causal ? seq.w - seq.z : 0;  // bottom-right aligned mask
        } else {
            mb = p.m_blocks - 1 - idx / bh_count;
            w.seq = 0;
            const int bh = idx % bh_count;
            w.b = bh / p.heads;
            w.h = bh % p.heads;
            w.q_tok0 = 0;
            w.kv_tok0 = 0;
            w.seq_q = p.seq_q;
            w.seq_kv = p.seq_kv;
            w.diagonal = p.diagonal;
        }
        w.h_kv = w.h / (p.heads / p.kv_heads);
        w.m0[0] = (mb * QT) * kBlockM;
        w.m0[1] = (mb * QT + 1) * kBlockM;
        w.ntiles[0] = TilesFor<BN>(w.m0[0], w.seq_q, w.seq_kv, p.causal, w.diagonal);
        w.ntiles[1] = QT > 1 ? TilesFor<BN>(w.m0[1], w.seq_q, w.seq_kv, p.causal, w.diagonal) : 0;
        w.n_max = max(w.ntiles[0], w.ntiles[1]);
        return w;
    };
    const int rounds = (total_items + gridDim.x - 1) / gridDim.x;
    auto item_of_round = [&](int r) {  // -1: this CTA has no item in round r (only in the last, partial round)
        const int pos = (r & 1) ? static_cast<int>(gridDim.x - 1 - blockIdx.x) : static_cast<int>(blockIdx.x);
        const int idx = r * static_cast<int>(gridDim.x) + pos;
        return idx < total_items ? idx : -1;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            MbarInit(bar(kQFull + i), 1);
            MbarInit(bar(kQEmpty + i), 1);
            MbarInit(bar(kSFull + i), 1);
            MbarInit(bar(kPFull + i), 128);
            MbarInit(bar(kODone + i), 1);
            MbarInit(bar(kOFree + i), 128);
        }
        for (int i = 0; i < G::kSlots; ++i) {
            MbarInit(bar(kKvFull + i), 1);
            MbarInit(bar(kKvEmpty + i), 1);
            MbarInit(bar(kVReady + i), kConverterThreads);
        }
        *abort_flag = 0;
        FenceBarrierInit();
    }
    if (warp == 2) {
        TmemAlloc(SmemAddr(tmem_slot), kTmemColumns);
        TmemRelinquish();
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmem_base = *tmem_slot;

    bool failed = false;

    if (warp == 0 && kPaged) {
        // ================================ TMA producer, paged K/V ===================================
        // The whole warp walks the work list: the lanes fetch the page ids of a tile together (one coalesced read
        // of the table row), lane 0 waits for the ring slot and issues one box load per page and column block. A
        // page that is unmapped (entry < 0 or >= num_kv_blocks) is loaded from beyond the pool, i.e. zero-filled,
        // and its columns are masked in the softmax through valid_ring.
        if (lane == 0) {
            PrefetchTensorMap(&map_q);
            PrefetchTensorMap(&map_k);
            PrefetchTensorMap(&map_v);
        }
        uint32_t q_uses[2] = {0, 0};
        uint32_t kv_loads = 0;
        uint32_t tiles_before = 0;  // KV tiles of the items this CTA has finished
        const int pages_per_tile = BN >> p.block_shift;
        const int page_bytes = p.block_size * 128;  // one page inside one 64-element column block
        bool ok = true;
        for (int r = 0; r < rounds && ok; ++r) {
            const int idx = item_of_round(r);
            if (idx < 0) continue;
            const Item w = decode_item(idx);
            if (lane == 0) {
                for (int t = 0; t < QT && ok; ++t) {
                    if (w.ntiles[t] == 0) continue;
                    if (q_uses[t] > 0) ok = MbarWait(bar(kQEmpty + t), (q_uses[t] - 1) & 1u, abort_flag);
                    if (!ok) break;
                    MbarExpectTx(bar(kQFull + t), G::kQTileBytes);
                    for (int kb = 0; kb < G::kKBlocks; ++kb) {
                        TmaLoad4D(q_smem + t * G::kQTileBytes + kb * G::kQBlockBytes, &map_q, bar(kQFull + t), kb * 64,
                                  w.q_tok0 + w.m0[t], w.h, w.b);
                    }
                    ++q_uses[t];
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            const int32_t* row = p.page_table + static_cast<int64_t>(w.seq) * p.max_blocks_per_seq;
            for (int it = 0; it < 2 * w.n_max && ok; ++it, ++kv_loads) {
                bool is_v;
                int tile;
                if (kDoubleS) {
                    const int n = w.n_max;
                    const int lead = n > 1 ? 2 : 1;
                    if (it < lead) {
                        is_v = false;
                        tile = it;
                    } else {
                        const int f = it - lead, kk = n - lead;
                        is_v = f >= 2 * kk || (f & 1) == 0;
                        tile = f < 2 * kk ? (is_v ? (f >> 1) : (f >> 1) + 2) : kk + (f - 2 * kk);
                    }
                } else {
                    is_v = (it & 1) != 0;
                    tile = it >> 1;
                }
                // page ids of this tile, one per lane
                const int logical = tile * pages_per_tile + lane;
                int32_t phys = -1;
                if (lane < pages_per_tile && logical < p.max_blocks_per_seq &&
                    (static_cast<int64_t>(logical) << p.block_shift) < w.seq_kv) {
                    phys = __ldg(row + logical);
                }
                const bool mapped = phys >= 0 && phys < p.num_kv_blocks;
                const uint32_t valid = __ballot_sync(0xffffffffu, mapped);
                const uint32_t slot = kv_loads % G::kSlots;
                const uint32_t phase = (kv_loads / G::kSlots) & 1u;
                if (lane == 0) {
                    ok = MbarWait(bar(kKvEmpty + slot), phase ^ 1u, abort_flag);
                    if (ok) {
                        if (!is_v) valid_ring[(tiles_before + tile) % kValidRing] = valid;
                        MbarExpectTx(bar(kKvFull + slot), G::kKvTileBytes);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                const CUtensorMap* map = is_v ? &map_v : &map_k;
                for (int pg = 0; pg < pages_per_tile; ++pg) {
                    const int32_t id = __shfl_sync(0xffffffffu, phys, pg);
                    // an unmapped page reads from the first row behind the pool: all zeros
                    const int first_row = ((valid >> pg) & 1u) ? (id << p.block_shift) : (p.num_kv_blocks << p.block_shift);
                    if (lane == 0) {
                        for (int kb = 0; kb < G::kKBlocks; ++kb) {
                            TmaLoad4D(ring_smem + slot * G::kKvTileBytes + kb * G::kKvBlockBytes + pg * page_bytes, map,
                                      bar(kKvFull + slot), kb * 64, first_row, w.h_kv, 0);
                        }
                    }
                }
            }
            tiles_before += static_cast<uint32_t>(w.n_max);
        }
        failed = !ok;
    } else if (warp == 0) {
        // ================================ TMA producer =============================================
        if (lane == 0) {
            PrefetchTensorMap(&map_q);
            PrefetchTensorMap(&map_k);
            PrefetchTensorMap(&map_v);
            uint32_t q_uses[2] = {0, 0};   // how often each query buffer has been filled so far
            uint32_t kv_loads = 0;         // K/V tiles loaded so far (ring position)
            bool ok = true;
            for (int r = 0; r < rounds && ok; ++r) {
                const int idx = item_of_round(r);
                if (idx < 0) continue;
                const Item w = decode_item(idx);
                for (int t = 0; t < QT && ok; ++t) {
                    if (w.ntiles[t] == 0) continue;
                    // the previous item's last S = Q K^T must have read the buffer
                    if (q_uses[t] > 0) ok = MbarWait(bar(kQEmpty + t), (q_uses[t] - 1) & 1u, abort_flag);
                    if (!ok) break;
                    MbarExpectTx(bar(kQFull + t), G::kQTileBytes);
                    for (int kb = 0; kb < G::kKBlocks; ++kb) {
                        TmaLoad4D(q_smem + t * G::kQTileBytes + kb * G::kQBlockBytes, &map_q, bar(kQFull + t), kb * 64,
                                  w.q_tok0 + w.m0[t], w.h, w.b);
                    }
                    ++q_uses[t];
                }
                // ring order = the order the MMA stream consumes the tiles: K_0 V_0 K_1 V_1 ..., or with double-
                // buffered scores K_0 K_1 V_0 K_2 V_1 K_3 ... (S(j+2) follows P(j) V_j)
                for (int it = 0; it < 2 * w.n_max && ok; ++it, ++kv_loads) {
                    bool is_v;
                    int tile;
                    if (kDoubleS) {
                        const int n = w.n_max;
                        const int lead = n > 1 ? 2 : 1;
                        if (it < lead) {
                            is_v = false;
                            tile = it;
                        } else {
                            const int f = it - lead, kk = n - lead;  // kk K tiles still to come, one after each V
                            is_v = f >= 2 * kk || (f & 1) == 0;
                            tile = f < 2 * kk ? (is_v ? (f >> 1) : (f >> 1) + 2) : kk + (f - 2 * kk);
                        }
                    } else {
                        is_v = (it & 1) != 0;
                        tile = it >> 1;
                    }
                    const uint32_t slot = kv_loads % G::kSlots;
                    const uint32_t phase = (kv_loads / G::kSlots) & 1u;
                    ok = MbarWait(bar(kKvEmpty + slot), phase ^ 1u, abort_flag);
                    if (!ok) break;
                    MbarExpectTx(bar(kKvFull + slot), G::kKvTileBytes);
                    const CUtensorMap* map = is_v ? &map_v : &map_k;
                    for (int kb = 0; kb < G::kKBlocks; ++kb) {
                        TmaLoad4D(ring_smem + slot * G::kKvTileBytes + kb * G::kKvBlockBytes, map, bar(kKvFull + slot),
                                  kb * 64, w.kv_tok0 + tile * BN, w.h_kv, w.b);
                    }
                }
            }
            failed = !ok;
        }
    } else if (warp == 1) {
        // ================================ MMA issuer ================================================
        if (lane == 0) {
            constexpr uint32_t fmt = std::is_same<T, __half>::value ? kFmtF16 : kFmtBf16;
            constexpr uint32_t idesc_s = MakeInstrDesc(fmt, fmt, 0, 0, kBlockM, BN);  // Q K^T: both K-major
            // P V: V is MN-major; both operands in the P V format (fp16 also for bf16 inputs, see PvFormat: V then
            // comes from the fp16 copy map_v points at)
            constexpr uint32_t fmt_pv = PvFormat<T>::kConvertV ? kFmtF16 : fmt;
            constexpr uint32_t idesc_o = MakeInstrDesc(fmt_pv, fmt_pv, 0, 1, kBlockM, DP);
            // Descriptors are built once and advanced by compile-time constants, so that issuing one
            // tcgen05.mma costs a handful of instructions (this thread alone has to keep the tensor pipe fed).
            const uint64_t kmajor_hi = MakeSmemDesc(0, 16, 1024);                 // K-major operands (Q and K)
            const uint64_t vmajor_hi = MakeSmemDesc(0, G::kKvBlockBytes, 1024);   // MN-major operand (V)
            const uint64_t q_desc[2] = {kmajor_hi | (q_smem >> 4), kmajor_hi | ((q_smem + G::kQTileBytes) >> 4)};
            const uint32_t s_tmem[2] = {tmem_base + G::kSCol, tmem_base + G::kSCol + 128};
            uint32_t s_tmem_db = tmem_base + G::kSCol;  // current score buffer when the scores are double-buffered
            const uint32_t o_tmem[2] = {tmem_base + G::kOCol, tmem_base + G::kOCol + DP};
            auto issue_s = [&](int t, uint32_t slot) {
                const uint64_t a0 = q_desc[t];
                const uint64_t b0 = kmajor_hi | ((ring_smem + slot * G::kKvTileBytes) >> 4);
#pragma unroll
                for (int ks = 0; ks < DP / 16; ++ks) {
                    constexpr int kStep = 32 >> 4;  // 16 elements = 32 bytes inside a 128-byte swizzle row
                    const uint32_t qa = ((ks >> 2) * G::kQBlockBytes >> 4) + (ks & 3) * kStep;
                    const uint32_t kb = ((ks >> 2) * G::kKvBlockBytes >> 4) + (ks & 3) * kStep;
                    const uint32_t d = kDoubleS ? s_tmem_db : s_tmem[t];
                    if (ks == 0) MmaSS<false>(d, a0 + qa, b0 + kb, idesc_s);
                    else MmaSS<true>(d, a0 + qa, b0 + kb, idesc_s);
                }
            };
            auto issue_pv = [&](int t, uint32_t slot, bool first) {
                const uint64_t b0 = vmajor_hi | ((ring_smem + slot * G::kKvTileBytes) >> 4);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    // 16 keys further: 8 packed P columns in tensor memory, 16 rows (2048 bytes) of V
                    const uint32_t a = kDoubleS ? s_tmem_db : s_tmem[t];
                    if (ks == 0) MmaTSFlag(o_tmem[t], a, b0, idesc_o, first ? 0u : 1u);
                    else MmaTS<true>(o_tmem[t], a + ks * 8, b0 + ks * (2048 >> 4), idesc_o);
                }
            };
            uint32_t q_uses[2] = {0, 0};    // items finished per query buffer
            uint32_t steps[2] = {0, 0};     // KV tiles processed per query tile (phase of s_full / p_full / o_done)
            uint32_t kv_base = 0;           // ring position of this item's K_0
            uint32_t v_uses[G::kSlots] = {};  // V tiles consumed per ring slot (phase of v_ready)
            bool ok = true;
            if constexpr (kDoubleS) {
                // single query tile, two score buffers: S(0), S(1), then P(j) V_j followed by S(j+2) into the buffer
                // P(j) came from (same in-order stream, so the overwrite happens after the read)
                uint32_t buf_uses[2] = {0, 0};  // P tiles consumed per score buffer (phase of p_full)
                auto next_slot = [&](uint32_t* slot, bool is_v) {
                    *slot = kv_base % G::kSlots;
                    const uint32_t phase = (kv_base / G::kSlots) & 1u;
                    ++kv_base;
                    if (kCvtInKernel && is_v) return MbarWait(bar(kVReady + *slot), v_uses[*slot]++ & 1u, abort_flag);
                    return MbarWait(bar(kKvFull + *slot), phase, abort_flag);
                };
                for (int r = 0; r < rounds && ok; ++r) {
                    const int idx = item_of_round(r);
                    if (idx < 0) continue;
                    const Item w = decode_item(idx);
                    const int n = w.n_max;
                    if (n == 0) continue;
                    ok = MbarWait(bar(kQFull), q_uses[0] & 1u, abort_flag);
                    uint32_t slot = 0;
                    for (int i = 0; i < 2 && i < n && ok; ++i) {
                        ok = next_slot(&slot, false);
                        if (!ok) break;
                        TcFenceAfter();
                        s_tmem_db = tmem_base + G::kSCol + i * 64;
                        issue_s(0, slot);
                        MmaCommit(bar(kSFull + i));
                        if (i == n - 1) MmaCommit(bar(kQEmpty));
                        MmaCommit(bar(kKvEmpty + slot));
                    }
                    for (int j = 0; j < n && ok; ++j) {
                        const uint32_t buf = j & 1;
                        ok = MbarWait(bar(kPFull + buf), buf_uses[buf] & 1u, abort_flag);
                        ++buf_uses[buf];
                        if (ok && j == 0 && q_uses[0] > 0) ok = MbarWait(bar(kOFree), (q_uses[0] - 1) & 1u, abort_flag);
                        if (ok) ok = next_slot(&slot, true);  // V_j
                        if (!ok) break;
                        TcFenceAfter();
                        s_tmem_db = tmem_base + G::kSCol + buf * 64;
                        issue_pv(0, slot, j == 0);
                        MmaCommit(bar(kODone + buf));
                        MmaCommit(bar(kKvEmpty + slot));
                        if (j + 2 < n) {
                            ok = next_slot(&slot, false);  // K_j+2
                            if (!ok) break;
                            TcFenceAfter();
                            issue_s(0, slot);
                            MmaCommit(bar(kSFull + buf));
                            if (j + 2 == n - 1) MmaCommit(bar(kQEmpty));
                            MmaCommit(bar(kKvEmpty + slot));
                        }
                    }
                    ++q_uses[0];
                }
            }
            for (int r = 0; r < rounds && ok && !kDoubleS; ++r) {
                const int idx = item_of_round(r);
                if (idx < 0) continue;
                const Item w = decode_item(idx);
                auto slot_of = [&](int it) { return (kv_base + it) % G::kSlots; };
                auto phase_of = [&](int it) { return ((kv_base + it) / G::kSlots) & 1u; };
                for (int t = 0; t < QT && ok; ++t) {
                    if (w.ntiles[t] > 0) ok = MbarWait(bar(kQFull + t), q_uses[t] & 1u, abort_flag);
                }
                if (ok && w.n_max > 0) {
                    ok = MbarWait(bar(kKvFull + slot_of(0)), phase_of(0), abort_flag);
                    if (ok) {
                        TcFenceAfter();
                        for (int t = 0; t < QT; ++t) {
                            if (w.ntiles[t] == 0) continue;
                            issue_s(t, slot_of(0));
                            MmaCommit(bar(kSFull + t));
                            if (w.ntiles[t] == 1) MmaCommit(bar(kQEmpty + t));  // last read of this query tile
                        }
                        MmaCommit(bar(kKvEmpty + slot_of(0)));
                    }
                }
                for (int j = 0; j < w.n_max && ok; ++j) {
                    const int it_v = 2 * j + 1;
                    const int it_k = 2 * j + 2;
                    if (kCvtInKernel) ok = MbarWait(bar(kVReady + slot_of(it_v)), v_uses[slot_of(it_v)]++ & 1u, abort_flag);
                    else ok = MbarWait(bar(kKvFull + slot_of(it_v)), phase_of(it_v), abort_flag);
                    if (ok && j + 1 < w.n_max) ok = MbarWait(bar(kKvFull + slot_of(it_k)), phase_of(it_k), abort_flag);
                    if (!ok) break;
                    for (int t = 0; t < QT; ++t) {
                        if (j >= w.ntiles[t]) continue;
                        ok = MbarWait(bar(kPFull + t), steps[t] & 1u, abort_flag);
                        // the first P V of an item overwrites O: the previous item's O must have been read out
                        if (ok && j == 0 && q_uses[t] > 0) ok = MbarWait(bar(kOFree + t), (q_uses[t] - 1) & 1u, abort_flag);
                        if (!ok) break;
                        TcFenceAfter();
                        issue_pv(t, slot_of(it_v), j == 0);
                        MmaCommit(bar(kODone + t));
                        ++steps[t];
                        if (j + 1 < w.ntiles[t]) {
                            issue_s(t, slot_of(it_k));
                            MmaCommit(bar(kSFull + t));
                            if (j + 2 == w.ntiles[t]) MmaCommit(bar(kQEmpty + t));
                        }
                    }
                    if (!ok) break;
                    MmaCommit(bar(kKvEmpty + slot_of(it_v)));
                    if (j + 1 < w.n_max) MmaCommit(bar(kKvEmpty + slot_of(it_k)));
                }
                for (int t = 0; t < QT; ++t) {
                    if (w.ntiles[t] > 0) ++q_uses[t];
                }
                kv_base += 2 * w.n_max;
            }
            failed = !ok;
        }
    } else if (kCvtInKernel && warp < 4) {
        // ================================ V converter (warps 2 and 3, paged bf16) ====================
        // Walks the ring in the producer's order; every V tile is rewritten in place from bf16 to fp16 once its
        // bytes have landed, then handed to the MMA thread through v_ready. K tiles are not touched.
        const int tid = threadIdx.x - 64;
        uint32_t kv_loads = 0;
        bool ok = true;
        for (int r = 0; r < rounds && ok; ++r) {
            const int idx = item_of_round(r);
            if (idx < 0) continue;
            const Item w = decode_item(idx);
            for (int it = 0; it < 2 * w.n_max && ok; ++it, ++kv_loads) {
                bool is_v;
                if (kDoubleS) {
                    const int n = w.n_max;
                    const int lead = n > 1 ? 2 : 1;
                    if (it < lead) {
                        is_v = false;
                    } else {
                        const int f = it - lead, kk = n - lead;
                        is_v = f >= 2 * kk || (f & 1) == 0;
                    }
                } else {
                    is_v = (it & 1) != 0;
                }
                if (!is_v) continue;
                const uint32_t slot = kv_loads % G::kSlots;
                const uint32_t phase = (kv_loads / G::kSlots) & 1u;
                ok = __all_sync(0xffffffffu, MbarWait(bar(kKvFull + slot), phase, abort_flag));
                if (!ok) break;
                uint4* tile = reinterpret_cast<uint4*>(smem + (ring_smem - smem_base) + slot * G::kKvTileBytes);
#pragma unroll 4
                for (int c = tid; c < G::kKvTileBytes / 16; c += kConverterThreads) {
                    uint4 x = tile[c];
                    uint32_t* word = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = Unpack2<__nv_bfloat16>(word[e]);
                        // one instruction for both lanes; values beyond the fp16 range saturate instead of becoming inf
                        asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(word[e]) : "f"(f.y), "f"(f.x));
                    }
                    tile[c] = x;
                }
                FenceProxyAsync();  // generic-proxy writes -> visible to the tensor core's reads
                MbarArrive(bar(kVReady + slot));
            }
        }
        failed = !ok;
    } else if (warp >= 4) {
        // ================================ softmax groups ============================================
        const int t = (warp - 4) >> 2;
        const int quad = warp & 3;
        const int row_in_tile = quad * 32 + lane;
        const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t s_addr0 = tmem_base + lane_bits + G::kSCol + t * 128;
        const uint32_t o_addr = tmem_base + lane_bits + G::kOCol + t * DP;
        uint32_t steps = 0;  // KV tiles this group has processed (phase of s_full / p_full / o_done)
        uint32_t buf_steps0 = 0, buf_steps1 = 0;  // double-buffered scores: tiles taken from each buffer
        uint32_t tiles_before = 0;  // paged K/V: KV tiles of the items this CTA has finished (index into valid_ring)
        const uint32_t all_pages = kPaged ? ((BN >> p.block_shift) >= 32 ? 0xffffffffu : (1u << (BN >> p.block_shift)) - 1u) : 0u;
        bool ok = true;

        for (int r = 0; r < rounds && ok && t < QT; ++r) {
            const int idx = item_of_round(r);
            if (idx < 0) continue;
            const Item w = decode_item(idx);
            const int n_t = w.ntiles[t];
            const uint32_t tiles_base = tiles_before;
            tiles_before += static_cast<uint32_t>(w.n_max);
            if (n_t == 0) continue;
            const int row = w.m0[t] + row_in_tile;
            float m_ref = -CUDART_INF_F;  // reference point of the exponentials (log2 domain)
            float l_sum = 0.0f;

            for (int j = 0; j < n_t; ++j, ++steps) {
                // which score buffer / barrier set this step uses, and the phases to wait for
                const uint32_t buf = kDoubleS ? (j & 1) : 0;
                const uint32_t s_addr = s_addr0 + buf * 64;
                const int sync = kDoubleS ? static_cast<int>(buf) : t;          // index into s_full / p_full
                const uint32_t s_phase = kDoubleS ? ((buf ? buf_steps1 : buf_steps0) & 1u) : (steps & 1u);
                // the product P(j-1) V_j-1 that must be complete before O may be rescaled
                const int prev_sync = kDoubleS ? static_cast<int>(buf ^ 1) : t;
                const uint32_t prev_phase = kDoubleS ? (((buf ? buf_steps0 : buf_steps1) - 1) & 1u) : ((steps - 1) & 1u);
                if (kDoubleS) {
                    if (buf) ++buf_steps1; else ++buf_steps0;
                }
                ok = __all_sync(0xffffffffu, MbarWait(bar(kSFull + sync), s_phase, abort_flag));
                if (!ok) break;
                TcFenceAfter();
                // One pass over the S row, 64 columns at a time. The exponentials use the reference point the row
                // already has; the half's own max is only checked against it. If a half exceeds the reference by
                // more than the threshold (always true for the first half of an item), the reference moves and
                // whatever was accumulated under the old one is rescaled: O, the row sum and the half of P that
                // this step has already written. P (16-bit pairs) lands on the first BN / 2 columns of S_t;
                // the half-row written in step h only covers columns that step h has already consumed.
                const int col0 = j * BN;
                const int kv_limit = w.seq_kv - col0;                                   // columns >= kv_limit do not exist
                const int causal_limit = p.causal ? (row + w.diagonal - col0 + 1) : BN;  // columns >= limit are masked
                const int limit = min(kv_limit, causal_limit);
                const uint32_t pages = kPaged ? valid_ring[(tiles_base + j) % kValidRing] : 0u;
                const bool holes = kPaged && pages != all_pages;   // some page of this tile is unmapped
                const bool ragged = limit < BN || holes;
                float part4[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // this step's share of the row sum
    #pragma unroll
                for (int half = 0; half < BN / 64; ++half) {
                    uint32_t ra[32], rb[32];
                    TmemLd32(s_addr + half * 64, ra);
                    TmemLd32(s_addr + half * 64 + 32, rb);
                    TmemWaitLd();
                    if (ragged) {
    #pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int ca = half * 64 + i, cb = half * 64 + 32 + i;
                            const bool gone_a = kPaged && holes && !((pages >> (ca >> p.block_shift)) & 1u);
                            const bool gone_b = kPaged && holes && !((pages >> (cb >> p.block_shift)) & 1u);
                            if (ca >= limit || gone_a) ra[i] = 0xff800000u;       // -inf
                            if (cb >= limit || gone_b) rb[i] = 0xff800000u;
                        }
                    }
                    float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
    #pragma unroll
                    for (int i = 0; i < 32; i += 4) {
    #pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            mx4[e] = fmaxf(mx4[e], fmaxf(__uint_as_float(ra[i + e]), __uint_as_float(rb[i + e])));
                        }
                    }
                    const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;  // scale > 0
                    const bool move = mx > m_ref + kRescaleThreshold;  // false for a fully masked half (-inf)
                    if (__any_sync(0xffffffffu, move)) {
                        const float alpha = move ? Exp2(m_ref - mx) : 1.0f;  // m_ref = -inf -> 0
                        if (j > 0) {
                            ok = __all_sync(0xffffffffu, MbarWait(bar(kODone + prev_sync), prev_phase, abort_flag));
                            if (!ok) break;
                            TcFenceAfter();
    #pragma unroll 1
                            for (int cblk = 0; cblk < DP / 32; ++cblk) {
                                uint32_t r[32];
                                TmemLd32(o_addr + cblk * 32, r);
                                TmemWaitLd();
    #pragma unroll
                                for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                                TmemSt32(o_addr + cblk * 32, r);
                            }
                        }
                        l_sum *= alpha;
    #pragma unroll
                        for (int e = 0; e < 4; ++e) part4[e] *= alpha;
                        if (half > 0) {  // the first half of P was written under the old reference
                            uint32_t q[32];
                            TmemWaitSt();
                            TmemLd32(s_addr, q);
                            TmemWaitLd();
    #pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const float2 f = Unpack2<PT>(q[i]);
                                q[i] = Pack2<PT>(f.x * alpha, f.y * alpha);
                            }
                            TmemSt32(s_addr, q);
                        }
                        if (move) m_ref = mx;
                    }
                    const float neg_m = (m_ref == -CUDART_INF_F) ? 0.0f : -m_ref;
                    uint32_t pk[32];
                    const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
                    const float2 shift2 = make_float2(neg_m, neg_m);
                    float2 sum_a = make_float2(part4[0], part4[1]), sum_b = make_float2(part4[2], part4[3]);
    #pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float2 xa = Fma2(make_float2(__uint_as_float(ra[i]), __uint_as_float(ra[i + 1])), scale2, shift2);
                        const float2 xb = Fma2(make_float2(__uint_as_float(rb[i]), __uint_as_float(rb[i + 1])), scale2, shift2);
                        const float2 ea = make_float2(Exp2(xa.x), Exp2(xa.y));
                        const float2 eb = make_float2(Exp2(xb.x), Exp2(xb.y));
                        sum_a = Add2(sum_a, ea);
                        sum_b = Add2(sum_b, eb);
                        pk[i / 2] = Pack2<PT>(ea.x, ea.y);
                        pk[16 + i / 2] = Pack2<PT>(eb.x, eb.y);
                    }
                    part4[0] = sum_a.x;
                    part4[1] = sum_a.y;
                    part4[2] = sum_b.x;
                    part4[3] = sum_b.y;
                    TmemSt32(s_addr + half * 32, pk);
                }
                if (!ok) break;
                l_sum += (part4[0] + part4[1]) + (part4[2] + part4[3]);
                TmemWaitSt();
                TcFenceBefore();
                MbarArrive(bar(kPFull + sync));
            }
            if (!ok) break;

            // ---- epilogue: O / l -> global, optional LSE; O is handed back as soon as it is in registers ----
            if (kDoubleS) {
                const uint32_t last = (n_t - 1) & 1;
                ok = __all_sync(0xffffffffu, MbarWait(bar(kODone + last), ((last ? buf_steps1 : buf_steps0) - 1) & 1u, abort_flag));
            } else {
                ok = __all_sync(0xffffffffu, MbarWait(bar(kODone + t), (steps - 1) & 1u, abort_flag));
            }
            if (!ok) break;
            TcFenceAfter();
            const float inv = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
            T* o_row = reinterpret_cast<T*>(p.out) + w.b * p.o_sb + w.h * p.o_sh + static_cast<int64_t>(w.q_tok0 + row) * p.o_ss;
#pragma unroll
            for (int cblk = 0; cblk < DP / 32; ++cblk) {
                uint32_t r[32];
                TmemLd32(o_addr + cblk * 32, r);
                TmemWaitLd();
                if (cblk == DP / 32 - 1) {
                    TcFenceBefore();
                    MbarArrive(bar(kOFree + t));
                }
                if (row < w.seq_q) {
#pragma unroll
                    for (int v8 = 0; v8 < 4; ++v8) {
                        const int d0 = cblk * 32 + v8 * 8;
                        if (d0 < p.head_dim) {
                            uint4 pk;
                            pk.x = Pack2<T>(__uint_as_float(r[v8 * 8 + 0]) * inv, __uint_as_float(r[v8 * 8 + 1]) * inv);
                            pk.y = Pack2<T>(__uint_as_float(r[v8 * 8 + 2]) * inv, __uint_as_float(r[v8 * 8 + 3]) * inv);
                            pk.z = Pack2<T>(__uint_as_float(r[v8 * 8 + 4]) * inv, __uint_as_float(r[v8 * 8 + 5]) * inv);
                            pk.w = Pack2<T>(__uint_as_float(r[v8 * 8 + 6]) * inv, __uint_as_float(r[v8 * 8 + 7]) * inv);
                            *reinterpret_cast<uint4*>(o_row + d0) = pk;
                        }
                    }
                }
            }
            if (p.lse != nullptr && row < w.seq_q) {
                p.lse[(static_cast<int64_t>(w.b) * p.heads + w.h) * p.seq_q + row] =
                    l_sum > 0.0f ? (m_ref + log2f(l_sum)) * kLn2 : -CUDART_INF_F;
            }
        }
        failed = !ok;
    }

    if (failed && p.error_word != nullptr) *p.error_word = 1 + warp;

    // ---- teardown ------------------------------------------------------------------------------------
    TcFenceBefore();
    __syncthreads();
    if (warp == 2) {
        TcFenceAfter();
        TmemDealloc(tmem_base, kTmemColumns);
    }
}

// V [batch, heads, seq, D] (any strides, bf16) -> compact fp16 [batch, heads, seq, D]; 8 elements per thread.
__global__ void __launch_bounds__(256) flash_v_to_f16_kernel(const __nv_bfloat16* __restrict__ v, __half* __restrict__ out,
                                                              int64_t batch, int64_t heads, int64_t seq, int64_t head_dim,
                                                              int64_t sb, int64_t sh, int64_t ss) {
    const int64_t chunks_per_row = head_dim / 8;
    const int64_t total = batch * heads * seq * chunks_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int64_t rest = i;
        const int64_t c = rest % chunks_per_row;
        rest /= chunks_per_row;
        const int64_t s = rest % seq;
        rest /= seq;
        const int64_t h = rest % heads;
        const int64_t b = rest / heads;
        uint4 x = *reinterpret_cast<const uint4*>(v + b * sb + h * sh + s * ss + c * 8);
        uint32_t* word = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = Unpack2<__nv_bfloat16>(word[e]);
            // one instruction for both lanes; values beyond the fp16 range saturate instead of becoming inf
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(word[e]) : "f"(f.y), "f"(f.x));
        }
        reinterpret_cast<uint4*>(out)[i] = x;
    }
}

// ---- host side -----------------------------------------------------------------------------------------
constexpr int kMaxStatusDevices = 64;

// Stream-ordered temporaries come from a pool of this library's own (one per device, created on first use) that keeps
// what is freed: the default pool hands its memory back to the driver at every synchronisation, after which the next
// allocation costs a trip to the driver again.
cudaMemPool_t TemporaryPool() {
    static std::mutex mu;
    static cudaMemPool_t pools[kMaxStatusDevices] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxStatusDevices) {
        cudaGetLastError();
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (pools[device] == nullptr) {
        cudaMemPoolProps props{};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = device;
        cudaMemPool_t pool = nullptr;
        if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        unsigned long long keep = ~0ull;
        if (cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess) cudaGetLastError();
        pools[device] = pool;
    }
    return pools[device];
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn GetEncodeTiled() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            sym = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// [batch][heads][seq][D] through element strides (sb, sh, ss); box = 64 elements x box_rows rows, 128B swizzle,
// out-of-range elements read as zero.
int MakeMap(CUtensorMap* map, const void* base, int dtype_id, int64_t d, int64_t seq, int64_t heads, int64_t batch,
            int64_t ss, int64_t sh, int64_t sb, int box_rows, const char* what) {
    EncodeTiledFn encode = GetEncodeTiled();
    if (encode == nullptr) return Fail(SCA_CUDA_ERROR, "flash attention: cuTensorMapEncodeTiled is unavailable");
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(seq),
                                static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss) * 2, static_cast<cuuint64_t>(sh) * 2,
                                   static_cast<cuuint64_t>(sb) * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    const CUtensorMapDataType type =
        dtype_id == SCA_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const CUresult rc = encode(map, type, 4, const_cast<void*>(base), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        return Fail(SCA_INVALID_ARGUMENT, std::string("flash attention: tensor map for ") + what +
                                              " rejected (CUresult " + std::to_string(static_cast<int>(rc)) +
                                              "); base must be 16-byte aligned and strides multiples of 8 elements");
    }
    return SCA_OK;
}

// One host-visible word per device that a kernel sets when one of its bounded waits expires (1 + the warp that
// gave up). The words live in one pinned, mapped, portable allocation; sca_flash_status reads and clears them.

int* ErrorWords(int** host_view) {
    static int* host = nullptr;
    static int* dev = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaHostAlloc(reinterpret_cast<void**>(&host), kMaxStatusDevices * sizeof(int),
                          cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            cudaGetLastError();
            host = nullptr;
            return;
        }
        for (int i = 0; i < kMaxStatusDevices; ++i) host[i] = 0;
        if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev), host, 0) != cudaSuccess) {
            cudaGetLastError();
            dev = nullptr;
        }
    });
    if (host_view != nullptr) *host_view = host;
    return dev;
}

// Device-side address of the current device's word (nullptr when the mapping could not be made).
int* ErrorWordForCurrentDevice() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    int* dev = ErrorWords(nullptr);
    return (dev != nullptr && device >= 0 && device < kMaxStatusDevices) ? dev + device : nullptr;
}

// A packed variable-length batch: host offsets and a device scratch area for the work list.
struct VarlenWork {
    const int32_t* cu_q;
    const int32_t* cu_kv;
    int64_t num_seqs;
    void* workspace;
    int64_t workspace_bytes;
};

int64_t VarlenWorkspaceBytes(int64_t num_seqs, int64_t total_q) {
    // one int4 per sequence + one int2 per block of 128 query rows (an upper bound for both geometries)
    return num_seqs * 16 + (total_q / kBlockM + num_seqs) * 8 + 64;
}

// Builds {first q token, first kv token, S_q, S_kv} per sequence and the (sequence, query block) list, heaviest
// block first, and copies both into the workspace (stream-ordered; the host vectors may die on return).
int UploadVarlenWork(const VarlenWork& vw, int rows_per_entry, int block_n, bool causal, cudaStream_t stream,
                     const int4** seqs_out, const int2** entries_out, int* num_entries_out) {
    std::vector<int4> seqs(static_cast<size_t>(vw.num_seqs));
    struct Weighted {
        int2 entry;
        int64_t tiles;
    };
    std::vector<Weighted> list;
    for (int64_t s = 0; s < vw.num_seqs; ++s) {
        const int64_t sq = static_cast<int64_t>(vw.cu_q[s + 1]) - vw.cu_q[s];
        const int64_t skv = static_cast<int64_t>(vw.cu_kv[s + 1]) - vw.cu_kv[s];
        if (sq <= 0 || skv <= 0 || (causal && skv < sq)) {
            return Fail(SCA_INVALID_ARGUMENT, "flash varlen: sequence " + std::to_string(s) + " has S_q=" + std::to_string(sq) +
                                                  ", S_kv=" + std::to_string(skv) + (causal ? " (causal needs 0 < S_q <= S_kv)" : " (both must be > 0)"));
        }
        seqs[static_cast<size_t>(s)] = make_int4(vw.cu_q[s], vw.cu_kv[s], static_cast<int>(sq), static_cast<int>(skv));
        for (int64_t mb = 0; mb * rows_per_entry < sq; ++mb) {
            int64_t limit = skv;
            if (causal) limit = std::min<int64_t>(limit, std::min<int64_t>(sq, (mb + 1) * rows_per_entry) + (skv - sq));
            list.push_back({make_int2(static_cast<int>(s), static_cast<int>(mb)), (limit + block_n - 1) / block_n});
        }
    }
    std::stable_sort(list.begin(), list.end(), [](const Weighted& a, const Weighted& b) { return a.tiles > b.tiles; });
    std::vector<int2> entries(list.size());
    for (size_t i = 0; i < list.size(); ++i) entries[i] = list[i].entry;
    const size_t seq_bytes = seqs.size() * sizeof(int4);
    const size_t entry_bytes = entries.size() * sizeof(int2);
    if (vw.workspace == nullptr || static_cast<int64_t>(seq_bytes + entry_bytes) > vw.workspace_bytes) {
        return Fail(SCA_INVALID_ARGUMENT, "flash varlen: workspace of " + std::to_string(vw.workspace_bytes) + " bytes is too small (" +
                                              std::to_string(seq_bytes + entry_bytes) + " needed)");
    }
    unsigned char* base = static_cast<unsigned char*>(vw.workspace);
    if (cudaError_t e = cudaMemcpyAsync(base, seqs.data(), seq_bytes, cudaMemcpyHostToDevice, stream); e != cudaSuccess) {
        return FailCuda(e, "cudaMemcpyAsync(varlen sequences)");
    }
    if (cudaError_t e = cudaMemcpyAsync(base + seq_bytes, entries.data(), entry_bytes, cudaMemcpyHostToDevice, stream); e != cudaSuccess) {
        return FailCuda(e, "cudaMemcpyAsync(varlen work list)");
    }
    *seqs_out = reinterpret_cast<const int4*>(base);
    *entries_out = reinterpret_cast<const int2*>(base + seq_bytes);
    *num_entries_out = static_cast<int>(entries.size());
    return SCA_OK;
}

// A paged KV pool behind a packed batch: f.k / f.v point at one layer's pool [num_blocks, block_size, H_kv, D].
struct PagedWork {
    const int32_t* page_table;
    int64_t num_blocks, block_size, max_blocks_per_seq;
};

template <typename T, int DP, int QT, int BN>
int LaunchFlash(const ScaFlashFwdParams& f, cudaStream_t stream, const VarlenWork* varlen = nullptr,
                const PagedWork* paged = nullptr) {
    using G = FlashGeom<DP, QT, BN>;
    CUtensorMap map_q, map_k, map_v;
    if (int rc = MakeMap(&map_q, f.q, f.dtype_id, f.head_dim, f.seq_q, f.num_heads, f.batch, f.q_ss, f.q_sh, f.q_sb, kBlockM, "q")) return rc;
    if (paged != nullptr) {
        // the pool as [rows = blocks * block_size, H_kv, D]; one box = one page of one kv head and column block
        const int64_t rows = paged->num_blocks * paged->block_size;
        const int64_t row_elems = f.num_kv_heads * f.head_dim;
        if (int rc = MakeMap(&map_k, f.k, f.dtype_id, f.head_dim, rows, f.num_kv_heads, 1, row_elems, f.head_dim, rows * row_elems,
                             static_cast<int>(paged->block_size), "k pool")) return rc;
        if (int rc = MakeMap(&map_v, f.v, f.dtype_id, f.head_dim, rows, f.num_kv_heads, 1, row_elems, f.head_dim, rows * row_elems,
                             static_cast<int>(paged->block_size), "v pool")) return rc;
    } else
    if (int rc = MakeMap(&map_k, f.k, f.dtype_id, f.head_dim, f.seq_kv, f.num_kv_heads, f.batch, f.k_ss, f.k_sh, f.k_sb, BN, "k")) return rc;
    // bf16: V goes through an fp16 copy (PvFormat). The copy is a stream-ordered temporary, released behind the launch.
    struct Temporary {
        void* ptr = nullptr;
        cudaStream_t stream = nullptr;
        ~Temporary() {
            if (ptr != nullptr && cudaFreeAsync(ptr, stream) != cudaSuccess) cudaGetLastError();
        }
    } v16;
    if (paged != nullptr) {
        // map_v is set above: the pool is read in place, in the input format
    } else if (PvFormat<T>::kConvertV) {
        if (!Aligned16(f.v) || f.v_sb % 8 != 0 || f.v_sh % 8 != 0 || f.v_ss % 8 != 0 || f.head_dim % 8 != 0) {
            return Fail(SCA_INVALID_ARGUMENT, "flash attention: v must be 16-byte aligned with strides that are multiples of 8 elements");
        }
        const int64_t elements = f.batch * f.num_kv_heads * f.seq_kv * f.head_dim;
        v16.stream = stream;
        cudaMemPool_t pool = TemporaryPool();
        const cudaError_t e = pool != nullptr ? cudaMallocFromPoolAsync(&v16.ptr, static_cast<size_t>(elements) * 2, pool, stream)
                                              : cudaMallocAsync(&v16.ptr, static_cast<size_t>(elements) * 2, stream);
        if (e != cudaSuccess) {
            v16.ptr = nullptr;
            cudaGetLastError();
            return FailCuda(e, "flash attention: cudaMallocAsync(fp16 copy of V)");
        }
        const int64_t threads_needed = elements / 8;
        const unsigned blocks = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((threads_needed + 255) / 256, static_cast<int64_t>(SmCount()) * 16)));
        flash_v_to_f16_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(f.v), static_cast<__half*>(v16.ptr),
                                                          f.batch, f.num_kv_heads, f.seq_kv, f.head_dim, f.v_sb, f.v_sh, f.v_ss);
        if (int rc = CheckLaunch("flash_v_to_f16_kernel", stream)) return rc;
        if (int rc = MakeMap(&map_v, v16.ptr, SCA_DTYPE_F16, f.head_dim, f.seq_kv, f.num_kv_heads, f.batch, f.head_dim,
                             f.seq_kv * f.head_dim, f.num_kv_heads * f.seq_kv * f.head_dim, BN, "v (fp16 copy)")) return rc;
    } else {
        if (int rc = MakeMap(&map_v, f.v, f.dtype_id, f.head_dim, f.seq_kv, f.num_kv_heads, f.batch, f.v_ss, f.v_sh, f.v_sb, BN, "v")) return rc;
    }

    FlashKernelParams p{};
    p.out = f.out;
    p.lse = f.return_lse ? f.lse : nullptr;
    p.error_word = ErrorWordForCurrentDevice();
    p.seq_q = static_cast<int>(f.seq_q);
    p.seq_kv = static_cast<int>(f.seq_kv);
    p.heads = static_cast<int>(f.num_heads);
    p.kv_heads = static_cast<int>(f.num_kv_heads);
    p.head_dim = static_cast<int>(f.head_dim);
    p.batch = static_cast<int>(f.batch);
    p.o_sb = f.o_sb;
    p.o_sh = f.o_sh;
    p.o_ss = f.o_ss;
    p.scale_log2 = f.scale * kLog2e;
    p.causal = f.causal ? 1 : 0;
    p.diagonal = static_cast<int>(f.causal ? f.diagonal : 0);
    p.m_blocks = static_cast<int>((f.seq_q + QT * kBlockM - 1) / (QT * kBlockM));
    if (varlen != nullptr) {
        if (int rc = UploadVarlenWork(*varlen, QT * kBlockM, BN, f.causal != 0, stream, &p.seqs, &p.entries, &p.num_entries)) return rc;
    }
    const int64_t ctas = varlen != nullptr ? static_cast<int64_t>(p.num_entries) * p.heads
                                           : static_cast<int64_t>(p.m_blocks) * p.batch * p.heads;
    if (ctas <= 0 || ctas > 0x7fffffffLL) {
        return Fail(SCA_INVALID_ARGUMENT, "flash attention: grid of " + std::to_string(ctas) + " blocks is out of range");
    }
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(ctas, SmCount()));  // one persistent CTA per SM
    if (paged != nullptr) {
        p.page_table = paged->page_table;
        p.max_blocks_per_seq = static_cast<int>(paged->max_blocks_per_seq);
        p.num_kv_blocks = static_cast<int>(paged->num_blocks);
        p.block_size = static_cast<int>(paged->block_size);
        p.block_shift = 0;
        while ((1 << p.block_shift) < p.block_size) ++p.block_shift;
        const void* fn = reinterpret_cast<const void*>(&flash_fwd_sm100_kernel<T, DP, QT, BN, true, true>);
        if (int rc = EnsureDynamicSmem(fn, G::kSmemBytes, "flash_fwd_sm100_kernel")) return rc;
        flash_fwd_sm100_kernel<T, DP, QT, BN, true, true><<<grid, kFlashThreads, G::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
    } else if (varlen != nullptr) {
        const void* fn = reinterpret_cast<const void*>(&flash_fwd_sm100_kernel<T, DP, QT, BN, true>);
        if (int rc = EnsureDynamicSmem(fn, G::kSmemBytes, "flash_fwd_sm100_kernel")) return rc;
        flash_fwd_sm100_kernel<T, DP, QT, BN, true><<<grid, kFlashThreads, G::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
    } else {
        const void* fn = reinterpret_cast<const void*>(&flash_fwd_sm100_kernel<T, DP, QT, BN, false>);
        if (int rc = EnsureDynamicSmem(fn, G::kSmemBytes, "flash_fwd_sm100_kernel")) return rc;
        flash_fwd_sm100_kernel<T, DP, QT, BN, false><<<grid, kFlashThreads, G::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
    }
    if (int rc = CheckLaunch("flash_fwd_sm100_kernel", stream)) return rc;
    // With SCI_ATTENTION_DEBUG_SYNC=1 CheckLaunch has waited for the kernel: a wait that ran out is known now.
    if (DebugSyncEnabled()) {
        int device = 0, code = 0;
        if (cudaGetDevice(&device) == cudaSuccess && sca_flash_status(device, &code) == SCA_OK && code != 0) {
            return Fail(SCA_CUDA_ERROR, "flash attention: the launch gave up waiting on a barrier (role " +
                                            std::to_string(code) + "); its output is invalid");
        }
    }
    return SCA_OK;
}

int ValidateFlash(const ScaFlashFwdParams* params) {
    if (params == nullptr || params->q == nullptr || params->k == nullptr || params->v == nullptr ||
        params->out == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "flash attention: null tensor pointer");
    }
    const ScaFlashFwdParams& f = *params;
    if (f.dtype_id != SCA_DTYPE_F16 && f.dtype_id != SCA_DTYPE_BF16) {
        return Fail(SCA_INVALID_ARGUMENT, "flash attention: only fp16/bf16 are instantiated (dtype_id=" +
                                              std::to_string(f.dtype_id) + "); use the naive or tiled backend for FP32");
    }
    if (f.batch < 1 || f.num_heads < 1 || f.num_kv_heads < 1 || f.seq_q < 1 || f.seq_kv < 1 ||
        f.num_heads % f.num_kv_heads != 0) {
        return Fail(SCA_INVALID_ARGUMENT, "flash attention: invalid geometry");
    }
    if (f.seq_q > 0x7fffff00LL || f.seq_kv > 0x7fffff00LL) {
        return Fail(SCA_INVALID_ARGUMENT, "flash attention: sequence length exceeds the 32-bit tile index range");
    }
    if (!(f.scale > 0.0f)) return Fail(SCA_INVALID_ARGUMENT, "flash attention: scale must be > 0");
    if (f.return_lse && f.lse == nullptr) return Fail(SCA_INVALID_ARGUMENT, "flash attention: return_lse without a buffer");
    if (!Aligned16(f.out) || f.o_sb % 8 != 0 || f.o_sh % 8 != 0 || f.o_ss % 8 != 0) {
        return Fail(SCA_INVALID_ARGUMENT, "flash attention: out must be 16-byte aligned with strides that are multiples of 8 elements");
    }
    return SCA_OK;
}

template <typename T>
int LaunchFlashTyped(const ScaFlashFwdParams& f, cudaStream_t stream, const VarlenWork* varlen = nullptr,
                     const PagedWork* paged = nullptr) {
    // head dims that are not a multiple of 64 run on the next padded geometry: the TMA unit
    // zero-fills the missing columns of Q, K and V, which leaves S and the real columns of O unchanged
    switch (f.head_dim) {
        case 32:
        case 64: return LaunchFlash<T, 64, 2, 128>(f, stream, varlen, paged);
        case 96:
        case 128: return LaunchFlash<T, 128, 2, 128>(f, stream, varlen, paged);
        case 160:
        case 192:
        case 256: return LaunchFlash<T, 256, 1, 64>(f, stream, varlen, paged);
        default: break;
    }
    return Fail(SCA_INVALID_ARGUMENT, "flash attention: head_dim=" + std::to_string(f.head_dim) + " is not instantiated");
}

}  // namespace
}  // namespace sca_b200

using namespace sca_b200;

extern "C" int sca_flash_status(int device_id, int32_t* status_out) {
    if (status_out == nullptr) return Fail(SCA_INVALID_ARGUMENT, "flash status: null output");
    if (device_id < 0 || device_id >= kMaxStatusDevices) {
        return Fail(SCA_INVALID_ARGUMENT, "flash status: device index " + std::to_string(device_id) + " is out of range");
    }
    int* host = nullptr;
    ErrorWords(&host);
    // the kernel writes the word over the bus with a plain store; the host takes it with one atomic exchange
    *status_out = host != nullptr ? __atomic_exchange_n(host + device_id, 0, __ATOMIC_ACQ_REL) : 0;
    return SCA_OK;
}

extern "C" long long sca_flash_smem_bytes_for(int head_dim, long long elem_bytes, int block_m, int block_n,
                                              int stages) {
    if (head_dim <= 0 || elem_bytes <= 0 || block_m <= 0 || block_n <= 0 || stages <= 0) return -1;
    const long long q = static_cast<long long>(block_m) * head_dim * elem_bytes;
    const long long kv = static_cast<long long>(block_n) * head_dim * elem_bytes * stages;
    return q + 2 * kv + 1024;
}

extern "C" int sca_launch_flash_fwd(const ScaFlashFwdParams* params, void* stream) {
    ClearError();
    if (int rc = ValidateFlash(params)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return params->dtype_id == SCA_DTYPE_F16 ? LaunchFlashTyped<__half>(*params, s)
                                             : LaunchFlashTyped<__nv_bfloat16>(*params, s);
}

extern "C" long long sca_flash_varlen_workspace_bytes(int64_t num_seqs, int64_t total_q) {
    if (num_seqs < 1 || total_q < 1) return -1;
    return VarlenWorkspaceBytes(num_seqs, total_q);
}

// Packed variable-length prefill in ONE launch (the reference loops over the sequences on the host,
// src/backends/flash/flash_backend.cpp:312-363): the persistent kernel's work list simply spans all sequences.
extern "C" int sca_launch_flash_varlen(const ScaFlashVarlenParams* params, void* stream) {
    ClearError();
    if (params == nullptr || params->cu_seqlens_q == nullptr || params->cu_seqlens_kv == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "flash varlen: null parameter block or host offsets");
    }
    const ScaFlashVarlenParams& x = *params;
    if (x.num_seqs < 1 || x.total_q < 1 || x.total_kv < 1) return Fail(SCA_INVALID_ARGUMENT, "flash varlen: empty batch");
    if (x.cu_seqlens_q[0] != 0 || x.cu_seqlens_kv[0] != 0 || x.cu_seqlens_q[x.num_seqs] != x.total_q ||
        x.cu_seqlens_kv[x.num_seqs] != x.total_kv) {
        return Fail(SCA_INVALID_ARGUMENT, "flash varlen: offsets must start at 0 and end at the token totals");
    }
    ScaFlashFwdParams f{};
    f.q = x.q;
    f.k = x.k;
    f.v = x.v;
    f.out = x.out;
    f.batch = 1;
    f.num_heads = x.num_heads;
    f.num_kv_heads = x.num_kv_heads;
    f.seq_q = x.total_q;
    f.seq_kv = x.total_kv;
    f.head_dim = x.head_dim;
    f.q_ss = x.num_heads * x.head_dim;
    f.q_sh = x.head_dim;
    f.q_sb = x.total_q * f.q_ss;
    f.k_ss = x.num_kv_heads * x.head_dim;
    f.k_sh = x.head_dim;
    f.k_sb = x.total_kv * f.k_ss;
    f.v_ss = f.k_ss;
    f.v_sh = f.k_sh;
    f.v_sb = f.k_sb;
    f.o_ss = f.q_ss;
    f.o_sh = f.q_sh;
    f.o_sb = f.q_sb;
    f.scale = x.scale;
    f.causal = x.causal;
    f.dtype_id = x.dtype_id;
    if (int rc = ValidateFlash(&f)) return rc;
    VarlenWork vw{x.cu_seqlens_q, x.cu_seqlens_kv, x.num_seqs, x.workspace, x.workspace_bytes};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return f.dtype_id == SCA_DTYPE_F16 ? LaunchFlashTyped<__half>(f, s, &vw)
                                       : LaunchFlashTyped<__nv_bfloat16>(f, s, &vw);
}

extern "C" int sca_launch_flash_paged(const ScaFlashPagedParams* params, void* stream) {
    ClearError();
    if (params == nullptr || params->cu_seqlens_q == nullptr || params->seq_lens_kv == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "flash paged: null parameter block or host lengths");
    }
    const ScaFlashPagedParams& x = *params;
    if (x.q == nullptr || x.out == nullptr || x.k_pool == nullptr || x.v_pool == nullptr || x.page_table == nullptr) {
        return Fail(SCA_INVALID_ARGUMENT, "flash paged: null tensor pointer");
    }
    if (x.num_seqs < 1 || x.total_q < 1) return Fail(SCA_INVALID_ARGUMENT, "flash paged: empty batch");
    if (x.cu_seqlens_q[0] != 0 || x.cu_seqlens_q[x.num_seqs] != x.total_q) {
        return Fail(SCA_INVALID_ARGUMENT, "flash paged: query offsets must start at 0 and end at total_q");
    }
    if (x.block_size != 8 && x.block_size != 16 && x.block_size != 32 && x.block_size != 64) {
        return Fail(SCA_INVALID_ARGUMENT, "flash paged: block_size=" + std::to_string(x.block_size) +
                                              " (pages are loaded as boxes of 8, 16, 32 or 64 tokens)");
    }
    if (x.num_blocks < 1 || x.max_blocks_per_seq < 1 || x.num_blocks * x.block_size > 0x7fffff00LL) {
        return Fail(SCA_INVALID_ARGUMENT, "flash paged: invalid pool geometry");
    }
    // kv offsets for the shared work-list builder: only the lengths are used on the device
    std::vector<int32_t> cu_kv(static_cast<size_t>(x.num_seqs) + 1, 0);
    for (int64_t s = 0; s < x.num_seqs; ++s) {
        const int64_t have = x.seq_lens_kv[s];
        if (have < 1 || have > x.max_blocks_per_seq * x.block_size) {
            return Fail(SCA_INVALID_ARGUMENT, "flash paged: sequence " + std::to_string(s) + " has " + std::to_string(have) +
                                                  " tokens in the cache (the page-table row holds " +
                                                  std::to_string(x.max_blocks_per_seq * x.block_size) + ")");
        }
        const int64_t next = static_cast<int64_t>(cu_kv[static_cast<size_t>(s)]) + have;
        if (next > 0x7fffffffLL) return Fail(SCA_INVALID_ARGUMENT, "flash paged: more than 2^31 cached tokens in one call");
        cu_kv[static_cast<size_t>(s) + 1] = static_cast<int32_t>(next);
    }
    ScaFlashFwdParams f{};
    f.q = x.q;
    f.k = x.k_pool;
    f.v = x.v_pool;
    f.out = x.out;
    f.batch = 1;
    f.num_heads = x.num_heads;
    f.num_kv_heads = x.num_kv_heads;
    f.seq_q = x.total_q;
    f.seq_kv = cu_kv.back();
    f.head_dim = x.head_dim;
    f.q_ss = x.num_heads * x.head_dim;
    f.q_sh = x.head_dim;
    f.q_sb = x.total_q * f.q_ss;
    f.o_ss = f.q_ss;
    f.o_sh = f.q_sh;
    f.o_sb = f.q_sb;
    f.scale = x.scale;
    f.causal = x.causal;
    f.dtype_id = x.dtype_id;
    if (int rc = ValidateFlash(&f)) return rc;
    VarlenWork vw{x.cu_seqlens_q, cu_kv.data(), x.num_seqs, x.workspace, x.workspace_bytes};
    PagedWork pw{x.page_table, x.num_blocks, x.block_size, x.max_blocks_per_seq};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (f.dtype_id) {
        case SCA_DTYPE_F16: return LaunchFlashTyped<__half>(f, s, &vw, &pw);
        case SCA_DTYPE_BF16: return LaunchFlashTyped<__nv_bfloat16>(f, s, &vw, &pw);
        default: break;
    }
    return Fail(SCA_INVALID_ARGUMENT, "flash paged: unsupported dtype id");
}
