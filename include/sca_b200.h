/*
 * sca_b200.h - C ABI of the sm_100a attention kernels (libsca_b200.so).
 *
 * This is the seam between the C++ host layer (sca:: public API, dispatcher, KV cache) and the
 * hand-written CUDA. Every entry point replaces one launch function of the reference and keeps
 * its argument meaning; the reference interface each one stands in for is cited beside it
 * (paths relative to the reference repository).
 *
 * Conventions
 *   - plain pointers and sizes only; `stream` is a cudaStream_t passed as void* (NULL = default
 *     stream); all data pointers are DEVICE pointers unless a comment says "host";
 *   - return value: 0 on success, otherwise a sci::StatusCode value
 *     (4 = InvalidArgument, 5 = NotImplemented, 100 = CudaError, 102 = CudaOutOfMemory);
 *     sca_last_error() returns the message of the last failing call on the calling thread;
 *   - launches are asynchronous with respect to `stream`; launch errors are checked immediately
 *     with cudaGetLastError (reference: src/runtime/launcher.cu:94-100);
 *   - strides are in ELEMENTS, the head dimension is always contiguous (stride 1).
 *   - there is no CPU fallback: without a CUDA device every launch returns a CudaError code.
 */
#ifndef SCA_B200_H_
#define SCA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SCA_ABI __attribute__((visibility("default")))
#else
#define SCA_ABI
#endif

/* dtype ids shared by every entry point (reference: decode_splitk.cuh:34 DecodeDtype,
 * flash_fwd_kernel.cuh:52 dtype_id use the same numbering). */
enum { SCA_DTYPE_F32 = 0, SCA_DTYPE_F16 = 1, SCA_DTYPE_BF16 = 2 };

/* status codes returned by the entry points (values of sci::StatusCode) */
enum {
    SCA_OK = 0,
    SCA_INVALID_ARGUMENT = 4,
    SCA_NOT_IMPLEMENTED = 5,
    SCA_CUDA_ERROR = 100,
    SCA_CUDA_NOT_AVAILABLE = 101,
    SCA_CUDA_OOM = 102,
    SCA_TIMEOUT = 500 /* a bounded wait for other ranks ran out (sci::StatusCode::kDeviceError) */
};

/* Message of the most recent failing call on this thread ("" when none). */
SCA_ABI const char* sca_last_error(void);

/* ------------------------------------------------------------------------------------------ */
/* device probe - replaces src/runtime/device_probe.h:14-36 (already a C ABI in the reference)  */
/* ------------------------------------------------------------------------------------------ */
#define SCA_DEVICE_NAME_MAX 256

typedef struct ScaDeviceProbe {
    char name[SCA_DEVICE_NAME_MAX];
    int major;
    int minor;
    int sm_count;
    unsigned long long smem_per_sm;
    unsigned long long smem_per_block_default;
    unsigned long long smem_per_block_optin;
    unsigned long long regs_per_sm;
    unsigned long long max_threads_per_sm;
    unsigned long long l2_bytes;
    unsigned long long total_mem_bytes;
    unsigned long long free_mem_bytes;
    int cuda_available;
    int binary_has_sm80;   /* kept for source compatibility; always 1 (sm_100a is a superset)   */
    int binary_has_sm90;   /* kept for source compatibility; always 1                           */
} ScaDeviceProbe;          /* same fields, order and size as the reference struct: a caller built
                              against src/runtime/device_probe.h passes its own struct unchanged */

/* Fills `out` for `device_id`. 0 on success, non-zero CUDA error code otherwise. */
SCA_ABI int sca_probe_device(int device_id, ScaDeviceProbe* out);

/* Blackwell additions (no counterpart in the reference): the reference probe followed by what the
 * sm_100a kernels need to know. Kept in a struct of its own so that sca_probe_device never writes
 * past the end of a reference-sized ScaDeviceProbe. */
typedef struct ScaDeviceProbeB200 {
    ScaDeviceProbe base;
    int binary_has_sm100a; /* this library carries sm_100a code (tcgen05 / TMEM / TMA)           */
    int tmem_columns;      /* tensor-memory columns per SM (512 on sm_100), 0 when absent        */
    int max_cluster_size;  /* portable thread-block-cluster limit                                */
} ScaDeviceProbeB200;
SCA_ABI int sca_probe_device_b200(int device_id, ScaDeviceProbeB200* out);
/* cudaMemGetInfo wrapper for the current device. 0 on success. */
SCA_ABI int sca_mem_get_info(unsigned long long* free_bytes, unsigned long long* total_bytes);

/* ------------------------------------------------------------------------------------------ */
/* flash prefill - replaces sca::cuda::LaunchFlashFwd / FlashFwdParams                          */
/* (src/backends/flash/flash_fwd_kernel.cuh:32-60, flash_fwd_launch.cu:100-137)                 */
/* ------------------------------------------------------------------------------------------ */
typedef struct ScaFlashFwdParams {
    const void* q;   /* [batch, heads, seq_q, D] through (q_sb, q_sh, q_ss)                      */
    const void* k;   /* [batch, kv_heads, seq_kv, D] through (k_sb, k_sh, k_ss)                  */
    const void* v;
    void* out;       /* same element type as q, through (o_sb, o_sh, o_ss)                       */
    float* lse;      /* [batch, heads, seq_q] fp32, natural log; may be NULL                     */
    int64_t batch, num_heads, num_kv_heads, seq_q, seq_kv, head_dim;
    int64_t q_sb, q_sh, q_ss;
    int64_t k_sb, k_sh, k_ss;
    int64_t v_sb, v_sh, v_ss;
    int64_t o_sb, o_sh, o_ss;
    float scale;      /* multiplies Q.K; must be > 0                                              */
    int32_t causal;   /* bottom-right aligned: key j visible from query i when j <= i + diagonal  */
    int32_t return_lse;
    int64_t diagonal; /* seq_kv - seq_q for causal, ignored otherwise                             */
    int32_t dtype_id; /* SCA_DTYPE_F16 or SCA_DTYPE_BF16                                          */
} ScaFlashFwdParams;

SCA_ABI int sca_launch_flash_fwd(const ScaFlashFwdParams* params, void* stream);

/* Outcome of earlier flash launches on `device_id` (no counterpart in the reference, whose kernel has no waits
 * that can give up). Every barrier wait inside the flash kernel is bounded; when one runs out the kernel stops,
 * leaves its output undefined and stores 1 + the index of the warp that gave up in a per-device word. The launch
 * call itself has long returned SCA_OK by then, so a caller that wants to know asks here after synchronising the
 * stream: *status_out = 0 (every launch so far ran to completion) or that code; reading clears the word. With
 * SCI_ATTENTION_DEBUG_SYNC=1 the launch call synchronises, checks the word itself and returns SCA_CUDA_ERROR. */
SCA_ABI int sca_flash_status(int device_id, int32_t* status_out);

/* Shared-memory bytes of one flash tile (replaces FlashSmemBytesFor, flash_fwd_kernel.cuh:56).
 * On sm_100a: Q tile + `stages` K tiles + `stages` V tiles, unpadded (TMA 128B swizzle needs no
 * row padding) + 1 KiB of barriers and alignment slack. Returns -1 for a non-positive argument. */
SCA_ABI long long sca_flash_smem_bytes_for(int head_dim, long long elem_bytes, int block_m,
                                           int block_n, int stages);

/* ------------------------------------------------------------------------------------------ */
/* split-K decode (seq_q = 1) - replaces sca::cuda::LaunchDecodeSplitK / DecodeFwdParams          */
/* (src/backends/decode/decode_splitk.cuh:23-57, decode_splitk.cu:229-253)                        */
/* ------------------------------------------------------------------------------------------ */
typedef struct ScaDecodeStrides {
    int64_t s_b, s_h, s_s;
} ScaDecodeStrides;

typedef struct ScaDecodeFwdParams {
    const void* q;      /* [batch, heads, 1, D]                                                  */
    const void* k;      /* contiguous: [batch, kv_heads, seq_kv, D] through k_stride;            */
    const void* v;      /* paged: origin of one layer's pool [blocks, block_size, kv_heads, D]   */
    void* out;          /* [batch, heads, 1, D] through o_stride                                  */
    float* partial_m;   /* [batch*heads*num_splits]      running max (natural units, scaled)      */
    float* partial_l;   /* [batch*heads*num_splits]      sum of exp(s - m)                        */
    float* partial_o;   /* [batch*heads*num_splits, D]   sum of exp(s - m) * V (unnormalised)     */
    int64_t batch, num_heads, num_kv_heads, seq_kv, head_dim, num_splits;
    ScaDecodeStrides q_stride, k_stride, v_stride, o_stride;
    float scale;
    int32_t dtype;      /* SCA_DTYPE_*                                                            */
    /* page-table indirection; page_table == NULL selects the contiguous path */
    const int32_t* page_table; /* [batch, max_blocks_per_seq], -1 = unmapped (weight 0)           */
    int64_t block_size, max_blocks_per_seq, num_kv_blocks;
    const int32_t* seq_lens;   /* [batch] or NULL (= seq_kv for every sequence)                   */
} ScaDecodeFwdParams;          /* 248 bytes: field for field the reference's DecodeFwdParams      */

/* partial kernel + merge kernel on `stream` */
SCA_ABI int sca_launch_decode_splitk(const ScaDecodeFwdParams* params, void* stream);
/* same, but requires the page-table fields (decode_splitk.cu:245-253) */
SCA_ABI int sca_launch_decode_splitk_paged(const ScaDecodeFwdParams* params, void* stream);

/* paged attention - replaces sca::cuda::LaunchPagedAttention / PagedDecodeParams
 * (src/backends/paged/paged_attention.cuh:21-32, paged_attention.cu:12-22) */
typedef struct ScaPagedDecodeParams {
    ScaDecodeFwdParams base;
    const int32_t* page_table;
    int64_t block_size, max_blocks_per_seq, num_kv_blocks;
} ScaPagedDecodeParams;

SCA_ABI int sca_launch_paged_attention(const ScaPagedDecodeParams* params, void* stream);

/* Paged attention with a scheduling hint (no counterpart in the reference). `seq_order` is a device
 * int32 [batch] permutation of 0 .. batch-1; thread blocks are handed out in that order, so listing the
 * longest sequences first shortens the tail of a ragged batch. Results do not depend on it; entries
 * outside 0 .. batch-1 are ignored (their thread blocks do nothing). NULL = sequence order, i.e. exactly
 * sca_launch_paged_attention. */
SCA_ABI int sca_launch_paged_attention_ordered(const ScaPagedDecodeParams* params,
                                               const int32_t* seq_order, void* stream);

/* Sequence-split decode across GPUs (no counterpart in the reference, which is single-GPU).
 * sca_launch_decode_triples runs the partial kernel and merges this GPU's splits WITHOUT the
 * final normalisation: triples[(b*heads + h) * (2 + D)] = { m, l, O[D] } (fp32). After the
 * triples of all ranks have been gathered ([ranks][batch*heads][2 + D]),
 * sca_launch_merge_triples applies the same merge rule (decode_splitk.cu:143-182) across ranks
 * and writes the normalised output. `out_dtype` is SCA_DTYPE_*. */
SCA_ABI int sca_launch_decode_triples(const ScaDecodeFwdParams* params, float* triples, void* stream);
SCA_ABI int sca_launch_merge_triples(const float* gathered, int64_t ranks, int64_t rows,
                                     int64_t head_dim, void* out, int32_t out_dtype, void* stream);

/* Packed variable-length prefill in one launch - replaces the per-sequence launch loop of
 * FlashBackend::ForwardVarlen (src/backends/flash/flash_backend.cpp:312-363). q / out are packed
 * [total_q, num_heads, head_dim], k / v [total_kv, num_kv_heads, head_dim]; the offsets are HOST arrays of
 * num_seqs + 1 int32 (as in the reference API); causal masks are bottom-right aligned per sequence.
 * `workspace` is device memory of at least sca_flash_varlen_workspace_bytes(num_seqs, total_q) bytes that
 * must stay untouched until the launch has finished. */
typedef struct ScaFlashVarlenParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    int64_t total_q, total_kv, num_heads, num_kv_heads, head_dim, num_seqs;
    const int32_t* cu_seqlens_q;
    const int32_t* cu_seqlens_kv;
    float scale;
    int32_t causal;
    int32_t dtype_id;
    void* workspace;
    int64_t workspace_bytes;
} ScaFlashVarlenParams;
SCA_ABI long long sca_flash_varlen_workspace_bytes(int64_t num_seqs, int64_t total_q);
SCA_ABI int sca_launch_flash_varlen(const ScaFlashVarlenParams* params, void* stream);

/* Chunked prefill over a paged KV cache in one launch (no counterpart in the reference, which lists it as the step
 * after the packed variable-length prefill: docs/flash_attention.md:95). A batch of sequences, each with S_q new
 * query tokens and S_kv >= S_q tokens already in the cache (the new ones included, appended beforehand):
 *   q / out  packed [total_q, num_heads, head_dim];  cu_seqlens_q: HOST int32 [num_seqs + 1]
 *   k_pool / v_pool  one layer of the pool, [num_blocks, block_size, num_kv_heads, head_dim]
 *   page_table  DEVICE int32 [num_seqs, max_blocks_per_seq]; seq_lens_kv: HOST int32 [num_seqs] = S_kv per sequence
 * Keys are fetched page by page (one TMA box per page, block_size in {8, 16, 32, 64}); an entry < 0 or >= num_blocks
 * contributes weight 0, as in the decode kernel (src/backends/paged/page_table.cuh:18-36). The causal mask is
 * bottom-right aligned per sequence: query i of S_q sees keys j <= i + (S_kv - S_q).
 * `workspace`: device memory of sca_flash_varlen_workspace_bytes(num_seqs, total_q) bytes, untouched until the launch
 * has finished. */
typedef struct ScaFlashPagedParams {
    const void* q;
    void* out;
    const void* k_pool;
    const void* v_pool;
    const int32_t* page_table;
    int64_t total_q, num_heads, num_kv_heads, head_dim, num_seqs;
    int64_t num_blocks, block_size, max_blocks_per_seq;
    const int32_t* cu_seqlens_q;
    const int32_t* seq_lens_kv;
    float scale;
    int32_t causal;
    int32_t dtype_id;
    void* workspace;
    int64_t workspace_bytes;
} ScaFlashPagedParams;
SCA_ABI int sca_launch_flash_paged(const ScaFlashPagedParams* params, void* stream);

/* Sequence-split decode without a library collective (no counterpart in the reference).
 *
 * Every rank creates one exchange buffer (sca_peer_buffer_bytes / _create), hands its 64-byte handle to
 * the other ranks by any host channel, and maps theirs (_open). sca_launch_seqsplit_exchange then does,
 * in one kernel: merge of this rank's split-K partials (as written by sca_launch_decode_splitk's partial
 * kernel: m, l [rows][num_splits], O [rows][num_splits][D], fp32), store of the merged triples into the
 * buffers of all ranks over NVLink, a bounded wait until all ranks have done the same for `epoch`, and
 * the final merge into out [rows][D] (same rule as decode_splitk.cu:143-182, applied across ranks).
 * `epoch` starts at 1 and grows by 1 per call, identically on every rank; calls of one rank must be
 * ordered (one stream). With epoch = 0 the kernel counts the calls itself in the buffer (every rank must then
 * use 0 on every call): the parameters no longer change from step to step, so the step can be captured in a
 * CUDA graph and replayed. peer_buffers[rank] is the rank's own buffer. If a peer does not show up within
 * about a second the kernel gives up, fills `out` with NaN and records the step in the status word that
 * sca_peer_exchange_status reads back (0 = all waits were satisfied). One process per GPU: ranks that
 * share a GPU would wait on kernels that cannot run at the same time. */
#define SCA_PEER_MAX_RANKS 16
#define SCA_PEER_HANDLE_BYTES 64
typedef struct ScaSeqSplitExchange {
    void* peer_buffers[SCA_PEER_MAX_RANKS];
    int32_t rank, world;
    int64_t rows, head_dim, num_splits; /* rows = batch * query heads; head_dim <= 256 */
    uint32_t epoch;
    const float* partial_m;
    const float* partial_l;
    const float* partial_o;
    void* out;
    int32_t out_dtype; /* SCA_DTYPE_* */
} ScaSeqSplitExchange;

/* the split-K partial kernel alone (fills params->partial_m / _l / _o; `out` is not used) */
SCA_ABI int sca_launch_decode_partials(const ScaDecodeFwdParams* params, void* stream);
SCA_ABI long long sca_peer_buffer_bytes(int32_t world, int64_t rows, int64_t head_dim);
SCA_ABI int sca_peer_buffer_create(int64_t bytes, void** device_ptr, unsigned char* handle_out);
SCA_ABI int sca_peer_buffer_open(const unsigned char* handle_in, void** device_ptr);
SCA_ABI int sca_peer_buffer_close(void* device_ptr);   /* a buffer mapped with _open */
SCA_ABI int sca_peer_buffer_destroy(void* device_ptr); /* a buffer made with _create */
/* 0 = every wait so far was satisfied; otherwise the epoch (step number, from 1) of the first launch that gave up
 * waiting for a peer - that launch wrote NaN instead of a result. The value stays until sca_peer_exchange_clear.
 * Both calls synchronise with the device. */
SCA_ABI int sca_peer_exchange_status(const void* local_buffer, int32_t* status_out);
SCA_ABI int sca_peer_exchange_clear(void* local_buffer);
SCA_ABI int sca_launch_seqsplit_exchange(const ScaSeqSplitExchange* params, void* stream);

/* Multi-GPU plumbing with bounded waits (no counterpart in the reference, which is single-GPU): a NCCL communicator
 * for the all-gather of the (m, l, O) triples between sca_launch_decode_triples and sca_launch_merge_triples.
 * NCCL is loaded at run time (libnccl.so.2, or the file the environment variable SCA_NCCL_LIBRARY names); without it
 * the calls return SCA_NOT_IMPLEMENTED. One process per GPU; rank 0 makes the id (sca_mgpu_unique_id) and hands its
 * 128 bytes to the other ranks over any host channel. The communicator is non-blocking: sca_mgpu_init waits at most
 * `timeout_ms` for the other ranks (<= 0: one minute), sca_mgpu_allgather_triples at most `timeout_ms` for the collective to complete
 * (timeout_ms <= 0: it only enqueues and returns; the caller orders later work on `stream`). When a limit passes,
 * the communicator is aborted - which also releases a collective kernel that is waiting for a peer - and the call
 * returns SCA_TIMEOUT; an aborted communicator only accepts sca_mgpu_destroy.
 *   gathered [world][floats_per_rank] <- mine [floats_per_rank] of every rank, rank-major (fp32, device memory). */
#define SCA_MGPU_ID_BYTES 128
SCA_ABI int sca_mgpu_unique_id(unsigned char* id_out);
SCA_ABI int sca_mgpu_init(const unsigned char* id, int32_t rank, int32_t world, int32_t timeout_ms, void** comm_out);
SCA_ABI int sca_mgpu_allgather_triples(void* comm, const float* mine, float* gathered, int64_t floats_per_rank,
                                       void* stream, int32_t timeout_ms);
SCA_ABI int sca_mgpu_abort(void* comm);
SCA_ABI int sca_mgpu_destroy(void* comm);

/* Allocation-free split-K decode. No counterpart in the reference.
 *
 * For callers that are not allowed to obtain device memory around the call: code running while a
 * stream is being captured, serving loops that have handed every free byte of the GPU to their own
 * pool (so a cudaMalloc would fail or stall the device), and hosts that forbid allocation after
 * start-up. It computes exactly what sca_launch_decode_splitk computes, but ignores
 * params->partial_m / partial_l / partial_o (they may be NULL) and keeps the split-K partials in a
 * fixed array inside the library: 4 Mi floats (16 MiB) that every GPU using the library holds until
 * the process ends. The call itself uses no cudaMalloc, cudaFree or allocating library routine.
 *
 * Limit: batch * num_heads * num_splits * (2 + head_dim) <= 4 194 304 floats, otherwise
 * SCA_INVALID_ARGUMENT with the required size in the message.
 * The first call on each device looks up the array's device address (one cudaGetSymbolAddress with
 * that device current); make that first call before starting any stream capture.
 * All calls share the one array and it keeps the previous call's contents; nothing in it has to start
 * at zero because every (batch, head, split) entry is rewritten before it is read. Two calls whose
 * kernels may overlap on the GPU (different streams without an ordering between them) race on it. */
SCA_ABI int sca_launch_decode_splitk_static(const ScaDecodeFwdParams* params, void* stream);

/* ------------------------------------------------------------------------------------------ */
/* reference-level backends kept for API completeness (functional, not tuned).                    */
/* Parameter block of both: ScaFlashFwdParams; dtype_id may also be SCA_DTYPE_F32.               */
/* ------------------------------------------------------------------------------------------ */
/* Level-1 naive attention - replaces LaunchNaiveForward (src/backends/naive/attention_naive.cuh:28-60): scores,
 * row softmax and P.V as three kernels with the score matrix MATERIALISED in `scores`, fp32
 * [batch, heads, seq_q, seq_kv] = sca_naive_score_bytes(...) bytes of caller-provided device memory (the
 * reference's NaiveFwdParams::scores). */
SCA_ABI long long sca_naive_score_bytes(int64_t batch, int64_t heads, int64_t seq_q, int64_t seq_kv);
SCA_ABI int sca_launch_naive_forward(const ScaFlashFwdParams* params, float* scores, void* stream);
/* One SIMT kernel with a running softmax and no score matrix - replaces LaunchTiledForward
 * (src/backends/tiled/attention_tiled.cuh:57); it is also the fp32 case of the decode partial kernel. */
SCA_ABI int sca_launch_simt_forward(const ScaFlashFwdParams* params, void* stream);

/* ------------------------------------------------------------------------------------------ */
/* KV cache data movement - replaces LaunchKvAppend / LaunchKvResetBlock / LaunchKvGather         */
/* (src/kv_cache/kv_cache_kernels.cuh:20-33, kv_cache_layout.cuh:24-38)                           */
/* ------------------------------------------------------------------------------------------ */
typedef struct ScaKvCacheShape {
    int64_t num_blocks, block_size, num_kv_heads, head_dim;
} ScaKvCacheShape;

/* rows [num_tokens, kv_heads, D] -> slot = block * block_size + offset; slot < 0 and
 * block >= num_blocks are skipped */
SCA_ABI int sca_launch_kv_append(void* layer_k, void* layer_v, const void* k_new, const void* v_new,
                                 const int32_t* slot_mapping, int64_t num_tokens,
                                 const ScaKvCacheShape* shape, int64_t elem_bytes, void* stream);
/* zeroes the listed blocks of K and V; ids < 0 or >= num_blocks are skipped. `block_ids` (here and in
 * sca_launch_kv_gather) is normally device memory; a list in host memory is accepted too and copied to the
 * device first, because the reference's PagedKVCache::ResetSeq passes the ids of a std::vector
 * (src/kv_cache/paged_kv_cache.cpp:150-156). */
SCA_ABI int sca_launch_kv_reset_block(void* layer_k, void* layer_v, const int32_t* block_ids,
                                      int64_t num_blocks, const ScaKvCacheShape* shape,
                                      int64_t elem_bytes, void* stream);
/* copies the listed blocks into a contiguous buffer; invalid ids gather zeros */
SCA_ABI int sca_launch_kv_gather(const void* layer, const int32_t* block_ids, int64_t num_blocks,
                                 void* out, const ScaKvCacheShape* shape, int64_t elem_bytes,
                                 void* stream);

/* Multi-sequence append (no counterpart in the reference, whose PagedKVCache::AppendTokens issues
 * one launch and one blocking 4-byte upload per sequence, src/kv_cache/paged_kv_cache.cpp:52-142).
 * One new token per sequence: slot = page_table[s, pos/bs] * bs + pos % bs with pos = seq_lens[s] - 1
 * (seq_lens already includes the new token). Sequences whose page is unmapped are skipped. */
SCA_ABI int sca_launch_kv_append_batched(void* layer_k, void* layer_v, const void* k_new,
                                         const void* v_new, const int32_t* page_table,
                                         const int32_t* seq_lens, int64_t num_seqs,
                                         int64_t max_blocks_per_seq, const ScaKvCacheShape* shape,
                                         int64_t elem_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SCA_B200_H_ */
