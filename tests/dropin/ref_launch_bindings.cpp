// The reference's launch layer re-implemented as forwarding calls into libsca_b200.so.
//
// This is the file a maintainer of the reference adds in place of its CUDA translation units
// (src/backends/*/*.cu, src/kv_cache/kv_cache_kernels.cu): one definition per function of
// src/backends/backends_stub.cpp:30-56 and src/kv_cache/kv_cache_kernels_stub.cpp:27-40. It is compiled here
// against the reference's OWN headers (the include path comes from the build script), so every field
// name below is checked by the compiler against the reference PODs, and the static_asserts pin the
// layouts the C ABI promises. The probe (sca_probe_device / sca_mem_get_info) needs no binding: the
// library exports the reference's C symbols with the reference's struct.
//
// Parameter blocks are copied field by field: the C structs use int32 where the reference uses bool and
// may grow trailing fields, so no pointer cast between the two families is ever valid.
#include <cstddef>
#include <cstdint>

#include "backends/decode/decode_splitk.cuh"
#include "backends/flash/flash_fwd_kernel.cuh"
#include "backends/naive/attention_naive.cuh"
#include "backends/paged/paged_attention.cuh"
#include "backends/tiled/attention_tiled.cuh"
#include "device/stream.hpp"
#include "kv_cache/kv_cache_kernels.cuh"
#include "kv_cache/kv_cache_layout.cuh"
#include "sca_b200.h"

namespace {

using sca::cuda::DecodeFwdParams;
using sca::cuda::FlashFwdParams;
using sca::cuda::KVCacheShape;
using sca::cuda::PagedDecodeParams;

// ---- layouts the C ABI mirrors (reference: decode_splitk.cuh:23-51, paged_attention.cuh:21-27,
// kv_cache_layout.cuh:24-29, flash_fwd_kernel.cuh:32-53) --------------------------------------------------
static_assert(sizeof(DecodeFwdParams) == 248 && sizeof(ScaDecodeFwdParams) == sizeof(DecodeFwdParams),
              "ScaDecodeFwdParams must have the size of the reference's DecodeFwdParams");
#define SCA_SAME_OFFSET(ref_t, c_t, field) \
    static_assert(offsetof(ref_t, field) == offsetof(c_t, field), "field offset differs: " #field)
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, q);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, out);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, partial_m);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, partial_o);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, batch);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, num_splits);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, q_stride);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, o_stride);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, scale);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, dtype);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, page_table);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, block_size);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, num_kv_blocks);
SCA_SAME_OFFSET(DecodeFwdParams, ScaDecodeFwdParams, seq_lens);
static_assert(sizeof(PagedDecodeParams) == sizeof(ScaPagedDecodeParams), "PagedDecodeParams size");
SCA_SAME_OFFSET(PagedDecodeParams, ScaPagedDecodeParams, page_table);
SCA_SAME_OFFSET(PagedDecodeParams, ScaPagedDecodeParams, num_kv_blocks);
static_assert(sizeof(KVCacheShape) == sizeof(ScaKvCacheShape) && sizeof(KVCacheShape) == 32, "KVCacheShape size");
SCA_SAME_OFFSET(KVCacheShape, ScaKvCacheShape, num_blocks);
SCA_SAME_OFFSET(KVCacheShape, ScaKvCacheShape, head_dim);
// FlashFwdParams: the pointer / extent / stride prefix is identical; from `causal` on the reference packs two
// bools where C has two int32, so the blocks differ in size on purpose and are only ever copied by field.
SCA_SAME_OFFSET(FlashFwdParams, ScaFlashFwdParams, lse);
SCA_SAME_OFFSET(FlashFwdParams, ScaFlashFwdParams, batch);
SCA_SAME_OFFSET(FlashFwdParams, ScaFlashFwdParams, o_ss);
SCA_SAME_OFFSET(FlashFwdParams, ScaFlashFwdParams, scale);
static_assert(sizeof(FlashFwdParams) == 208 && sizeof(ScaFlashFwdParams) == 216, "FlashFwdParams sizes");
// the probe struct of src/runtime/device_probe.h (checked against that header in probe_layout_check.cpp)
static_assert(sizeof(ScaDeviceProbe) == 352, "probe struct size");
static_assert(offsetof(ScaDeviceProbe, major) == 256 && offsetof(ScaDeviceProbe, smem_per_sm) == 272 &&
                  offsetof(ScaDeviceProbe, free_mem_bytes) == 328 && offsetof(ScaDeviceProbe, cuda_available) == 336 &&
                  offsetof(ScaDeviceProbe, binary_has_sm90) == 344,
              "probe struct offsets");

sci::Status FromCode(int rc) {
    if (rc == 0) return sci::Status::Ok();
    return sci::Status(static_cast<sci::StatusCode>(rc), sca_last_error());
}

// nullptr means "the current stream" everywhere in the reference (src/runtime/launcher.cu:44-47)
void* Handle(sci::Stream* stream) { return stream != nullptr ? stream->handle() : sci::Stream::GetCurrent().handle(); }

template <typename Strides>
ScaDecodeStrides CopyStrides(const Strides& s) {
    return ScaDecodeStrides{s.s_b, s.s_h, s.s_s};
}

ScaDecodeFwdParams CopyDecode(const DecodeFwdParams& p) {
    ScaDecodeFwdParams c{};
    c.q = p.q;
    c.k = p.k;
    c.v = p.v;
    c.out = p.out;
    c.partial_m = p.partial_m;
    c.partial_l = p.partial_l;
    c.partial_o = p.partial_o;
    c.batch = p.batch;
    c.num_heads = p.num_heads;
    c.num_kv_heads = p.num_kv_heads;
    c.seq_kv = p.seq_kv;
    c.head_dim = p.head_dim;
    c.num_splits = p.num_splits;
    c.q_stride = CopyStrides(p.q_stride);
    c.k_stride = CopyStrides(p.k_stride);
    c.v_stride = CopyStrides(p.v_stride);
    c.o_stride = CopyStrides(p.o_stride);
    c.scale = p.scale;
    c.dtype = static_cast<int32_t>(p.dtype);
    c.page_table = p.page_table;
    c.block_size = p.block_size;
    c.max_blocks_per_seq = p.max_blocks_per_seq;
    c.num_kv_blocks = p.num_kv_blocks;
    c.seq_lens = p.seq_lens;
    return c;
}

// NaiveFwdParams and TiledFwdParams carry the same fields as the flash block (NaiveFwdParams adds the score
// workspace, passed separately).
template <typename P>
ScaFlashFwdParams CopyStridedForward(const P& p, int32_t dtype_id) {
    ScaFlashFwdParams c{};
    c.q = p.q;
    c.k = p.k;
    c.v = p.v;
    c.out = p.out;
    c.lse = p.lse;
    c.batch = p.batch;
    c.num_heads = p.num_heads;
    c.num_kv_heads = p.num_kv_heads;
    c.seq_q = p.seq_q;
    c.seq_kv = p.seq_kv;
    c.head_dim = p.head_dim;
    c.q_sb = p.q_stride.s_b; c.q_sh = p.q_stride.s_h; c.q_ss = p.q_stride.s_s;
    c.k_sb = p.k_stride.s_b; c.k_sh = p.k_stride.s_h; c.k_ss = p.k_stride.s_s;
    c.v_sb = p.v_stride.s_b; c.v_sh = p.v_stride.s_h; c.v_ss = p.v_stride.s_s;
    c.o_sb = p.o_stride.s_b; c.o_sh = p.o_stride.s_h; c.o_ss = p.o_stride.s_s;
    c.scale = p.scale;
    c.causal = p.causal ? 1 : 0;
    c.return_lse = p.return_lse ? 1 : 0;
    c.diagonal = p.diagonal;
    c.dtype_id = dtype_id;
    return c;
}

ScaKvCacheShape CopyShape(const KVCacheShape& s) {
    return ScaKvCacheShape{s.num_blocks, s.block_size, s.num_kv_heads, s.head_dim};
}

}  // namespace

namespace sca {
namespace cuda {

sci::Status LaunchFlashFwd(const FlashFwdParams& p, sci::Stream* stream) {
    ScaFlashFwdParams c{};
    c.q = p.q;
    c.k = p.k;
    c.v = p.v;
    c.out = p.out;
    c.lse = p.lse;
    c.batch = p.batch;
    c.num_heads = p.num_heads;
    c.num_kv_heads = p.num_kv_heads;
    c.seq_q = p.seq_q;
    c.seq_kv = p.seq_kv;
    c.head_dim = p.head_dim;
    c.q_sb = p.q_sb; c.q_sh = p.q_sh; c.q_ss = p.q_ss;
    c.k_sb = p.k_sb; c.k_sh = p.k_sh; c.k_ss = p.k_ss;
    c.v_sb = p.v_sb; c.v_sh = p.v_sh; c.v_ss = p.v_ss;
    c.o_sb = p.o_sb; c.o_sh = p.o_sh; c.o_ss = p.o_ss;
    c.scale = p.scale;
    c.causal = p.causal ? 1 : 0;
    c.return_lse = p.return_lse ? 1 : 0;
    c.diagonal = p.diagonal;
    c.dtype_id = p.dtype_id;
    return FromCode(sca_launch_flash_fwd(&c, Handle(stream)));
}

int64_t FlashSmemBytesFor(int32_t head_dim, int64_t elem_bytes, int32_t block_m, int32_t block_n, int32_t stages) {
    return sca_flash_smem_bytes_for(head_dim, elem_bytes, block_m, block_n, stages);
}

sci::Status LaunchDecodeSplitK(const DecodeFwdParams& p, sci::Stream* stream) {
    const ScaDecodeFwdParams c = CopyDecode(p);
    return FromCode(sca_launch_decode_splitk(&c, Handle(stream)));
}

sci::Status LaunchDecodeSplitKPaged(const DecodeFwdParams& p, sci::Stream* stream) {
    const ScaDecodeFwdParams c = CopyDecode(p);
    return FromCode(sca_launch_decode_splitk_paged(&c, Handle(stream)));
}

sci::Status LaunchPagedAttention(const PagedDecodeParams& p, sci::Stream* stream) {
    ScaPagedDecodeParams c{};
    c.base = CopyDecode(p.base);
    c.page_table = p.page_table;
    c.block_size = p.block_size;
    c.max_blocks_per_seq = p.max_blocks_per_seq;
    c.num_kv_blocks = p.num_kv_blocks;
    return FromCode(sca_launch_paged_attention(&c, Handle(stream)));
}

sci::Status LaunchNaiveForward(const NaiveFwdParams& p, sci::Stream* stream) {
    const ScaFlashFwdParams c = CopyStridedForward(p, static_cast<int32_t>(p.dtype));
    return FromCode(sca_launch_naive_forward(&c, p.scores, Handle(stream)));
}

sci::Status LaunchTiledForward(const TiledFwdParams& p, sci::Stream* stream, int32_t, int32_t, int32_t) {
    const ScaFlashFwdParams c = CopyStridedForward(p, static_cast<int32_t>(p.dtype));
    return FromCode(sca_launch_simt_forward(&c, Handle(stream)));
}

// The kernel behind LaunchTiledForward keeps its row state in registers and uses no shared memory. The
// reference's tile selector (src/backends/tiled/tiled_backend.cpp:60-86) only accepts a positive byte count
// below the device limit, so the binding reports one 16-byte granule for every valid geometry.
int64_t TiledSmemBytes(int32_t head_dim, int64_t elem_bytes, int32_t block_m, int32_t block_n) {
    if (head_dim <= 0 || elem_bytes <= 0 || block_m <= 0 || block_n <= 0) return -1;
    return 16;
}

sci::Status LaunchKvAppend(void* layer_k, void* layer_v, const void* k_new, const void* v_new,
                           const int32_t* slot_mapping, int64_t num_tokens, const KVCacheShape& shape,
                           int64_t elem_bytes, sci::Stream* stream) {
    const ScaKvCacheShape c = CopyShape(shape);
    return FromCode(sca_launch_kv_append(layer_k, layer_v, k_new, v_new, slot_mapping, num_tokens, &c, elem_bytes,
                                         Handle(stream)));
}

sci::Status LaunchKvResetBlock(void* layer_k, void* layer_v, const int32_t* block_ids, int64_t num_blocks,
                               const KVCacheShape& shape, int64_t elem_bytes, sci::Stream* stream) {
    const ScaKvCacheShape c = CopyShape(shape);
    return FromCode(sca_launch_kv_reset_block(layer_k, layer_v, block_ids, num_blocks, &c, elem_bytes, Handle(stream)));
}

sci::Status LaunchKvGather(const void* layer, const int32_t* block_ids, int64_t num_blocks, void* out,
                           const KVCacheShape& shape, int64_t elem_bytes, sci::Stream* stream) {
    const ScaKvCacheShape c = CopyShape(shape);
    return FromCode(sca_launch_kv_gather(layer, block_ids, num_blocks, out, &c, elem_bytes, Handle(stream)));
}

}  // namespace cuda
}  // namespace sca
