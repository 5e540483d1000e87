"""Python harness over the C ABI: the same operators the C++ host layer exposes
(sca::decode_attention, sca::paged_attention, sca::flash_attention, KVCache::Append/Reset/Gather),
taking torch CUDA tensors only as device memory + stream providers.

Argument meaning follows the reference's public API (include/scicompute_attention/*.hpp):
q is [B, H_q, S_q, D] (layout "bhsd") or [B, S_q, H_q, D] ("bshd"); k/v likewise with H_kv;
outputs are always freshly allocated contiguous BHSD tensors.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from ._lib import (DTYPE_BF16, DTYPE_F16, DTYPE_F32, DecodeFwdParams, DecodeStrides, FlashFwdParams,
                   KvCacheShape, PagedDecodeParams, check, lib)

MAX_SPLITS = 64          # upper bound of the automatic split count on B200

_DTYPE_IDS = {torch.float32: DTYPE_F32, torch.float16: DTYPE_F16, torch.bfloat16: DTYPE_BF16}
_scratch: dict[tuple[int, int], torch.Tensor] = {}
_sm_count: dict[int, int] = {}


def dtype_id(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_IDS[dtype]
    except KeyError:
        raise _lib.ScaError(4, f"dtype={dtype} (supported: float32, float16, bfloat16)")


def _stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise _lib.ScaError(5, "device=cpu (attention kernels run on CUDA devices only; there is no CPU path)")


def sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def acquire_scratch_fp32(elements: int, device: torch.device, kind: int = 1) -> torch.Tensor:
    """Process-wide grow-only fp32 scratch per (device, kind); same growth rule as the reference's
    pool (src/runtime/scratch_pool.cpp:38-60): 1.25 x request + 1024 elements."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, kind)
    cur = _scratch.get(key)
    if cur is None or cur.numel() < elements:
        grown = int(elements * 1.25) + 1024
        cur = torch.empty(grown, dtype=torch.float32, device=device)
        _scratch[key] = cur
    return cur


DECODE_STEP_TOKENS = 64  # tokens one CTA of the decode kernel consumes per step (4 warps x 16)


def slots_for_schedule(column_steps: int, longest_steps: int, columns: int, sms: int) -> int:
    """Partial slots per row for the decode kernel's schedule: one wave of resident CTAs (2 per SM), the same number
    for every (kv head, head chunk) column; the CTAs of a column split its list of 64-token steps (sequence after
    sequence) into equal contiguous shares, and a sequence cut by share boundaries yields one partial per piece.
    Needed: the pieces of the longest sequence, plus one for a share that starts in its middle. (The reference's rule,
    one CTA per fixed split, is ceil(seq_kv / 512) capped at 16: src/backends/decode/decode_config.hpp:24-31.)"""
    if column_steps <= 0 or longest_steps <= 1:
        return 1
    resident = 2 * (sms if sms > 0 else 148)
    sharers = max(1, resident // max(1, columns))
    per_cta = max(1, -(-column_steps // sharers))
    return max(2, min(-(-longest_steps // per_cta) + 1, MAX_SPLITS))


def splits_for(seq_kv: int, batch: int, num_kv_heads: int, group: int, sms: int) -> int:
    """Automatic slot count for equally long sequences."""
    if seq_kv <= 0:
        return 1
    steps = -(-seq_kv // DECODE_STEP_TOKENS)
    return slots_for_schedule(max(1, batch) * steps, steps, num_kv_heads * ((group + 15) // 16), sms)


def paged_splits_for(typical_len: int, num_seqs: int, num_kv_heads: int, group: int, sms: int, longest_len: int = 0) -> int:
    """Slot count for a ragged batch of mean length `typical_len`; the longest sequence is taken as twice the mean
    unless `longest_len` says otherwise."""
    if typical_len <= 0:
        return 1
    steps = -(-typical_len // DECODE_STEP_TOKENS)
    longest = -(-longest_len // DECODE_STEP_TOKENS) if longest_len > 0 else 2 * steps
    return slots_for_schedule(max(1, num_seqs) * steps, longest, num_kv_heads * ((group + 15) // 16), sms)


def _strides(layout: str, seq: int, heads: int, d: int) -> tuple[int, int, int]:
    """(s_b, s_h, s_s) in elements (reference: detail/layout_traits.hpp:32-45)."""
    if layout == "bhsd":
        return heads * seq * d, seq * d, d
    if layout == "bshd":
        return seq * heads * d, d, heads * d
    raise _lib.ScaError(4, f"layout={layout} (supported: bhsd, bshd)")


def _dims(t: torch.Tensor, layout: str):
    if t.dim() != 4:
        raise _lib.ScaError(4, f"tensor ndims={t.dim()} (expected 4)")
    if not t.is_contiguous():
        raise _lib.ScaError(4, "non-contiguous input rejected; pass a contiguous tensor")
    if layout == "bhsd":
        b, h, s, d = t.shape
    else:
        b, s, h, d = t.shape
    return b, h, s, d


def effective_scale(scale, head_dim: int) -> float:
    """cfg.scale > 0 wins, otherwise float(1 / sqrt(double(D))) (reference: api_validate.cpp:31-35)."""
    if scale is not None and scale > 0:
        return float(scale)
    return float(torch.tensor(1.0 / math.sqrt(float(head_dim)), dtype=torch.float32).item())


# ------------------------------------------------------------------------------------------------
# decode / paged
# ------------------------------------------------------------------------------------------------
def decode_attention(q, k, v, *, scale=None, num_splits: int = 0, layout: str = "bhsd",
                     seq_lens=None, stream=None, return_stats: bool = False):
    """Split-K decode over a contiguous KV cache; S_q must be 1 (sca::decode_attention)."""
    _require_cuda(q, k, v)
    b, hq, sq, d = _dims(q, layout)
    bk, hkv, skv, dk = _dims(k, layout)
    if sq != 1:
        raise _lib.ScaError(5, f"decode backend requires seq_q=1; seq_q={sq} belongs to the flash backend")
    if (bk, dk) != (b, d) or tuple(v.shape) != tuple(k.shape) or q.dtype != k.dtype or q.dtype != v.dtype:
        raise _lib.ScaError(4, "q/k/v shape or dtype mismatch")
    if hq % hkv != 0:
        raise _lib.ScaError(4, f"num_heads={hq} % num_kv_heads={hkv} != 0")
    splits = min(num_splits, MAX_SPLITS) if num_splits > 0 else splits_for(skv, b, hkv, hq // hkv, sm_count(q.device))
    base = b * hq * splits
    ws = acquire_scratch_fp32(base * (2 + d), q.device)
    out = torch.empty((b, hq, 1, d), dtype=q.dtype, device=q.device)

    p = DecodeFwdParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.partial_m = ws.data_ptr()
    p.partial_l = ws.data_ptr() + 4 * base
    p.partial_o = ws.data_ptr() + 8 * base
    p.batch, p.num_heads, p.num_kv_heads, p.seq_kv, p.head_dim, p.num_splits = b, hq, hkv, skv, d, splits
    p.q_stride = DecodeStrides(*_strides(layout, 1, hq, d))
    p.k_stride = DecodeStrides(*_strides(layout, skv, hkv, d))
    p.v_stride = p.k_stride
    p.o_stride = DecodeStrides(*_strides("bhsd", 1, hq, d))
    p.scale = effective_scale(scale, d)
    p.dtype = dtype_id(q.dtype)
    p.page_table = None
    p.seq_lens = seq_lens.data_ptr() if seq_lens is not None else None
    check(lib().sca_launch_decode_splitk(C.byref(p), _stream_ptr(stream)))
    if return_stats:
        return out, {"num_splits": splits, "workspace_bytes": base * (2 + d) * 4}
    return out


def paged_attention(q, k_pool, v_pool, page_table, seq_lens, *, block_size: int, scale=None,
                    num_splits: int = 0, typical_len: int = 0, longest_len: int = 0, stream=None,
                    return_stats: bool = False, seq_order=None):
    """Decode over page-table-indirected K/V (sca::paged_attention).

    q [num_seqs, H_q, 1, D]; pools [num_blocks, block_size, H_kv, D]; page_table int32
    [num_seqs, max_blocks_per_seq] on the device (-1 = unmapped); seq_lens int32 [num_seqs] on the
    device or None (every sequence then scans max_blocks_per_seq * block_size positions).
    `typical_len` / `longest_len` are optional host-side hints (the mean and the maximum sequence length, which a
    cache object tracks anyway) used only to size the partial scratch: enough slots for an even schedule. seq_order
    is accepted for compatibility and ignored: the kernel balances the work itself."""
    _require_cuda(q, k_pool, v_pool, page_table, seq_lens)
    if q.dim() != 4:
        raise _lib.ScaError(4, f"paged_attention expects q=[num_seqs, H_q, seq_q, D]; got ndims={q.dim()}")
    s, hq, sq, d = q.shape
    if sq != 1:
        raise _lib.ScaError(5, f"paged attention implements the decode form only (seq_q=1); got seq_q={sq}")
    nblk, bs, hkv, dk = k_pool.shape
    if bs != block_size or dk != d or tuple(v_pool.shape) != tuple(k_pool.shape):
        raise _lib.ScaError(4, "pool geometry mismatch")
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.shape[0] < s:
        raise _lib.ScaError(4, "page_table must be int32 [num_seqs, max_blocks_per_seq]")
    max_blocks = page_table.shape[1]
    upper = nblk * bs
    if num_splits > 0:
        splits = min(num_splits, MAX_SPLITS)
    else:
        splits = paged_splits_for(typical_len if typical_len > 0 else min(upper, max_blocks * bs), s, hkv,
                                  hq // hkv, sm_count(q.device), longest_len)
    base = s * hq * splits
    ws = acquire_scratch_fp32(base * (2 + d), q.device)
    out = torch.empty((s, hq, 1, d), dtype=q.dtype, device=q.device)

    p = DecodeFwdParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr()
    p.partial_m = ws.data_ptr()
    p.partial_l = ws.data_ptr() + 4 * base
    p.partial_o = ws.data_ptr() + 8 * base
    p.batch, p.num_heads, p.num_kv_heads, p.seq_kv, p.head_dim, p.num_splits = s, hq, hkv, upper, d, splits
    p.q_stride = DecodeStrides(hq * d, d, d)
    p.o_stride = DecodeStrides(hq * d, d, d)
    p.k_stride = DecodeStrides(0, d, hkv * d)   # row = one token of the pool (reference: paged_backend.cpp:131-134)
    p.v_stride = p.k_stride
    p.scale = effective_scale(scale, d)
    p.dtype = dtype_id(q.dtype)
    p.seq_lens = seq_lens.data_ptr() if seq_lens is not None else None
    order_ptr = None
    if seq_order is not None:
        if seq_order.dtype != torch.int32 or seq_order.numel() != s or not seq_order.is_cuda:
            raise _lib.ScaError(4, "seq_order must be a device int32 permutation of the sequences")
        order_ptr = seq_order.data_ptr()
    pp = PagedDecodeParams()
    pp.base = p
    pp.page_table = page_table.data_ptr()
    pp.block_size, pp.max_blocks_per_seq, pp.num_kv_blocks = bs, max_blocks, nblk
    check(lib().sca_launch_paged_attention_ordered(C.byref(pp), order_ptr, _stream_ptr(stream)))
    if return_stats:
        return out, {"num_splits": splits, "workspace_bytes": base * (2 + d) * 4}
    return out


def decode_triples(q, k, v, *, scale=None, num_splits: int = 0, stream=None):
    """This rank's share of a sequence-split decode: merged but unnormalised {m, l, O[D]} per
    (batch, head), fp32 [B*H_q, 2 + D]."""
    _require_cuda(q, k, v)
    b, hq, sq, d = _dims(q, "bhsd")
    _, hkv, skv, _ = _dims(k, "bhsd")
    splits = min(num_splits, MAX_SPLITS) if num_splits > 0 else splits_for(skv, b, hkv, hq // hkv, sm_count(q.device))
    base = b * hq * splits
    ws = acquire_scratch_fp32(base * (2 + d), q.device)
    triples = torch.empty((b * hq, 2 + d), dtype=torch.float32, device=q.device)
    p = DecodeFwdParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), None
    p.partial_m = ws.data_ptr()
    p.partial_l = ws.data_ptr() + 4 * base
    p.partial_o = ws.data_ptr() + 8 * base
    p.batch, p.num_heads, p.num_kv_heads, p.seq_kv, p.head_dim, p.num_splits = b, hq, hkv, skv, d, splits
    p.q_stride = DecodeStrides(*_strides("bhsd", 1, hq, d))
    p.k_stride = DecodeStrides(*_strides("bhsd", skv, hkv, d))
    p.v_stride = p.k_stride
    p.o_stride = DecodeStrides(*_strides("bhsd", 1, hq, d))
    p.scale = effective_scale(scale, d)
    p.dtype = dtype_id(q.dtype)
    check(lib().sca_launch_decode_triples(C.byref(p), triples.data_ptr(), _stream_ptr(stream)))
    return triples


def decode_partials(q, k, v, *, scale=None, num_splits: int = 0, stream=None):
    """The split-K partial kernel alone. Returns (m [rows, splits], l [rows, splits], O [rows, splits, D],
    splits) as fp32 views of the scratch pool (valid until the next decode call on this device)."""
    _require_cuda(q, k, v)
    b, hq, sq, d = _dims(q, "bhsd")
    _, hkv, skv, _ = _dims(k, "bhsd")
    splits = min(num_splits, MAX_SPLITS) if num_splits > 0 else splits_for(skv, b, hkv, hq // hkv, sm_count(q.device))
    base = b * hq * splits
    ws = acquire_scratch_fp32(base * (2 + d), q.device)
    p = DecodeFwdParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), None
    p.partial_m = ws.data_ptr()
    p.partial_l = ws.data_ptr() + 4 * base
    p.partial_o = ws.data_ptr() + 8 * base
    p.batch, p.num_heads, p.num_kv_heads, p.seq_kv, p.head_dim, p.num_splits = b, hq, hkv, skv, d, splits
    p.q_stride = DecodeStrides(*_strides("bhsd", 1, hq, d))
    p.k_stride = DecodeStrides(*_strides("bhsd", skv, hkv, d))
    p.v_stride = p.k_stride
    p.o_stride = DecodeStrides(*_strides("bhsd", 1, hq, d))
    p.scale = effective_scale(scale, d)
    p.dtype = dtype_id(q.dtype)
    check(lib().sca_launch_decode_partials(C.byref(p), _stream_ptr(stream)))
    return ws[:base], ws[base: 2 * base], ws[2 * base: base * (2 + d)], splits


def merge_triples(gathered, out_dtype, *, stream=None):
    """gathered fp32 [ranks, rows, 2 + D] -> normalised output [rows, D] of `out_dtype`."""
    _require_cuda(gathered)
    ranks, rows, width = gathered.shape
    d = width - 2
    out = torch.empty((rows, d), dtype=out_dtype, device=gathered.device)
    check(lib().sca_launch_merge_triples(gathered.data_ptr(), ranks, rows, d, out.data_ptr(),
                                         dtype_id(out_dtype), _stream_ptr(stream)))
    return out


# ------------------------------------------------------------------------------------------------
# prefill
# ------------------------------------------------------------------------------------------------
def _fwd_params(q, k, v, out, lse, causal, scale, layout):
    b, hq, sq, d = _dims(q, layout)
    bk, hkv, skv, dk = _dims(k, layout)
    if (bk, dk) != (b, d) or tuple(v.shape) != tuple(k.shape) or q.dtype != k.dtype or q.dtype != v.dtype:
        raise _lib.ScaError(4, "q/k/v shape or dtype mismatch")
    if causal and skv < sq:
        raise _lib.ScaError(4, f"causal=true but seq_kv({skv}) < seq_q({sq})")
    p = FlashFwdParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.lse = lse.data_ptr() if lse is not None else None
    p.batch, p.num_heads, p.num_kv_heads, p.seq_q, p.seq_kv, p.head_dim = b, hq, hkv, sq, skv, d
    p.q_sb, p.q_sh, p.q_ss = _strides(layout, sq, hq, d)
    p.k_sb, p.k_sh, p.k_ss = _strides(layout, skv, hkv, d)
    p.v_sb, p.v_sh, p.v_ss = p.k_sb, p.k_sh, p.k_ss
    p.o_sb, p.o_sh, p.o_ss = _strides("bhsd", sq, hq, d)
    p.scale = effective_scale(scale, d)
    p.causal = int(bool(causal))
    p.return_lse = int(lse is not None)
    p.diagonal = (skv - sq) if causal else 0
    p.dtype_id = dtype_id(q.dtype)
    return p


def _alloc_out(q, layout, return_lse):
    b, hq, sq, d = _dims(q, layout)
    out = torch.empty((b, hq, sq, d), dtype=q.dtype, device=q.device)
    lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device) if return_lse else None
    return out, lse


def flash_status(device=None) -> int:
    """0 when every flash launch on `device` so far ran to completion, otherwise 1 + the warp whose bounded wait ran
    out (that launch's output is invalid). Synchronise the stream first; reading clears the record."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    code = C.c_int32(0)
    check(lib().sca_flash_status(int(index or 0), C.byref(code)))
    return int(code.value)


def flash_attention(q, k, v, *, causal=False, scale=None, return_lse=False, layout="bhsd", stream=None,
                    out=None, lse=None):
    """tcgen05 flash prefill (sca::flash_attention); fp16 / bf16 only."""
    _require_cuda(q, k, v)
    if q.dtype == torch.float32:
        raise _lib.ScaError(4, "flash backend computes in fp16/bf16; dtype=float32 is served by the naive "
                               "(reference) or tiled backend")
    if out is None:
        out, lse = _alloc_out(q, layout, return_lse)
    p = _fwd_params(q, k, v, out, lse, causal, scale, layout)
    check(lib().sca_launch_flash_fwd(C.byref(p), _stream_ptr(stream)))
    return (out, lse) if return_lse else out


def flash_attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_kv, *, causal=False, scale=None, stream=None):
    """Packed variable-length prefill in one launch. q [T_q, H_q, D], k / v [T_kv, H_kv, D] on the device;
    cu_seqlens_* are HOST int32 offsets (num_seqs + 1 entries, as in the reference API). Returns [T_q, H_q, D]."""
    import numpy as np
    _require_cuda(q, k, v)
    if q.dim() != 3 or k.dim() != 3 or tuple(k.shape) != tuple(v.shape) or not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise _lib.ScaError(4, "varlen expects contiguous packed [T, H, D] tensors")
    cu_q = np.ascontiguousarray(cu_seqlens_q, dtype=np.int32)
    cu_kv = np.ascontiguousarray(cu_seqlens_kv, dtype=np.int32)
    if cu_q.ndim != 1 or cu_q.shape != cu_kv.shape or cu_q.shape[0] < 2:
        raise _lib.ScaError(4, "cu_seqlens_q / cu_seqlens_kv must be host int32 arrays of num_seqs + 1 entries")
    tq, hq, d = q.shape
    tkv, hkv, _ = k.shape
    n = cu_q.shape[0] - 1
    out = torch.empty_like(q)
    ws_bytes = lib().sca_flash_varlen_workspace_bytes(n, tq)
    ws = torch.empty(max(int(ws_bytes), 16), dtype=torch.uint8, device=q.device)
    p = _lib.FlashVarlenParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.total_q, p.total_kv, p.num_heads, p.num_kv_heads, p.head_dim, p.num_seqs = tq, tkv, hq, hkv, d, n
    p.cu_seqlens_q, p.cu_seqlens_kv = cu_q.ctypes.data, cu_kv.ctypes.data
    p.scale = effective_scale(scale, d)
    p.causal = 1 if causal else 0
    p.dtype_id = dtype_id(q.dtype)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    check(lib().sca_launch_flash_varlen(C.byref(p), _stream_ptr(stream)))
    if stream is None:
        ws.record_stream(torch.cuda.current_stream(q.device))
    return out


def flash_attention_paged(q, k_pool, v_pool, page_table, cu_seqlens_q, seq_lens_kv, *, causal=True, scale=None, stream=None):
    """Chunked prefill over a paged KV cache in one launch: q packed [T_q, H_q, D] (the new tokens of every
    sequence), pools [num_blocks, block_size, H_kv, D], page_table int32 [num_seqs, max_blocks_per_seq] on the device,
    cu_seqlens_q (num_seqs + 1) and seq_lens_kv (num_seqs: tokens of each sequence in the cache, the new ones
    included) on the HOST. Returns [T_q, H_q, D]."""
    import numpy as np
    _require_cuda(q, k_pool, v_pool, page_table)
    if q.dim() != 3 or k_pool.dim() != 4 or tuple(k_pool.shape) != tuple(v_pool.shape) or not (
            q.is_contiguous() and k_pool.is_contiguous() and v_pool.is_contiguous() and page_table.is_contiguous()):
        raise _lib.ScaError(4, "paged prefill expects packed q [T, H, D] and contiguous pools [blocks, block_size, H_kv, D]")
    if page_table.dtype != torch.int32 or page_table.dim() != 2:
        raise _lib.ScaError(4, "page_table must be int32 [num_seqs, max_blocks_per_seq]")
    cu_q = np.ascontiguousarray(cu_seqlens_q, dtype=np.int32)
    lens = np.ascontiguousarray(seq_lens_kv, dtype=np.int32)
    n = lens.shape[0]
    if cu_q.ndim != 1 or cu_q.shape[0] != n + 1 or page_table.shape[0] < n:
        raise _lib.ScaError(4, "cu_seqlens_q needs num_seqs + 1 entries, seq_lens_kv and the page table num_seqs")
    tq, hq, d = q.shape
    nblk, bs, hkv, dk = k_pool.shape
    if dk != d:
        raise _lib.ScaError(4, "pool head_dim differs from q")
    out = torch.empty_like(q)
    ws_bytes = lib().sca_flash_varlen_workspace_bytes(n, tq)
    ws = torch.empty(max(int(ws_bytes), 16), dtype=torch.uint8, device=q.device)
    p = _lib.FlashPagedParams()
    p.q, p.out, p.k_pool, p.v_pool, p.page_table = q.data_ptr(), out.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr()
    p.total_q, p.num_heads, p.num_kv_heads, p.head_dim, p.num_seqs = tq, hq, hkv, d, n
    p.num_blocks, p.block_size, p.max_blocks_per_seq = nblk, bs, page_table.shape[1]
    p.cu_seqlens_q, p.seq_lens_kv = cu_q.ctypes.data, lens.ctypes.data
    p.scale = effective_scale(scale, d)
    p.causal = 1 if causal else 0
    p.dtype_id = dtype_id(q.dtype)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    check(lib().sca_launch_flash_paged(C.byref(p), _stream_ptr(stream)))
    if stream is None:
        ws.record_stream(torch.cuda.current_stream(q.device))
    return out


def simt_attention(q, k, v, *, causal=False, scale=None, return_lse=False, layout="bhsd", stream=None):
    """Functional SIMT attention behind the naive / tiled backends (any compute dtype)."""
    _require_cuda(q, k, v)
    out, lse = _alloc_out(q, layout, return_lse)
    p = _fwd_params(q, k, v, out, lse, causal, scale, layout)
    check(lib().sca_launch_simt_forward(C.byref(p), _stream_ptr(stream)))
    return (out, lse) if return_lse else out


def naive_attention(q, k, v, *, causal=False, scale=None, return_lse=False, layout="bhsd", stream=None):
    """Level-1 attention with the fp32 score matrix materialised in scratch (sca::naive_attention)."""
    _require_cuda(q, k, v)
    out, lse = _alloc_out(q, layout, return_lse)
    p = _fwd_params(q, k, v, out, lse, causal, scale, layout)
    need = lib().sca_naive_score_bytes(p.batch, p.num_heads, p.seq_q, p.seq_kv)
    if need <= 0:
        raise _lib.ScaError(4, "naive attention: invalid geometry")
    scores = acquire_scratch_fp32(need // 4, q.device)
    check(lib().sca_launch_naive_forward(C.byref(p), scores.data_ptr(), _stream_ptr(stream)))
    return (out, lse) if return_lse else out


# ------------------------------------------------------------------------------------------------
# KV cache data movement (pools are [num_blocks, block_size, H_kv, D])
# ------------------------------------------------------------------------------------------------
def _kv_shape(pool: torch.Tensor) -> KvCacheShape:
    nblk, bs, hkv, d = pool.shape
    return KvCacheShape(nblk, bs, hkv, d)


def kv_append(layer_k, layer_v, k_new, v_new, slot_mapping, *, stream=None) -> None:
    """k_new/v_new [num_tokens, H_kv, D]; slot_mapping int32 [num_tokens] on the device."""
    _require_cuda(layer_k, layer_v, k_new, v_new, slot_mapping)
    shape = _kv_shape(layer_k)
    check(lib().sca_launch_kv_append(layer_k.data_ptr(), layer_v.data_ptr(), k_new.data_ptr(),
                                     v_new.data_ptr(), slot_mapping.data_ptr(), k_new.shape[0],
                                     C.byref(shape), layer_k.element_size(), _stream_ptr(stream)))


def kv_append_batched(layer_k, layer_v, k_new, v_new, page_table, seq_lens, *, stream=None) -> None:
    """One new token per sequence; the slot comes from the page table at position seq_lens[s] - 1."""
    _require_cuda(layer_k, layer_v, k_new, v_new, page_table, seq_lens)
    shape = _kv_shape(layer_k)
    check(lib().sca_launch_kv_append_batched(layer_k.data_ptr(), layer_v.data_ptr(), k_new.data_ptr(),
                                             v_new.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(),
                                             k_new.shape[0], page_table.shape[1], C.byref(shape),
                                             layer_k.element_size(), _stream_ptr(stream)))


def kv_reset(layer_k, layer_v, block_ids, *, stream=None) -> None:
    _require_cuda(layer_k, layer_v, block_ids)
    shape = _kv_shape(layer_k)
    check(lib().sca_launch_kv_reset_block(layer_k.data_ptr(), layer_v.data_ptr(), block_ids.data_ptr(),
                                          block_ids.numel(), C.byref(shape), layer_k.element_size(),
                                          _stream_ptr(stream)))


def kv_gather(layer, block_ids, *, stream=None) -> torch.Tensor:
    _require_cuda(layer, block_ids)
    shape = _kv_shape(layer)
    out = torch.empty((block_ids.numel(),) + tuple(layer.shape[1:]), dtype=layer.dtype, device=layer.device)
    check(lib().sca_launch_kv_gather(layer.data_ptr(), block_ids.data_ptr(), block_ids.numel(),
                                     out.data_ptr(), C.byref(shape), layer.element_size(),
                                     _stream_ptr(stream)))
    return out
