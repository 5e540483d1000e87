"""ctypes view of the C ABI declared in include/sca_b200.h (libsca_b200.so).

There is no fallback of any kind: if the library has not been built, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB = os.path.join(PKG, "libsca_b200.so")

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
SCA_OK = 0
STATUS_NAMES = {0: "OK", 4: "InvalidArgument", 5: "NotImplemented", 100: "CudaError",
                101: "CudaNotAvailable", 102: "CudaOutOfMemory", 500: "Timeout"}
MGPU_ID_BYTES = 128

# every symbol include/sca_b200.h declares (tests check that the library exports all of them)
EXPORTED_SYMBOLS = [
    "sca_last_error", "sca_probe_device", "sca_probe_device_b200", "sca_mem_get_info", "sca_launch_flash_fwd", "sca_flash_status",
    "sca_flash_smem_bytes_for", "sca_launch_decode_splitk", "sca_launch_decode_splitk_paged",
    "sca_launch_paged_attention", "sca_launch_paged_attention_ordered", "sca_launch_decode_splitk_static", "sca_launch_decode_triples", "sca_launch_merge_triples",
    "sca_launch_simt_forward", "sca_naive_score_bytes", "sca_launch_naive_forward", "sca_launch_kv_append", "sca_launch_kv_reset_block",
    "sca_launch_kv_gather", "sca_launch_kv_append_batched", "sca_launch_decode_partials",
    "sca_peer_buffer_bytes", "sca_peer_buffer_create", "sca_peer_buffer_open", "sca_peer_buffer_close",
    "sca_peer_buffer_destroy", "sca_peer_exchange_status", "sca_peer_exchange_clear", "sca_launch_seqsplit_exchange",
    "sca_flash_varlen_workspace_bytes", "sca_launch_flash_varlen", "sca_launch_flash_paged",
    "sca_mgpu_unique_id", "sca_mgpu_init", "sca_mgpu_allgather_triples", "sca_mgpu_abort", "sca_mgpu_destroy",
]

PEER_MAX_RANKS = 16
PEER_HANDLE_BYTES = 64


class ScaError(RuntimeError):
    """A C-ABI call returned a non-zero status; `.code` is the sci::StatusCode value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


class DeviceProbe(C.Structure):
    _fields_ = [("name", C.c_char * 256), ("major", C.c_int), ("minor", C.c_int), ("sm_count", C.c_int),
                ("smem_per_sm", C.c_ulonglong), ("smem_per_block_default", C.c_ulonglong),
                ("smem_per_block_optin", C.c_ulonglong), ("regs_per_sm", C.c_ulonglong),
                ("max_threads_per_sm", C.c_ulonglong), ("l2_bytes", C.c_ulonglong),
                ("total_mem_bytes", C.c_ulonglong), ("free_mem_bytes", C.c_ulonglong),
                ("cuda_available", C.c_int), ("binary_has_sm80", C.c_int), ("binary_has_sm90", C.c_int)]


class DeviceProbeB200(C.Structure):
    _fields_ = [("base", DeviceProbe), ("binary_has_sm100a", C.c_int), ("tmem_columns", C.c_int),
                ("max_cluster_size", C.c_int)]


class FlashFwdParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
                ("lse", C.c_void_p)] + [(n, C.c_int64) for n in (
                    "batch", "num_heads", "num_kv_heads", "seq_q", "seq_kv", "head_dim",
                    "q_sb", "q_sh", "q_ss", "k_sb", "k_sh", "k_ss", "v_sb", "v_sh", "v_ss",
                    "o_sb", "o_sh", "o_ss")] + [
                    ("scale", C.c_float), ("causal", C.c_int32), ("return_lse", C.c_int32),
                    ("diagonal", C.c_int64), ("dtype_id", C.c_int32)]


class DecodeStrides(C.Structure):
    _fields_ = [("s_b", C.c_int64), ("s_h", C.c_int64), ("s_s", C.c_int64)]


class DecodeFwdParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
                ("partial_m", C.c_void_p), ("partial_l", C.c_void_p), ("partial_o", C.c_void_p),
                ("batch", C.c_int64), ("num_heads", C.c_int64), ("num_kv_heads", C.c_int64),
                ("seq_kv", C.c_int64), ("head_dim", C.c_int64), ("num_splits", C.c_int64),
                ("q_stride", DecodeStrides), ("k_stride", DecodeStrides), ("v_stride", DecodeStrides),
                ("o_stride", DecodeStrides), ("scale", C.c_float), ("dtype", C.c_int32),
                ("page_table", C.c_void_p), ("block_size", C.c_int64),
                ("max_blocks_per_seq", C.c_int64), ("num_kv_blocks", C.c_int64),
                ("seq_lens", C.c_void_p)]


class PagedDecodeParams(C.Structure):
    _fields_ = [("base", DecodeFwdParams), ("page_table", C.c_void_p), ("block_size", C.c_int64),
                ("max_blocks_per_seq", C.c_int64), ("num_kv_blocks", C.c_int64)]


class KvCacheShape(C.Structure):
    _fields_ = [("num_blocks", C.c_int64), ("block_size", C.c_int64), ("num_kv_heads", C.c_int64),
                ("head_dim", C.c_int64)]


class FlashVarlenParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p)] + [
        (n, C.c_int64) for n in ("total_q", "total_kv", "num_heads", "num_kv_heads", "head_dim", "num_seqs")] + [
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_kv", C.c_void_p), ("scale", C.c_float), ("causal", C.c_int32),
        ("dtype_id", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64)]


class FlashPagedParams(C.Structure):
    _fields_ = [("q", C.c_void_p), ("out", C.c_void_p), ("k_pool", C.c_void_p), ("v_pool", C.c_void_p),
                ("page_table", C.c_void_p)] + [
        (n, C.c_int64) for n in ("total_q", "num_heads", "num_kv_heads", "head_dim", "num_seqs", "num_blocks", "block_size",
                                 "max_blocks_per_seq")] + [
        ("cu_seqlens_q", C.c_void_p), ("seq_lens_kv", C.c_void_p), ("scale", C.c_float), ("causal", C.c_int32),
        ("dtype_id", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64)]


class SeqSplitExchange(C.Structure):
    _fields_ = [("peer_buffers", C.c_void_p * PEER_MAX_RANKS), ("rank", C.c_int32), ("world", C.c_int32),
                ("rows", C.c_int64), ("head_dim", C.c_int64), ("num_splits", C.c_int64), ("epoch", C.c_uint32),
                ("partial_m", C.c_void_p), ("partial_l", C.c_void_p), ("partial_o", C.c_void_p),
                ("out", C.c_void_p), ("out_dtype", C.c_int32)]


_lib = None


def lib() -> C.CDLL:
    """Loads libsca_b200.so (raises when it is missing: build it with
    `python -m scicompute_attention_b200.build`)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(KERNEL_LIB):
        raise RuntimeError(
            f"{KERNEL_LIB} is missing: the CUDA extension has not been built "
            "(python -m scicompute_attention_b200.build). There is no CPU fallback.")
    l = C.CDLL(KERNEL_LIB)
    l.sca_last_error.restype = C.c_char_p
    l.sca_probe_device.argtypes = [C.c_int, C.POINTER(DeviceProbe)]
    l.sca_probe_device_b200.argtypes = [C.c_int, C.POINTER(DeviceProbeB200)]
    l.sca_mem_get_info.argtypes = [C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)]
    if hasattr(l, "sca_launch_flash_fwd"):
        l.sca_launch_flash_fwd.argtypes = [C.POINTER(FlashFwdParams), C.c_void_p]
        l.sca_flash_status.argtypes = [C.c_int, C.POINTER(C.c_int32)]
        l.sca_flash_smem_bytes_for.argtypes = [C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_int]
        l.sca_flash_smem_bytes_for.restype = C.c_longlong
    l.sca_launch_simt_forward.argtypes = [C.POINTER(FlashFwdParams), C.c_void_p]
    l.sca_launch_naive_forward.argtypes = [C.POINTER(FlashFwdParams), C.c_void_p, C.c_void_p]
    l.sca_naive_score_bytes.argtypes = [C.c_int64] * 4
    l.sca_naive_score_bytes.restype = C.c_longlong
    l.sca_launch_decode_splitk.argtypes = [C.POINTER(DecodeFwdParams), C.c_void_p]
    l.sca_launch_decode_splitk_paged.argtypes = [C.POINTER(DecodeFwdParams), C.c_void_p]
    l.sca_launch_paged_attention.argtypes = [C.POINTER(PagedDecodeParams), C.c_void_p]
    l.sca_launch_paged_attention_ordered.argtypes = [C.POINTER(PagedDecodeParams), C.c_void_p, C.c_void_p]
    l.sca_launch_decode_splitk_static.argtypes = [C.POINTER(DecodeFwdParams), C.c_void_p]
    l.sca_launch_decode_triples.argtypes = [C.POINTER(DecodeFwdParams), C.c_void_p, C.c_void_p]
    l.sca_launch_merge_triples.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                           C.c_int32, C.c_void_p]
    l.sca_launch_kv_append.argtypes = [C.c_void_p] * 5 + [C.c_int64, C.POINTER(KvCacheShape), C.c_int64, C.c_void_p]
    l.sca_launch_kv_append_batched.argtypes = [C.c_void_p] * 6 + [C.c_int64, C.c_int64,
                                                                   C.POINTER(KvCacheShape), C.c_int64, C.c_void_p]
    l.sca_launch_kv_reset_block.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                            C.POINTER(KvCacheShape), C.c_int64, C.c_void_p]
    l.sca_launch_kv_gather.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                       C.POINTER(KvCacheShape), C.c_int64, C.c_void_p]
    l.sca_flash_varlen_workspace_bytes.argtypes = [C.c_int64, C.c_int64]
    l.sca_flash_varlen_workspace_bytes.restype = C.c_longlong
    l.sca_launch_flash_varlen.argtypes = [C.POINTER(FlashVarlenParams), C.c_void_p]
    l.sca_launch_flash_paged.argtypes = [C.POINTER(FlashPagedParams), C.c_void_p]
    l.sca_mgpu_unique_id.argtypes = [C.c_char_p]
    l.sca_mgpu_init.argtypes = [C.c_char_p, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]
    l.sca_mgpu_allgather_triples.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32]
    l.sca_mgpu_abort.argtypes = [C.c_void_p]
    l.sca_mgpu_destroy.argtypes = [C.c_void_p]
    l.sca_launch_decode_partials.argtypes = [C.POINTER(DecodeFwdParams), C.c_void_p]
    l.sca_peer_buffer_bytes.argtypes = [C.c_int32, C.c_int64, C.c_int64]
    l.sca_peer_buffer_bytes.restype = C.c_longlong
    l.sca_peer_buffer_create.argtypes = [C.c_int64, C.POINTER(C.c_void_p), C.c_char_p]
    l.sca_peer_buffer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    l.sca_peer_buffer_close.argtypes = [C.c_void_p]
    l.sca_peer_buffer_destroy.argtypes = [C.c_void_p]
    l.sca_peer_exchange_status.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    l.sca_peer_exchange_clear.argtypes = [C.c_void_p]
    l.sca_launch_seqsplit_exchange.argtypes = [C.POINTER(SeqSplitExchange), C.c_void_p]
    _lib = l
    return l


def check(rc: int) -> None:
    if rc != SCA_OK:
        raise ScaError(rc, lib().sca_last_error().decode("utf-8", "replace"))
