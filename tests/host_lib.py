"""ctypes view of libsci_attention.so's flat C facade (csrc/host/c_facade.cpp)."""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST_SO = os.path.join(ROOT, "scicompute_attention_b200", "libsci_attention.so")

_i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_lib = None


def lib():
    global _lib
    if _lib is None:
        l = C.CDLL(HOST_SO)
        for name in ("sca_c_validate", "sca_c_explain"):
            getattr(l, name).argtypes = [_i64p, _f32p, _i64p, C.c_char_p, C.c_int]
        l.sca_c_select.argtypes = [_i64p, _f32p, _i64p, C.c_char_p, C.c_int, C.c_void_p, C.c_void_p]
        l.sca_c_effective_scale.argtypes = [_i64p, _f32p, _i64p]
        l.sca_c_effective_scale.restype = C.c_float
        l.sca_c_status_info.argtypes = [C.c_int, C.POINTER(C.c_int), C.c_char_p, C.c_int]
        l.sca_c_varlen_validate.argtypes = [_i32p, C.c_int64, C.POINTER(C.c_int64), C.c_char_p, C.c_int]
        l.sca_c_dispatch_revision.restype = C.c_char_p
        l.sca_c_decode_splits_for.argtypes = [C.c_int64] * 5
        l.sca_c_decode_splits_for.restype = C.c_int64
        l.sca_c_paged_splits_for.argtypes = [C.c_int64] * 5
        l.sca_c_paged_splits_for.restype = C.c_int64
        l.sca_c_bm_create.argtypes = [C.c_int64] * 3 + [C.c_int, C.c_char_p, C.c_int]
        l.sca_c_bm_create.restype = C.c_void_p
        l.sca_c_bm_destroy.argtypes = [C.c_void_p]
        l.sca_c_bm_allocate.argtypes = [C.c_void_p, C.c_int64, _i32p, C.c_char_p, C.c_int]
        l.sca_c_bm_free.argtypes = [C.c_void_p, _i32p, C.c_int64]
        l.sca_c_bm_free.restype = None
        l.sca_c_bm_append_to_table.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_char_p, C.c_int]
        l.sca_c_bm_reset_seq.argtypes = [C.c_void_p, C.c_int64]
        for name in ("sca_c_bm_num_free", "sca_c_bm_allocation_failures", "sca_c_bm_double_free_events"):
            getattr(l, name).argtypes = [C.c_void_p]
            getattr(l, name).restype = C.c_int64
        l.sca_c_bm_revision.argtypes = [C.c_void_p]
        l.sca_c_bm_revision.restype = C.c_uint64
        l.sca_c_bm_table.argtypes = [C.c_void_p]
        l.sca_c_bm_table.restype = C.POINTER(C.c_int32)
        l.sca_c_slot_mapping.argtypes = [C.c_void_p] + [C.c_int64] * 4 + [_i32p, C.c_char_p, C.c_int]
        l.sca_c_kv_cache_bytes.argtypes = [C.c_int64] * 5 + [C.c_int, C.c_char_p, C.c_int]
        l.sca_c_kv_cache_bytes.restype = C.c_int64
        l.sca_c_max_blocks_for_budget.argtypes = [C.c_int64] * 4 + [C.c_int, C.c_uint64]
        l.sca_c_max_blocks_for_budget.restype = C.c_int64
        l.sca_c_paged_create.argtypes = [C.c_int64] * 5 + [C.c_int, C.c_int64, C.c_int, C.c_char_p, C.c_int]
        l.sca_c_paged_create.restype = C.c_void_p
        l.sca_c_paged_destroy.argtypes = [C.c_void_p]
        l.sca_c_paged_append.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_char_p, C.c_int]
        l.sca_c_paged_append_batch.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_char_p, C.c_int]
        l.sca_c_paged_reset_seq.argtypes = [C.c_void_p, C.c_int64]
        for name in ("sca_c_paged_seq_length", "sca_c_paged_logical_blocks"):
            getattr(l, name).argtypes = [C.c_void_p, C.c_int64]
            getattr(l, name).restype = C.c_int64
        l.sca_c_paged_max_blocks_per_seq.argtypes = [C.c_void_p]
        l.sca_c_paged_max_blocks_per_seq.restype = C.c_int64
        l.sca_c_paged_read_table.argtypes = [C.c_void_p, _i32p, C.c_void_p]
        l.sca_c_paged_read_layer.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
        l.sca_c_paged_read_layer.restype = None
        l.sca_c_paged_stats.argtypes = [C.c_void_p, C.POINTER(C.c_int64)]
        l.sca_c_paged_attention.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                            C.POINTER(C.c_int64), C.c_char_p, C.c_int]
        _lib = l
    return _lib


def records(cfg_i, cfg_f, shape):
    return (np.array(cfg_i, np.int64), np.array(cfg_f, np.float32), np.array(shape, np.int64))
