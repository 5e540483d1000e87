"""ctypes bindings for the CPU oracle (oracle/liboracle.so) and, when it has been built, for the
reference's own host code (oracle/_ref/libsca_ref.so).

Test infrastructure only: the test suite, the smoke check and the benchmark's CPU-baseline leg use it;
nothing under the product package imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ORACLE_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(ORACLE_DIR)
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libsca_ref.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")

DT_F32, DT_F16, DT_BF16 = 0, 1, 2  # same ids as sci::DType and the C ABI

_oracle = None
_ref = None


def build_oracle() -> None:
    subprocess.run(["make", "-C", ORACLE_DIR, "-s"], check=True)


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            build_oracle()
        lib = C.CDLL(ORACLE_SO)
        lib.oracle_random_floats.argtypes = [_f32p, C.c_size_t, C.c_uint32, C.c_float, C.c_float]
        lib.oracle_random_floats.restype = None
        lib.oracle_encode.argtypes = [_f32p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p]
        lib.oracle_encode.restype = None
        lib.oracle_attention_f64.argtypes = [_f32p, _f32p, _f32p] + [C.c_int64] * 6 + [
            C.c_int, C.c_double, _f64p, C.c_void_p, C.c_int]
        lib.oracle_attention_f64.restype = C.c_int
        lib.oracle_paged_decode_f64.argtypes = [_f32p, _f32p, _f32p, _i32p, C.c_void_p] + [
            C.c_int64] * 7 + [C.c_double, _f64p, C.c_int]
        lib.oracle_paged_decode_f64.restype = C.c_int
        lib.oracle_merge_parts_f64.argtypes = [_f64p, _f64p, _f64p, C.c_int64, C.c_int64, _f64p]
        lib.oracle_merge_parts_f64.restype = None
        lib.oracle_max_threads.restype = C.c_int
        for name in ("oracle_float_to_half_bits", "oracle_float_to_bf16_bits"):
            getattr(lib, name).argtypes = [C.c_float]
            getattr(lib, name).restype = C.c_uint16
        for name in ("oracle_half_bits_to_float", "oracle_bf16_bits_to_float"):
            getattr(lib, name).argtypes = [C.c_uint16]
            getattr(lib, name).restype = C.c_float
        # KV bookkeeping
        lib.oracle_bm_create.argtypes = [C.c_int64] * 3
        lib.oracle_bm_create.restype = C.c_void_p
        lib.oracle_bm_destroy.argtypes = [C.c_void_p]
        lib.oracle_bm_allocate.argtypes = [C.c_void_p, C.c_int64, _i32p]
        lib.oracle_bm_allocate.restype = C.c_int
        lib.oracle_bm_free.argtypes = [C.c_void_p, _i32p, C.c_int64]
        lib.oracle_bm_free.restype = None
        lib.oracle_bm_append_to_table.argtypes = [C.c_void_p, C.c_int64, _i32p, C.c_int64]
        lib.oracle_bm_append_to_table.restype = C.c_int
        lib.oracle_bm_reset_seq.argtypes = [C.c_void_p, C.c_int64]
        lib.oracle_bm_reset_seq.restype = C.c_int
        for name in ("oracle_bm_num_free", "oracle_bm_allocation_failures",
                     "oracle_bm_double_free_events"):
            getattr(lib, name).argtypes = [C.c_void_p]
            getattr(lib, name).restype = C.c_int64
        lib.oracle_bm_revision.argtypes = [C.c_void_p]
        lib.oracle_bm_revision.restype = C.c_uint64
        lib.oracle_bm_table.argtypes = [C.c_void_p]
        lib.oracle_bm_table.restype = C.POINTER(C.c_int32)
        lib.oracle_bm_free_list.argtypes = [C.c_void_p]
        lib.oracle_bm_free_list.restype = C.POINTER(C.c_int32)
        lib.oracle_slot_mapping.argtypes = [_i32p] + [C.c_int64] * 4 + [_i32p, C.POINTER(C.c_int64)]
        lib.oracle_slot_mapping.restype = C.c_int
        lib.oracle_kv_cache_bytes.argtypes = [C.c_int64] * 6
        lib.oracle_kv_cache_bytes.restype = C.c_int64
        lib.oracle_max_blocks_for_budget.argtypes = [C.c_int64] * 5 + [C.c_uint64]
        lib.oracle_max_blocks_for_budget.restype = C.c_int64
        lib.oracle_kv_append.argtypes = [_u8p, _u8p, _u8p, _u8p, _i32p] + [C.c_int64] * 6
        lib.oracle_kv_append.restype = None
        lib.oracle_kv_reset.argtypes = [_u8p, _u8p, _i32p] + [C.c_int64] * 6
        lib.oracle_kv_reset.restype = None
        lib.oracle_kv_gather.argtypes = [_u8p, _i32p, C.c_int64, _u8p] + [C.c_int64] * 5
        lib.oracle_kv_gather.restype = None
        _oracle = lib
    return _oracle


def have_ref() -> bool:
    return os.path.exists(REF_SO)


def ref() -> C.CDLL:
    """The reference's own host code; only available where oracle/build_ref.sh has run."""
    global _ref
    if _ref is None:
        lib = C.CDLL(REF_SO)
        lib.ref_random_floats.argtypes = [_f32p, C.c_uint64, C.c_uint32, C.c_float, C.c_float]
        lib.ref_random_floats.restype = None
        lib.ref_float_to_half_bits.argtypes = [C.c_float]
        lib.ref_float_to_half_bits.restype = C.c_uint16
        lib.ref_float_to_bf16_bits.argtypes = [C.c_float]
        lib.ref_float_to_bf16_bits.restype = C.c_uint16
        lib.ref_half_bits_to_float.argtypes = [C.c_uint16]
        lib.ref_half_bits_to_float.restype = C.c_float
        lib.ref_bf16_bits_to_float.argtypes = [C.c_uint16]
        lib.ref_bf16_bits_to_float.restype = C.c_float
        lib.ref_attention.argtypes = [_f32p, _f32p, _f32p] + [C.c_int64] * 6 + [C.c_int, _f64p]
        lib.ref_attention.restype = None
        lib.ref_tolerance.argtypes = [C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        lib.ref_bm_create.argtypes = [C.c_int64] * 3 + [C.c_char_p, C.c_int]
        lib.ref_bm_create.restype = C.c_void_p
        lib.ref_bm_destroy.argtypes = [C.c_void_p]
        lib.ref_bm_allocate.argtypes = [C.c_void_p, C.c_int64, _i32p, C.c_char_p, C.c_int]
        lib.ref_bm_free.argtypes = [C.c_void_p, _i32p, C.c_int64]
        lib.ref_bm_free.restype = None
        lib.ref_bm_append_to_table.argtypes = [C.c_void_p, C.c_int64, _i32p, C.c_int64, C.c_char_p, C.c_int]
        lib.ref_bm_reset_seq.argtypes = [C.c_void_p, C.c_int64]
        for name in ("ref_bm_num_free", "ref_bm_allocation_failures", "ref_bm_double_free_events"):
            getattr(lib, name).argtypes = [C.c_void_p]
            getattr(lib, name).restype = C.c_int64
        lib.ref_bm_revision.argtypes = [C.c_void_p]
        lib.ref_bm_revision.restype = C.c_uint64
        lib.ref_bm_table.argtypes = [C.c_void_p]
        lib.ref_bm_table.restype = C.POINTER(C.c_int32)
        lib.ref_slot_mapping.argtypes = [_i32p] + [C.c_int64] * 4 + [_i32p, C.c_char_p, C.c_int]
        lib.ref_kv_cache_bytes.argtypes = [C.c_int64] * 5 + [C.c_int, C.c_char_p, C.c_int]
        lib.ref_kv_cache_bytes.restype = C.c_int64
        lib.ref_max_blocks_for_budget.argtypes = [C.c_int64] * 4 + [C.c_int, C.c_uint64]
        lib.ref_max_blocks_for_budget.restype = C.c_int64
        lib.ref_paged_create.argtypes = [C.c_int64] * 5 + [C.c_int, C.c_int64, C.c_char_p, C.c_int]
        lib.ref_paged_create.restype = C.c_void_p
        lib.ref_paged_destroy.argtypes = [C.c_void_p]
        lib.ref_paged_append.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                         C.c_int64, C.c_char_p, C.c_int]
        lib.ref_paged_reset_seq.argtypes = [C.c_void_p, C.c_int64]
        for name in ("ref_paged_seq_length", "ref_paged_logical_blocks"):
            getattr(lib, name).argtypes = [C.c_void_p, C.c_int64]
            getattr(lib, name).restype = C.c_int64
        lib.ref_paged_max_blocks_per_seq.argtypes = [C.c_void_p]
        lib.ref_paged_max_blocks_per_seq.restype = C.c_int64
        lib.ref_paged_synced_table.argtypes = [C.c_void_p]
        lib.ref_paged_synced_table.restype = C.POINTER(C.c_int32)
        lib.ref_paged_layer.argtypes = [C.c_void_p, C.c_int64, C.c_int]
        lib.ref_paged_layer.restype = C.c_void_p
        lib.ref_paged_stats.argtypes = [C.c_void_p, C.POINTER(C.c_int64)]
        _i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
        for name in ("ref_validate", "ref_select", "ref_explain"):
            getattr(lib, name).argtypes = [_i64p, _f32p, _i64p, C.c_char_p, C.c_int]
        lib.ref_effective_scale.argtypes = [_i64p, _f32p, _i64p]
        lib.ref_effective_scale.restype = C.c_float
        lib.ref_status_info.argtypes = [C.c_int, C.POINTER(C.c_int), C.c_char_p, C.c_int]
        lib.ref_varlen_validate.argtypes = [_i32p, C.c_int64, C.POINTER(C.c_int64), C.c_char_p, C.c_int]
        _ref = lib
    return _ref


# ---------------------------------------------------------------------------------------------
# convenience wrappers
# ---------------------------------------------------------------------------------------------
def random_floats(count: int, seed: int, low: float = -1.0, high: float = 1.0) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    oracle().oracle_random_floats(out, count, seed, low, high)
    return out


def encode(values: np.ndarray, dtype: int):
    """Returns (storage bits as uint16 or the float32 array itself, dequantised float32)."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    if dtype == DT_F32:
        return values.copy(), values.copy()
    bits = np.empty(values.shape, dtype=np.uint16)
    deq = np.empty(values.shape, dtype=np.float32)
    oracle().oracle_encode(values.reshape(-1), values.size, dtype, bits.ctypes.data, deq.ctypes.data)
    return bits, deq


def decode_bits(bits: np.ndarray, dtype: int) -> np.ndarray:
    """uint16 storage -> float32 (exact)."""
    if dtype == DT_F32:
        return np.asarray(bits, dtype=np.float32)
    b = np.asarray(bits).astype(np.uint32)
    if dtype == DT_BF16:
        return (b << 16).view(np.float32)
    return np.asarray(bits).view(np.float16).astype(np.float32)


def attention_f64(q, k, v, causal=False, scale=0.0, want_lse=False, threads=0):
    """q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] float32 (already dequantised) -> float64 out (, lse)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    out = np.zeros((B, Hq, Sq, D), dtype=np.float64)
    lse = np.zeros((B, Hq, Sq), dtype=np.float64) if want_lse else None
    if threads <= 0:
        threads = oracle().oracle_max_threads()
    rc = oracle().oracle_attention_f64(q.reshape(-1), k.reshape(-1), v.reshape(-1), B, Hq, Hkv, Sq,
                                       Skv, D, int(causal), float(scale), out.reshape(-1),
                                       lse.ctypes.data if want_lse else None, threads)
    assert rc == 0
    return (out, lse) if want_lse else out


def paged_decode_f64(q, k_pool, v_pool, page_table, seq_lens, block_size, scale=0.0, threads=0):
    """q [S,Hq,D]; pools [num_blocks, bs, Hkv, D] float32; table [S, max_blocks] int32."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k_pool = np.ascontiguousarray(k_pool, dtype=np.float32)
    v_pool = np.ascontiguousarray(v_pool, dtype=np.float32)
    page_table = np.ascontiguousarray(page_table, dtype=np.int32)
    S, Hq, D = q.shape
    nblk, bs, Hkv, _ = k_pool.shape
    assert bs == block_size
    out = np.zeros((S, Hq, D), dtype=np.float64)
    lens_ptr = None
    if seq_lens is not None:
        seq_lens = np.ascontiguousarray(seq_lens, dtype=np.int32)
        lens_ptr = seq_lens.ctypes.data
    if threads <= 0:
        threads = oracle().oracle_max_threads()
    rc = oracle().oracle_paged_decode_f64(q.reshape(-1), k_pool.reshape(-1), v_pool.reshape(-1),
                                          page_table.reshape(-1), lens_ptr, S, Hq, Hkv, D, bs,
                                          page_table.shape[1], nblk, float(scale), out.reshape(-1),
                                          threads)
    assert rc == 0
    return out


class OracleBlockManager:
    """Python face of oracle/kv_oracle.c's allocator (mirrors sca::BlockManager's methods)."""

    def __init__(self, num_blocks, max_num_seqs, max_blocks_per_seq):
        self.lib = oracle()
        self.h = self.lib.oracle_bm_create(num_blocks, max_num_seqs, max_blocks_per_seq)
        assert self.h, "invalid arguments"
        self.num_blocks, self.max_num_seqs, self.max_blocks_per_seq = num_blocks, max_num_seqs, max_blocks_per_seq

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.oracle_bm_destroy(self.h)
            self.h = None

    def allocate(self, count):
        out = np.empty(max(count, 1), dtype=np.int32)
        rc = self.lib.oracle_bm_allocate(self.h, count, out)
        return rc, (out[:count].copy() if rc == 0 else None)

    def free(self, ids):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        self.lib.oracle_bm_free(self.h, ids, ids.size)

    def append_to_table(self, seq, ids):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        return self.lib.oracle_bm_append_to_table(self.h, seq, ids, ids.size)

    def reset_seq(self, seq):
        return self.lib.oracle_bm_reset_seq(self.h, seq)

    @property
    def num_free(self):
        return self.lib.oracle_bm_num_free(self.h)

    @property
    def allocation_failures(self):
        return self.lib.oracle_bm_allocation_failures(self.h)

    @property
    def double_free_events(self):
        return self.lib.oracle_bm_double_free_events(self.h)

    @property
    def revision(self):
        return self.lib.oracle_bm_revision(self.h)

    def table(self):
        p = self.lib.oracle_bm_table(self.h)
        return np.ctypeslib.as_array(p, shape=(self.max_num_seqs, self.max_blocks_per_seq)).copy()

    def free_list(self):
        p = self.lib.oracle_bm_free_list(self.h)
        return np.ctypeslib.as_array(p, shape=(self.num_blocks,))[: self.num_free].copy()


def slot_mapping(row, seq_start, num_tokens, block_size, max_blocks):
    row = np.ascontiguousarray(row, dtype=np.int32)
    out = np.full(max(num_tokens, 1), -1, dtype=np.int32)
    bad = C.c_int64(-1)
    rc = oracle().oracle_slot_mapping(row, seq_start, num_tokens, block_size, max_blocks, out, C.byref(bad))
    return rc, out[:max(num_tokens, 0)], bad.value
