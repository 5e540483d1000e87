"""CPU checks of the drop-in boundary: the shared library loads without a GPU and exports every
symbol include/sca_b200.h declares; argument validation answers with status codes, not crashes."""
import ctypes as C
import os
import re

import pytest

from scicompute_attention_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sca_b200.h")).read()
    return sorted(set(re.findall(r"SCA_ABI\s+[\w\s\*]+?\b(sca_\w+)\s*\(", text)))


def test_header_and_loader_agree():
    assert _declared_symbols() == sorted(_lib.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(_lib.KERNEL_LIB)
    missing = [s for s in _declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_struct_sizes_match_header_layout():
    # natural alignment on LP64: pointers/int64 are 8 bytes, so the ctypes mirrors must have
    # exactly these sizes (a mismatch would shift every field after it)
    assert C.sizeof(_lib.DecodeStrides) == 24
    assert C.sizeof(_lib.KvCacheShape) == 32
    # 248 = sizeof(DecodeFwdParams) of the reference (src/backends/decode/decode_splitk.cuh:23-51); the test that
    # compiles the binding stubs against the reference's own headers asserts the same with static_assert
    assert C.sizeof(_lib.DecodeFwdParams) == 7 * 8 + 6 * 8 + 4 * 24 + 8 + 8 + 3 * 8 + 8 == 248
    assert C.sizeof(_lib.DeviceProbe) == 352 and C.sizeof(_lib.DeviceProbeB200) == 368
    assert C.sizeof(_lib.FlashFwdParams) == 5 * 8 + 18 * 8 + 16 + 8 + 8
    assert C.sizeof(_lib.PagedDecodeParams) == C.sizeof(_lib.DecodeFwdParams) + 32
    assert C.sizeof(_lib.FlashVarlenParams) == 4 * 8 + 6 * 8 + 2 * 8 + 4 + 4 + 4 + 4 + 8 + 8
    assert C.sizeof(_lib.SeqSplitExchange) == 16 * 8 + 8 + 3 * 8 + 8 + 3 * 8 + 8 + 8


def test_null_arguments_are_invalid_argument_not_a_crash():
    lib = _lib.lib()
    p = _lib.DecodeFwdParams()
    assert lib.sca_launch_decode_splitk(C.byref(p), None) == 4
    assert b"null pointer" in lib.sca_last_error()
    assert lib.sca_launch_decode_splitk_paged(C.byref(p), None) == 4
    assert b"page_table is null" in lib.sca_last_error()
    pp = _lib.PagedDecodeParams()
    assert lib.sca_launch_paged_attention(C.byref(pp), None) == 4
    assert b"null page table" in lib.sca_last_error()
    shape = _lib.KvCacheShape(4, 16, 2, 64)
    assert lib.sca_launch_kv_append(None, None, None, None, None, 1, C.byref(shape), 2, None) == 4
    assert b"kv append: null pointer" in lib.sca_last_error()
    f = _lib.FlashFwdParams()
    assert lib.sca_launch_simt_forward(C.byref(f), None) == 4
    assert lib.sca_launch_flash_fwd(C.byref(f), None) == 4
    assert b"null tensor pointer" in lib.sca_last_error()


def test_probe_without_a_device_reports_unavailable():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    probe = _lib.DeviceProbeB200()
    rc = _lib.lib().sca_probe_device_b200(0, C.byref(probe))
    assert rc != 0 and probe.base.cuda_available == 0
    assert probe.binary_has_sm100a == 1


def test_reference_sized_probe_struct_is_not_overrun():
    """sca_probe_device must write exactly the reference's struct (src/runtime/device_probe.h): a caller built against
    that header hands in 352 bytes, so the bytes behind them must stay untouched."""
    buf = (C.c_ubyte * (C.sizeof(_lib.DeviceProbe) + 64))(*([0xAB] * (C.sizeof(_lib.DeviceProbe) + 64)))
    _lib.lib().sca_probe_device(0, C.cast(buf, C.POINTER(_lib.DeviceProbe)))
    assert bytes(buf[C.sizeof(_lib.DeviceProbe):]) == bytes([0xAB] * 64)


def test_python_ops_refuse_cpu_tensors():
    import torch
    from scicompute_attention_b200 import ops
    q = torch.zeros(1, 2, 1, 64, dtype=torch.float16)
    k = torch.zeros(1, 2, 8, 64, dtype=torch.float16)
    with pytest.raises(_lib.ScaError) as e:
        ops.decode_attention(q, k, k)
    assert "no CPU path" in str(e.value)
    # every operator of the package answers the same way: there is no host fallback anywhere
    packed = torch.zeros(8, 2, 64, dtype=torch.float16)
    table = torch.zeros(1, 4, dtype=torch.int32)
    for call in (lambda: ops.flash_attention(k, k, k),
                 lambda: ops.flash_attention_varlen(packed, packed, packed, [0, 8], [0, 8]),
                 lambda: ops.simt_attention(k, k, k),
                 lambda: ops.naive_attention(k, k, k),
                 lambda: ops.decode_partials(q, k, k),
                 lambda: ops.decode_triples(q, k, k),
                 lambda: ops.paged_attention(q, torch.zeros(4, 2, 2, 64, dtype=torch.float16),
                                             torch.zeros(4, 2, 2, 64, dtype=torch.float16), table, None, block_size=2)):
        with pytest.raises(_lib.ScaError) as e:
            call()
        assert "no CPU path" in str(e.value)


def test_new_entry_points_validate_before_touching_the_device():
    import numpy as np
    lib = _lib.lib()
    assert lib.sca_launch_flash_varlen(None, None) == 4
    p = _lib.FlashVarlenParams()
    cu = np.array([0, 5, 9], dtype=np.int32)
    p.cu_seqlens_q, p.cu_seqlens_kv = cu.ctypes.data, cu.ctypes.data
    p.num_seqs, p.total_q, p.total_kv = 2, 10, 9   # offsets end at 9, total_q says 10
    assert lib.sca_launch_flash_varlen(C.byref(p), None) == 4
    assert b"offsets" in lib.sca_last_error()
    assert lib.sca_flash_varlen_workspace_bytes(0, 10) == -1 and lib.sca_flash_varlen_workspace_bytes(3, 1000) > 3 * 16
    assert lib.sca_launch_seqsplit_exchange(None, None) == 4
    x = _lib.SeqSplitExchange()
    x.rank, x.world = 2, 2
    assert lib.sca_launch_seqsplit_exchange(C.byref(x), None) == 4 and b"rank" in lib.sca_last_error()
    assert lib.sca_peer_buffer_bytes(2, 256, 128) == 512 + 2 * 2 * 256 * 130 * 4
    assert lib.sca_launch_decode_partials(None, None) == 4
