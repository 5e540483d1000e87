"""The C++ host layer (libsci_attention.so) against the fixtures generated from the reference's own
host code: validation codes and messages, dispatch decisions and reason text, status mapping, the LIFO
allocator traces, slot mapping and budget arithmetic. Runs without a GPU; like the reference's CPU
build, every backend then answers "no CUDA device available", which is part of the pinned text.
The only intended differences are the dispatch-table revision string and the tile geometry."""
import ctypes as C
import json
import os

import numpy as np

import host_lib

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "golden.json")))
REV = host_lib.lib().sca_c_dispatch_revision().decode()


def _msg(n=2048):
    return C.create_string_buffer(n)


def test_revision_names_the_b200_table():
    assert REV == "b200-r1"


def test_validate_codes_messages_and_scale_match_the_reference():
    l = host_lib.lib()
    for case in GOLDEN["validate"]:
        ci, cf, sh = host_lib.records(case["cfg_i"], case["cfg_f"], case["shape"])
        buf = _msg()
        code = l.sca_c_validate(ci, cf, sh, buf, 2048)
        assert code == case["code"], case
        assert buf.value.decode() == case["message"], case
        assert l.sca_c_effective_scale(ci, cf, sh) == np.float32(case["scale"])


def _normalise(text):
    return text.replace("table=r0", "table=" + REV)


def test_dispatch_decisions_and_reasons_match_the_reference():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("fixtures were generated on a machine without a GPU")
    l = host_lib.lib()
    for case in GOLDEN["dispatch"]:
        ci, cf, sh = host_lib.records([case["backend_in"], 0, 0, 0, 0, 0, case["allow_fallback"], 0, 0], [0, 0],
                                      [1, case["seq_q"], case["seq_kv"], 8, 8, case["head_dim"]])
        buf = _msg()
        backend = l.sca_c_select(ci, cf, sh, buf, 2048, None, None)
        assert backend == case["backend"], case
        assert buf.value.decode() == _normalise(case["reason"]), case
    for case in GOLDEN["validate"]:
        ci, cf, sh = host_lib.records(case["cfg_i"], case["cfg_f"], case["shape"])
        buf = _msg()
        assert l.sca_c_select(ci, cf, sh, buf, 2048, None, None) == case["select_backend"], case
        assert buf.value.decode() == _normalise(case["select_reason"]), case


def test_explain_format_and_blackwell_tile_table():
    l = host_lib.lib()
    buf = _msg()
    ci, cf, sh = host_lib.records([0] * 9, [0, 0], [1, 1024, 1024, 8, 8, 128])
    l.sca_c_explain(ci, cf, sh, buf, 2048)
    text = buf.value.decode()
    for part in ("backend=flash", "tile={bm=128,bn=128,warps=12,stages=5,tma=on}", "workspace=", "reason=auto"):
        assert part in text, text
    tile = (C.c_int32 * 4)()
    for d, expect in ((64, (128, 128, 12, 8)), (128, (128, 128, 12, 5)), (256, (128, 64, 12, 4))):
        ci, cf, sh = host_lib.records([0] * 9, [0, 0], [1, 1024, 1024, 8, 8, d])
        l.sca_c_select(ci, cf, sh, buf, 2048, tile, None)
        assert tuple(tile) == expect


def test_status_mapping_matches_the_reference():
    l = host_lib.lib()
    for code, row in GOLDEN["status"].items():
        sci, name = C.c_int(), C.create_string_buffer(64)
        back = l.sca_c_status_info(int(code), C.byref(sci), name, 64)
        assert (sci.value, name.value.decode(), back) == (row["sci"], row["name"], row["roundtrip"])


def test_varlen_metadata_checks():
    l = host_lib.lib()
    mx, buf = C.c_int64(), _msg()
    assert l.sca_c_varlen_validate(np.array([0, 5, 9, 20], np.int32), 3, C.byref(mx), buf, 2048) == 0 and mx.value == 11
    assert l.sca_c_varlen_validate(np.array([1, 5, 9], np.int32), 2, C.byref(mx), buf, 2048) == 2005
    assert l.sca_c_varlen_validate(np.array([0, 5, 5], np.int32), 2, C.byref(mx), buf, 2048) == 2005
    assert "strictly increasing" in buf.value.decode()


def test_block_manager_traces_match_the_reference():
    l = host_lib.lib()
    for trace in GOLDEN["block_manager_traces"]:
        buf = _msg()
        h = l.sca_c_bm_create(trace["num_blocks"], trace["seqs"], trace["max_blocks"], -1, buf, 2048)
        assert h
        for op in trace["ops"]:
            if op["op"] == "allocate":
                out = np.zeros(max(op["count"], 1), np.int32)
                rc = l.sca_c_bm_allocate(h, op["count"], out, buf, 2048)
                assert rc == op["rc"], op
                if rc == 0:
                    assert out[: op["count"]].tolist() == op["ids"], op
            elif op["op"] == "free":
                ids = np.array(op["ids"], np.int32)
                l.sca_c_bm_free(h, ids, ids.size)
            elif op["op"] == "append":
                ids = np.array(op["ids"], np.int32)
                assert l.sca_c_bm_append_to_table(h, op["seq"], ids.ctypes.data, ids.size, buf, 2048) == op["rc"], op
            else:
                assert l.sca_c_bm_reset_seq(h, op["seq"]) == op["rc"], op
            assert l.sca_c_bm_num_free(h) == op["free"], op
            assert l.sca_c_bm_allocation_failures(h) == op["failures"], op
            assert l.sca_c_bm_double_free_events(h) == op["double_free"], op
            assert l.sca_c_bm_revision(h) == op["revision"], op
        n = trace["seqs"] * trace["max_blocks"]
        assert np.ctypeslib.as_array(l.sca_c_bm_table(h), shape=(n,)).tolist() == trace["table"]
        l.sca_c_bm_destroy(h)


def test_allocator_messages_and_known_answers():
    l = host_lib.lib()
    buf = _msg()
    h = l.sca_c_bm_create(8, 2, 8, -1, buf, 2048)
    out = np.zeros(8, np.int32)
    assert l.sca_c_bm_allocate(h, 8, out, buf, 2048) == 0 and out.tolist() == list(range(8))
    assert l.sca_c_bm_allocate(h, 1, out, buf, 2048) == 2007
    assert "only 0 of 8" in buf.value.decode()
    assert l.sca_c_bm_allocation_failures(h) == 1
    assert l.sca_c_bm_append_to_table(h, 7, None, 1, buf, 2048) == 2005
    l.sca_c_bm_destroy(h)
    assert not l.sca_c_bm_create(0, 1, 1, -1, buf, 2048)
    assert "num_blocks=0" in buf.value.decode()
    # slot mapping and the budget formula (tests/kv/test_kv_cache.cpp:38-81)
    slots = np.zeros(5, np.int32)
    row = np.array([3, 1, 0, -1], np.int32)
    assert l.sca_c_slot_mapping(row.ctypes.data, 17, 5, 16, 4, slots, buf, 2048) == 0 and slots.tolist() == [17, 18, 19, 20, 21]
    assert l.sca_c_slot_mapping(row.ctypes.data, 48, 1, 16, 4, slots, buf, 2048) == 2005 and "empty" in buf.value.decode()
    assert l.sca_c_slot_mapping(None, 0, 1, 16, 4, slots, buf, 2048) == 2005
    assert l.sca_c_kv_cache_bytes(32, 1536, 16, 8, 128, 1, buf, 2048) == 3221225472
    assert l.sca_c_max_blocks_for_budget(32, 16, 8, 128, 1, 3221225472) == 1536
    assert l.sca_c_max_blocks_for_budget(32, 16, 8, 128, 1, 3221225472 // 2) == 768
    assert l.sca_c_kv_cache_bytes(1, 4, 7, 8, 128, 1, buf, 2048) == -2005 and "block_size=7" in buf.value.decode()
    assert l.sca_c_kv_cache_bytes(1, 4, 16, 8, 48, 1, buf, 2048) == -2001


def test_split_policy_tables_agree_between_python_and_cpp():
    from scicompute_attention_b200 import ops
    l = host_lib.lib()
    for args in ((4096, 128, 8, 4, 148), (131072, 8, 8, 4, 148), (300, 1, 1, 1, 148), (4096, 16, 8, 4, 148), (32768, 8, 8, 32, 132)):
        assert l.sca_c_decode_splits_for(*args) == ops.splits_for(*args)
    for args in ((4352, 256, 8, 4, 148), (600, 4, 2, 2, 148), (8192, 32, 8, 4, 148)):
        assert l.sca_c_paged_splits_for(*args) == ops.paged_splits_for(*args)
