"""Pins the CPU oracle (oracle/*.c) before anything trusts it:
  * against the committed fixtures generated from the reference's own host code (tests/golden/), always;
  * against that code itself (oracle/_ref/libsca_ref.so) when it has been built on this machine;
  * against the known-answer values the reference's own tests assert (tests/kv/test_kv_cache.cpp:38-81,
    tests/kv/test_block_manager.cpp:30-75, tests/unit/test_config.cpp:84-99).
"""
import ctypes as C
import json
import os
import zlib

import numpy as np
import pytest

import oracle_lib as ol

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "golden.json")))
ATT = np.load(os.path.join(HERE, "golden", "attention_golden.npz"))


def _inputs(shape, seed, dt):
    vals = ol.random_floats(int(np.prod(shape)), seed).reshape(shape)
    return ol.encode(vals, dt)[1]


def test_attention_matches_reference_outputs_bit_for_bit():
    for i, (dt, b, hq, hkv, sq, skv, d, causal, seed) in enumerate(GOLDEN["attention_cases"]):
        q, k, v = _inputs((b, hq, sq, d), seed, dt), _inputs((b, hkv, skv, d), seed + 101, dt), _inputs((b, hkv, skv, d), seed + 202, dt)
        for threads in (1, 4):
            got = ol.attention_f64(q, k, v, causal=bool(causal), threads=threads)
            assert np.array_equal(got, ATT[f"att{i}_out"]), f"case {i} threads={threads}"


def test_rounding_and_status_tables():
    o = ol.oracle()
    for r in GOLDEN["rounding"]:
        assert o.oracle_float_to_half_bits(r["x"]) == r["half"], r
        assert o.oracle_float_to_bf16_bits(r["x"]) == r["bf16"], r
    # numpy's own conversions agree on normal values (the reference flushes fp16 subnormals to zero)
    x = ol.random_floats(4096, 9, -100.0, 100.0)
    bits, deq = ol.encode(x, ol.DT_F16)
    assert np.array_equal(bits, x.astype(np.float16).view(np.uint16))
    assert np.array_equal(ol.decode_bits(bits, ol.DT_F16), deq)
    bits, deq = ol.encode(x, ol.DT_BF16)
    assert np.array_equal(ol.decode_bits(bits, ol.DT_BF16), deq)


def _replay_block_manager(trace):
    bm = ol.OracleBlockManager(trace["num_blocks"], trace["seqs"], trace["max_blocks"])
    for op in trace["ops"]:
        if op["op"] == "allocate":
            rc, ids = bm.allocate(op["count"])
            assert rc == op["rc"], op
            if rc == 0:
                assert ids.tolist() == op["ids"], op
        elif op["op"] == "free":
            bm.free(np.array(op["ids"], np.int32))
        elif op["op"] == "append":
            assert bm.append_to_table(op["seq"], np.array(op["ids"], np.int32)) == op["rc"], op
        elif op["op"] == "reset":
            assert bm.reset_seq(op["seq"]) == op["rc"], op
        assert bm.num_free == op["free"], op
        assert bm.allocation_failures == op["failures"], op
        assert bm.double_free_events == op["double_free"], op
        assert bm.revision == op["revision"], op
    assert bm.table().reshape(-1).tolist() == trace["table"]


def test_block_manager_traces_match_the_reference():
    for trace in GOLDEN["block_manager_traces"]:
        _replay_block_manager(trace)


def test_paged_cache_trace_matches_the_reference():
    """PagedKVCache::AppendTokens / ResetSeq (src/kv_cache/paged_kv_cache.cpp:52-142) replayed with the
    oracle's allocator + slot mapping + byte scatter: table, lengths and pool contents must be equal."""
    t = GOLDEN["paged_trace"]
    layers, blocks, bs, hkv, d, seqs = t["cfg"]
    bm = ol.OracleBlockManager(blocks, seqs, blocks)
    lens = [0] * seqs
    owned = [[] for _ in range(seqs)]
    kpool = np.zeros(blocks * bs * hkv * d * 2, np.uint8)
    vpool = np.zeros_like(kpool)
    o = ol.oracle()
    for ev in t["events"]:
        s = ev["seq"]
        if ev["op"] == "reset":
            if owned[s]:
                ids = np.array(owned[s], np.int32)
                o.oracle_kv_reset(kpool, vpool, ids, ids.size, blocks, bs, hkv, d, 2)
            assert bm.reset_seq(s) == 0
            owned[s], lens[s] = [], 0
            assert ev["rc"] == 0
        else:
            n = ev["n"]
            need = -(-(lens[s] + n) // bs) - len(owned[s])
            ok = True
            if need > 0:
                rc, ids = bm.allocate(need)
                if rc != 0:
                    ok = False
                else:
                    assert bm.append_to_table(s, ids) == 0
                    owned[s] += ids.tolist()
            assert (ev["rc"] == 0) == ok, ev
            if ok:
                row = np.full(blocks, -1, np.int32)
                row[: len(owned[s])] = owned[s]
                rc, slots, _ = ol.slot_mapping(row, lens[s], n, bs, blocks)
                assert rc == 0
                data = np.random.default_rng(ev["data_seed"])
                k = data.integers(0, 65535, size=(n, hkv, d), dtype=np.uint16)
                v = data.integers(0, 65535, size=(n, hkv, d), dtype=np.uint16)
                o.oracle_kv_append(kpool, vpool, k.view(np.uint8).reshape(-1), v.view(np.uint8).reshape(-1),
                                   np.ascontiguousarray(slots), n, blocks, bs, hkv, d, 2)
                lens[s] += n
        assert lens == ev["lens"], ev
        assert [len(x) for x in owned] == ev["blocks"], ev
    table = np.full((seqs, t["max_blocks_per_seq"]), -1, np.int32)
    for s in range(seqs):
        table[s, : len(owned[s])] = owned[s]
    assert table.reshape(-1).tolist() == t["table"]
    assert zlib.crc32(kpool.tobytes()) == t["k_pool_crc"]
    assert zlib.crc32(vpool.tobytes()) == t["v_pool_crc"]
    assert t["stats"][1] == blocks - bm.num_free  # used blocks


def test_known_answers_from_the_reference_tests():
    # tests/kv/test_kv_cache.cpp:62-81
    rc, slots, _ = ol.slot_mapping(np.array([3, 1, 0, -1], np.int32), 17, 5, 16, 4)
    assert rc == 0 and slots.tolist() == [17, 18, 19, 20, 21]
    rc, _, bad = ol.slot_mapping(np.array([3, 1, 0, -1], np.int32), 48, 1, 16, 4)
    assert rc == 2005 and bad == 48          # "is empty (-1)"
    rc, _, _ = ol.slot_mapping(np.array([3, 1, 0, 2], np.int32), 64, 1, 16, 4)
    assert rc == 2007                          # logical block >= max_blocks
    # tests/kv/test_kv_cache.cpp:38-49
    o = ol.oracle()
    assert o.oracle_kv_cache_bytes(32, 1536, 16, 8, 128, 2) == 3221225472
    assert 3221225472 // 1536 == 2097152
    assert o.oracle_max_blocks_for_budget(32, 16, 8, 128, 2, 3221225472) == 1536
    assert o.oracle_max_blocks_for_budget(32, 16, 8, 128, 2, 3221225472 // 2) == 768
    # tests/kv/test_block_manager.cpp:30-75
    bm = ol.OracleBlockManager(16, 2, 8)
    rc, ids = bm.allocate(5)
    assert rc == 0 and ids.tolist() == [0, 1, 2, 3, 4] and bm.num_free == 11
    bm.free(ids)
    assert bm.num_free == 16
    bm2 = ol.OracleBlockManager(8, 1, 8)
    assert bm2.allocate(8)[0] == 0
    assert bm2.allocate(8)[0] == 2007 and bm2.allocation_failures == 1 and bm2.num_free == 0
    bm3 = ol.OracleBlockManager(4, 1, 4)
    rc, ids = bm3.allocate(2)
    bm3.free(ids)
    bm3.free(ids)                              # both ids again -> two double-free events
    assert bm3.double_free_events == 2 and bm3.num_free == 4
    # LIFO: blocks freed last are handed out first
    bm4 = ol.OracleBlockManager(6, 1, 6)
    rc, ids = bm4.allocate(6)
    bm4.free(np.array([4, 1, 5], np.int32))
    assert bm4.allocate(3)[1].tolist() == [5, 1, 4]


@pytest.mark.skipif(not ol.have_ref(), reason="oracle/_ref/libsca_ref.so not built on this machine")
def test_oracle_against_the_reference_library_itself():
    r = ol.ref()
    o = ol.oracle()
    a = ol.random_floats(5000, 77, -3.0, 3.0)
    b = np.empty_like(a)
    r.ref_random_floats(b, a.size, 77, -3.0, 3.0)
    assert np.array_equal(a, b)
    xs = np.concatenate([ol.random_floats(3000, 5, -70000, 70000), ol.random_floats(3000, 6, -1e-4, 1e-4),
                         np.array([0, -0.0, 65504, 65520, 1e9, np.inf, -np.inf], np.float32)])
    for x in xs:
        assert o.oracle_float_to_half_bits(float(x)) == r.ref_float_to_half_bits(float(x))
        assert o.oracle_float_to_bf16_bits(float(x)) == r.ref_float_to_bf16_bits(float(x))
    for (b_, hq, hkv, sq, skv, d, causal) in [(1, 4, 4, 48, 48, 128, 0), (2, 8, 2, 31, 77, 64, 1), (1, 3, 1, 1, 300, 32, 1)]:
        q, k, v = _inputs((b_, hq, sq, d), 11, 2), _inputs((b_, hkv, skv, d), 12, 2), _inputs((b_, hkv, skv, d), 13, 2)
        mine = ol.attention_f64(q, k, v, causal=bool(causal))
        ref = np.zeros_like(mine)
        r.ref_attention(q.reshape(-1), k.reshape(-1), v.reshape(-1), b_, hq, hkv, sq, skv, d, causal, ref.reshape(-1))
        assert np.array_equal(mine, ref)


def test_paged_oracle_equals_contiguous_oracle_on_gathered_kv():
    """The page-table walk of the oracle is checked against the (pinned) contiguous routine."""
    rng = np.random.default_rng(3)
    bs, nblk, hkv, hq, d = 8, 20, 2, 4, 32
    lens = [37, 8, 1]
    perm = rng.permutation(nblk)
    table = np.full((3, nblk), -1, np.int32)
    used = 0
    for s, n in enumerate(lens):
        nb = -(-n // bs)
        table[s, :nb] = perm[used:used + nb]
        used += nb
    kp = rng.standard_normal((nblk, bs, hkv, d)).astype(np.float32)
    vp = rng.standard_normal((nblk, bs, hkv, d)).astype(np.float32)
    q = rng.standard_normal((3, hq, d)).astype(np.float32)
    got = ol.paged_decode_f64(q, kp, vp, table, np.array(lens, np.int32), bs)
    for s, n in enumerate(lens):
        nb = -(-n // bs)
        k = kp[table[s, :nb]].reshape(-1, hkv, d)[:n].transpose(1, 0, 2)[None]
        v = vp[table[s, :nb]].reshape(-1, hkv, d)[:n].transpose(1, 0, 2)[None]
        exp = ol.attention_f64(q[s][None, :, None, :], k, v, causal=True)
        assert np.allclose(got[s], exp[0, :, 0, :], rtol=0, atol=1e-14)
