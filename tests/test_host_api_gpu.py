"""The C++ host layer on a real device: PagedKVCache bookkeeping replayed against the reference's
trace (page table on the DEVICE, lengths and pool bytes bit-exact), the one-launch batched append
against per-sequence appends, and paged attention through sca::paged_attention."""
import ctypes as C
import json
import os
import zlib

import numpy as np
import pytest

import helpers as H
import host_lib
import oracle_lib as ol

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "golden.json")))


def test_paged_cache_trace_matches_the_reference_on_the_device():
    l = host_lib.lib()
    t = GOLDEN["paged_trace"]
    layers, blocks, bs, hkv, d, seqs = t["cfg"]
    buf = C.create_string_buffer(1024)
    h = l.sca_c_paged_create(layers, blocks, bs, hkv, d, ol.DT_F16, seqs, 0, buf, 1024)
    assert h, buf.value
    for ev in t["events"]:
        if ev["op"] == "reset":
            assert l.sca_c_paged_reset_seq(h, ev["seq"]) == ev["rc"]
        else:
            data = np.random.default_rng(ev["data_seed"])
            k = data.integers(0, 65535, size=(ev["n"], hkv, d), dtype=np.uint16)
            v = data.integers(0, 65535, size=(ev["n"], hkv, d), dtype=np.uint16)
            rc = l.sca_c_paged_append(h, ev["seq"], 0, k.ctypes.data, v.ctypes.data, ev["n"], buf, 1024)
            assert rc == ev["rc"], (ev["op"], ev["seq"], ev["n"], buf.value)
        assert [l.sca_c_paged_seq_length(h, s) for s in range(seqs)] == ev["lens"]
        assert [l.sca_c_paged_logical_blocks(h, s) for s in range(seqs)] == ev["blocks"]
    maxb = l.sca_c_paged_max_blocks_per_seq(h)
    assert maxb == t["max_blocks_per_seq"]
    table = np.zeros(seqs * maxb, np.int32)
    lens = np.zeros(seqs, np.int32)
    assert l.sca_c_paged_read_table(h, table, lens.ctypes.data) == 0
    assert table.tolist() == t["table"]                     # device mirror after row-wise syncs
    assert lens.tolist() == t["events"][-1]["lens"]
    nbytes = blocks * bs * hkv * d * 2
    pool = np.zeros(nbytes, np.uint8)
    l.sca_c_paged_read_layer(h, 0, 1, pool.ctypes.data)
    assert zlib.crc32(pool.tobytes()) == t["k_pool_crc"]
    l.sca_c_paged_read_layer(h, 0, 0, pool.ctypes.data)
    assert zlib.crc32(pool.tobytes()) == t["v_pool_crc"]
    stats = (C.c_int64 * 7)()
    l.sca_c_paged_stats(h, stats)
    assert list(stats)[:5] == t["stats"][:5]
    l.sca_c_paged_destroy(h)


def test_batched_append_equals_per_sequence_appends_and_attention_matches_oracle():
    l = host_lib.lib()
    dt, layers, blocks, bs, hkv, hq, d, seqs = ol.DT_BF16, 1, 64, 16, 2, 8, 128, 5
    buf = C.create_string_buffer(1024)
    a = l.sca_c_paged_create(layers, blocks, bs, hkv, d, dt, seqs, 0, buf, 1024)
    b = l.sca_c_paged_create(layers, blocks, bs, hkv, d, dt, seqs, 0, buf, 1024)
    assert a and b
    rng = np.random.default_rng(5)
    prompt = [15, 16, 31, 1, 100]
    kd_all, vd_all = [[] for _ in range(seqs)], [[] for _ in range(seqs)]
    for s, n in enumerate(prompt):  # interleave-free prefill, identical on both caches
        kb, kd = H.normal_inputs((n, hkv, d), 100 + s, dt)
        vb, vd = H.normal_inputs((n, hkv, d), 200 + s, dt)
        for h in (a, b):
            assert l.sca_c_paged_append(h, s, 0, kb.ctypes.data, vb.ctypes.data, n, buf, 1024) == 0
        kd_all[s].append(kd)
        vd_all[s].append(vd)
    for step in range(20):        # 20 decode steps: cache a appends per sequence, cache b in one launch
        kb, kd = H.normal_inputs((seqs, hkv, d), 300 + step, dt)
        vb, vd = H.normal_inputs((seqs, hkv, d), 400 + step, dt)
        for s in range(seqs):
            assert l.sca_c_paged_append(a, s, 0, kb[s:s + 1].ctypes.data, vb[s:s + 1].ctypes.data, 1, buf, 1024) == 0
            kd_all[s].append(kd[s:s + 1])
            vd_all[s].append(vd[s:s + 1])
        assert l.sca_c_paged_append_batch(b, seqs, 0, kb.ctypes.data, vb.ctypes.data, buf, 1024) == 0, buf.value
    maxb = l.sca_c_paged_max_blocks_per_seq(a)
    ta, tb = np.zeros(seqs * maxb, np.int32), np.zeros(seqs * maxb, np.int32)
    la, lb = np.zeros(seqs, np.int32), np.zeros(seqs, np.int32)
    assert l.sca_c_paged_read_table(a, ta, la.ctypes.data) == 0 and l.sca_c_paged_read_table(b, tb, lb.ctypes.data) == 0
    assert np.array_equal(ta, tb) and np.array_equal(la, lb) and la.tolist() == [n + 20 for n in prompt]
    nbytes = blocks * bs * hkv * d * 2
    pa, pb = np.zeros(nbytes, np.uint8), np.zeros(nbytes, np.uint8)
    for is_key in (1, 0):
        l.sca_c_paged_read_layer(a, 0, is_key, pa.ctypes.data)
        l.sca_c_paged_read_layer(b, 0, is_key, pb.ctypes.data)
        assert np.array_equal(pa, pb)

    # attention over cache b through sca::paged_attention, against the FP64 oracle on the same tokens
    qb, qd = H.normal_inputs((seqs, hq, 1, d), 500, dt)
    out = np.zeros((seqs, hq, 1, d), np.uint16)
    used = C.c_int64()
    assert l.sca_c_paged_attention(b, qb.ctypes.data, seqs, hq, 0, out.ctypes.data, C.byref(used), buf, 1024) == 0, buf.value
    assert used.value >= 1
    got = ol.decode_bits(out, dt)
    for s in range(seqs):
        k = np.concatenate(kd_all[s]).transpose(1, 0, 2)[None]
        v = np.concatenate(vd_all[s]).transpose(1, 0, 2)[None]
        expect = ol.attention_f64(qd[s:s + 1], k, v, causal=True)
        H.check_close(got[s:s + 1], expect, dt, f"paged via C++ API, seq {s}")
    l.sca_c_paged_destroy(a)
    l.sca_c_paged_destroy(b)


def test_over_budget_cache_is_an_error_code_with_advice_not_an_oom():
    l = host_lib.lib()
    buf = C.create_string_buffer(1024)
    # 32 layers x 1,000,000 blocks of 2 MiB would need ~2 TB
    h = l.sca_c_paged_create(32, 1000000, 16, 8, 128, ol.DT_F16, 4, 0, buf, 1024)
    assert not h
    msg = buf.value.decode()
    assert "[SCA-2007]" in msg and "num_blocks <=" in msg
