#!/usr/bin/env python
"""Generates tests/golden/*.{json,npz} from the REFERENCE'S OWN host code (oracle/_ref/libsca_ref.so,
built by oracle/build_ref.sh from the reference checkout). Run it only where that library exists; the
committed fixtures let the oracle be checked on machines that do not have the reference.

    python tests/golden/make_golden.py
"""
import ctypes as C
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle_lib as ol  # noqa: E402

ATTENTION_CASES = [
    # (dtype, B, Hq, Hkv, Sq, Skv, D, causal, seed)
    (ol.DT_F16, 1, 2, 2, 33, 33, 64, 0, 101),
    (ol.DT_BF16, 1, 4, 2, 17, 40, 32, 1, 102),
    (ol.DT_F16, 2, 4, 1, 1, 129, 128, 1, 103),
    (ol.DT_F32, 1, 2, 2, 9, 9, 96, 1, 104),
    (ol.DT_BF16, 1, 8, 2, 24, 24, 128, 0, 105),
]


def ref_inputs(shape, seed, dt):
    """xorshift32 values + the reference's rounding -> dequantised float32 (all through the reference)."""
    r = ol.ref()
    n = int(np.prod(shape))
    vals = np.empty(n, np.float32)
    r.ref_random_floats(vals, n, seed, -1.0, 1.0)
    if dt == ol.DT_F16:
        vals = np.array([r.ref_half_bits_to_float(r.ref_float_to_half_bits(float(x))) for x in vals], np.float32)
    elif dt == ol.DT_BF16:
        vals = np.array([r.ref_bf16_bits_to_float(r.ref_float_to_bf16_bits(float(x))) for x in vals], np.float32)
    return vals.reshape(shape)


def block_manager_trace(seed, num_blocks=24, seqs=3, max_blocks=8, steps=120):
    """Random allocate / free / append / reset trace replayed on the reference BlockManager."""
    r = ol.ref()
    rng = np.random.default_rng(seed)
    msg = C.create_string_buffer(512)
    h = r.ref_bm_create(num_blocks, seqs, max_blocks, msg, 512)
    ops, held = [], []
    for _ in range(steps):
        kind = int(rng.integers(0, 5))
        if kind == 0:
            n = int(rng.integers(0, 7))
            out = np.zeros(max(n, 1), np.int32)
            rc = r.ref_bm_allocate(h, n, out, msg, 512)
            ids = out[:n].tolist() if rc == 0 else []
            held += ids
            ops.append({"op": "allocate", "count": n, "rc": rc, "ids": ids})
        elif kind == 1 and held:
            k = int(rng.integers(1, min(4, len(held)) + 1))
            ids = [held.pop(int(rng.integers(0, len(held)))) for _ in range(k)]
            if rng.random() < 0.3:
                ids.append(int(rng.integers(-2, num_blocks + 3)))  # may be invalid or a double free
            arr = np.array(ids, np.int32)
            r.ref_bm_free(h, arr, arr.size)
            ops.append({"op": "free", "ids": ids})
        elif kind == 2 and held:
            k = int(rng.integers(1, min(3, len(held)) + 1))
            ids = [held.pop(0) for _ in range(k)]
            seq = int(rng.integers(-1, seqs + 1))
            arr = np.array(ids, np.int32)
            rc = r.ref_bm_append_to_table(h, seq, arr, arr.size, msg, 512)
            if rc != 0:
                held += ids
            ops.append({"op": "append", "seq": seq, "ids": ids, "rc": rc})
        elif kind == 3:
            seq = int(rng.integers(-1, seqs + 1))
            rc = r.ref_bm_reset_seq(h, seq)
            ops.append({"op": "reset", "seq": seq, "rc": rc})
        else:
            continue
        ops[-1]["free"] = int(r.ref_bm_num_free(h))
        ops[-1]["failures"] = int(r.ref_bm_allocation_failures(h))
        ops[-1]["double_free"] = int(r.ref_bm_double_free_events(h))
        ops[-1]["revision"] = int(r.ref_bm_revision(h))
    table = np.ctypeslib.as_array(r.ref_bm_table(h), shape=(seqs * max_blocks,)).tolist()
    r.ref_bm_destroy(h)
    return {"num_blocks": num_blocks, "seqs": seqs, "max_blocks": max_blocks, "ops": ops, "table": table}


def paged_trace(seed):
    """PagedKVCache::AppendTokens / ResetSeq churn on the reference (host build): page table, lengths, pool bytes."""
    r = ol.ref()
    rng = np.random.default_rng(seed)
    layers, blocks, bs, hkv, d, seqs = 1, 12, 8, 2, 32, 3
    msg = C.create_string_buffer(512)
    h = r.ref_paged_create(layers, blocks, bs, hkv, d, ol.DT_F16, seqs, msg, 512)
    assert h, msg.value
    events = []
    for step in range(40):
        seq = int(rng.integers(0, seqs))
        if rng.random() < 0.2:
            rc = r.ref_paged_reset_seq(h, seq)
            events.append({"op": "reset", "seq": seq, "rc": rc})
        else:
            n = int(rng.integers(1, 20))
            data = np.random.default_rng(seed * 1000 + step)  # the test regenerates the same payload
            k = data.integers(0, 65535, size=(n, hkv, d), dtype=np.uint16)
            v = data.integers(0, 65535, size=(n, hkv, d), dtype=np.uint16)
            rc = r.ref_paged_append(h, seq, 0, k.ctypes.data, v.ctypes.data, n, msg, 512)
            events.append({"op": "append", "seq": seq, "n": n, "rc": rc, "data_seed": seed * 1000 + step})
        events[-1]["lens"] = [int(r.ref_paged_seq_length(h, s)) for s in range(seqs)]
        events[-1]["blocks"] = [int(r.ref_paged_logical_blocks(h, s)) for s in range(seqs)]
    maxb = int(r.ref_paged_max_blocks_per_seq(h))
    table = np.ctypeslib.as_array(r.ref_paged_synced_table(h), shape=(seqs * maxb,)).tolist()
    nbytes = blocks * bs * hkv * d * 2
    kpool = np.ctypeslib.as_array(C.cast(r.ref_paged_layer(h, 0, 1), C.POINTER(C.c_uint8)), shape=(nbytes,)).copy()
    vpool = np.ctypeslib.as_array(C.cast(r.ref_paged_layer(h, 0, 0), C.POINTER(C.c_uint8)), shape=(nbytes,)).copy()
    stats = (C.c_int64 * 7)()
    r.ref_paged_stats(h, stats)
    r.ref_paged_destroy(h)
    import zlib
    return {"cfg": [layers, blocks, bs, hkv, d, seqs], "events": events, "max_blocks_per_seq": maxb, "table": table,
            "k_pool_crc": zlib.crc32(kpool.tobytes()), "v_pool_crc": zlib.crc32(vpool.tobytes()), "stats": list(stats)}


def validate_cases():
    r = ol.ref()
    out = []
    base_cfg_i = [0, 0, 0, 0, 0, 0, 0, 0, 0]
    base_cfg_f = [0.0, 0.0]
    base_shape = [1, 128, 128, 8, 8, 128]
    variations = [
        ({}, {}), ({"layout": 7}, {}), ({}, {"batch": 0}), ({}, {"seq_q": 0}), ({}, {"seq_kv": 0}), ({}, {"heads": 0}),
        ({}, {"kv_heads": 0}), ({}, {"head_dim": 80}), ({}, {"heads": 6, "kv_heads": 4}), ({"causal": 1}, {"seq_q": 64, "seq_kv": 32}),
        ({}, {"heads": 4, "kv_heads": 8}), ({"sliding_window": 128}, {}), ({"softcap": -1.0}, {}), ({"softcap": 30.0, "backend": 1}, {}),
        ({"softcap": 30.0, "backend": 3}, {}), ({"scale": -0.5}, {}), ({"num_splits": -2}, {}), ({"cu_q": 1}, {}), ({"cu_q": 1, "cu_kv": 1}, {}),
        ({"scale": 0.125}, {}), ({"backend": 4}, {"seq_q": 1, "seq_kv": 4096}),
    ]
    ikeys = ["backend", "layout", "causal", "return_lse", "sliding_window", "num_splits", "allow_fallback", "cu_q", "cu_kv"]
    skeys = ["batch", "seq_q", "seq_kv", "heads", "kv_heads", "head_dim"]
    msg = C.create_string_buffer(1024)
    for cv, sv in variations:
        ci = list(base_cfg_i); cf = list(base_cfg_f); sh = list(base_shape)
        for k, v in cv.items():
            if k == "scale": cf[0] = v
            elif k == "softcap": cf[1] = v
            else: ci[ikeys.index(k)] = v
        for k, v in sv.items():
            sh[skeys.index(k)] = v
        a, f, s = np.array(ci, np.int64), np.array(cf, np.float32), np.array(sh, np.int64)
        code = r.ref_validate(a, f, s, msg, 1024)
        vmsg = msg.value.decode()
        scale = float(r.ref_effective_scale(a, f, s))
        backend = r.ref_select(a, f, s, msg, 1024)
        reason = msg.value.decode()
        r.ref_explain(a, f, s, msg, 1024)
        out.append({"cfg_i": ci, "cfg_f": cf, "shape": sh, "code": code, "message": vmsg, "scale": scale,
                    "select_backend": backend, "select_reason": reason, "explain": msg.value.decode()})
    return out


def dispatch_cases():
    """Select() for auto / explicit backends over the shapes the reference's unit tests use. The reference was
    built without CUDA here, so every backend answers 'no CUDA device available'; the backend choice and the
    rule text in front of that answer are what these fixtures pin."""
    r = ol.ref()
    msg = C.create_string_buffer(2048)
    out = []
    for (sq, skv, d, backend, fallback) in [(1, 2048, 128, 0, 0), (16, 4096, 128, 0, 0), (1024, 1024, 128, 0, 0), (64, 64, 128, 0, 0),
                                            (1024, 1024, 128, 1, 0), (1, 100, 64, 0, 0), (8, 64, 64, 0, 0), (2, 256, 128, 0, 0),
                                            (1, 4096, 128, 4, 1), (512, 8192, 256, 0, 1)]:
        ci = np.array([backend, 0, 0, 0, 0, 0, fallback, 0, 0], np.int64)
        cf = np.array([0, 0], np.float32)
        sh = np.array([1, sq, skv, 8, 8, d], np.int64)
        b = r.ref_select(ci, cf, sh, msg, 2048)
        out.append({"seq_q": sq, "seq_kv": skv, "head_dim": d, "backend_in": backend, "allow_fallback": fallback,
                    "backend": b, "reason": msg.value.decode()})
    return out


def main():
    assert ol.have_ref(), "build oracle/_ref first (oracle/build_ref.sh)"
    r = ol.ref()
    arrays = {}
    att = []
    for i, (dt, b, hq, hkv, sq, skv, d, causal, seed) in enumerate(ATTENTION_CASES):
        q = ref_inputs((b, hq, sq, d), seed, dt)
        k = ref_inputs((b, hkv, skv, d), seed + 101, dt)
        v = ref_inputs((b, hkv, skv, d), seed + 202, dt)
        out = np.zeros((b, hq, sq, d), np.float64)
        r.ref_attention(q.reshape(-1), k.reshape(-1), v.reshape(-1), b, hq, hkv, sq, skv, d, causal, out.reshape(-1))
        arrays[f"att{i}_out"] = out  # inputs are regenerated from the seed (generator and rounding are pinned separately)
        att.append([dt, b, hq, hkv, sq, skv, d, causal, seed])
    np.savez_compressed(os.path.join(HERE, "attention_golden.npz"), **arrays)

    tol = {}
    for dt in (0, 1, 2):
        a, m = C.c_double(), C.c_double()
        r.ref_tolerance(dt, C.byref(a), C.byref(m))
        tol[str(dt)] = [a.value, m.value]
    status = {}
    for code in (0, 2001, 2002, 2003, 2004, 2005, 2006, 2007, 2008, 2009, 2010):
        sci, name = C.c_int(), C.create_string_buffer(64)
        back = r.ref_status_info(code, C.byref(sci), name, 64)
        status[str(code)] = {"sci": sci.value, "name": name.value.decode(), "roundtrip": back}
    rounding_inputs = [0.0, -0.0, 1.0, -1.5, 0.1, 3.14159, 65504.0, 65520.0, 1e-5, 6e-8, 1e-8, 300000.0, 0.33325195, 0.99951172]
    golden = {
        "attention_cases": att,
        "reference_tolerances": tol,
        "status": status,
        "rounding": [{"x": x, "half": int(r.ref_float_to_half_bits(x)), "bf16": int(r.ref_float_to_bf16_bits(x))} for x in rounding_inputs],
        "block_manager_traces": [block_manager_trace(s) for s in (1, 2, 3)],
        "paged_trace": paged_trace(7),
        "validate": validate_cases(),
        "dispatch": dispatch_cases(),
    }
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(golden, f, indent=0, separators=(",", ":"))
    print("wrote", os.path.join(HERE, "golden.json"), os.path.getsize(os.path.join(HERE, "golden.json")), "bytes")


if __name__ == "__main__":
    main()
