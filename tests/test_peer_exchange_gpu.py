"""The fused merge / exchange / merge kernel on ONE GPU, through the C ABI.

(1) world = 1: the kernel exchanges with itself only and must reproduce the split-K decode result.
(2) A peer that never shows up: the kernel is given a second buffer (on the same GPU) as "rank 1", which nothing
    ever publishes an epoch in. The bounded wait must run out (about a second), the kernel must return, set the
    status word, and leave the context usable. No kernel here waits on another kernel.
"""
import ctypes as C

import numpy as np
import pytest

import helpers as H
import oracle_lib as ol

pytestmark = pytest.mark.gpu


def _make_buffer(world, rows, d):
    from scicompute_attention_b200 import _lib
    l = _lib.lib()
    nbytes = l.sca_peer_buffer_bytes(world, rows, d)
    assert nbytes > 0
    ptr = C.c_void_p()
    handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
    _lib.check(l.sca_peer_buffer_create(nbytes, C.byref(ptr), handle))
    return ptr.value


def _exchange(bufs, rank, world, rows, d, splits, epoch, pm, pl, po, out):
    from scicompute_attention_b200 import _lib, ops
    x = _lib.SeqSplitExchange()
    for r, b in enumerate(bufs):
        x.peer_buffers[r] = b
    x.rank, x.world, x.rows, x.head_dim, x.num_splits, x.epoch = rank, world, rows, d, splits, epoch
    x.partial_m, x.partial_l, x.partial_o = pm.data_ptr(), pl.data_ptr(), po.data_ptr()
    x.out, x.out_dtype = out.data_ptr(), ops.dtype_id(out.dtype)
    return _lib.lib().sca_launch_seqsplit_exchange(C.byref(x), ops._stream_ptr(None))


def _status(buf):
    from scicompute_attention_b200 import _lib
    v = C.c_int32(-1)
    _lib.check(_lib.lib().sca_peer_exchange_status(buf, C.byref(v)))
    return v.value


def test_single_rank_exchange_equals_split_k_decode_and_a_missing_peer_times_out():
    import torch
    from scicompute_attention_b200 import _lib, ops
    dt, b, hq, hkv, skv, d = ol.DT_F16, 2, 8, 2, 1500, 128
    qb, qd = H.normal_inputs((b, hq, 1, d), 71, dt)
    kb, kd = H.normal_inputs((b, hkv, skv, d), 72, dt)
    vb, vd = H.normal_inputs((b, hkv, skv, d), 73, dt)
    q, k, v = (H.to_device(x, dt) for x in (qb, kb, vb))
    rows = b * hq
    expect = ol.attention_f64(qd, kd, vd, causal=True)

    own = _make_buffer(1, rows, d)
    for epoch in (1, 2, 3):  # both halves of the buffer, and a reuse
        pm, pl, po, splits = ops.decode_partials(q, k, v, num_splits=4)
        out = torch.empty((rows, d), dtype=q.dtype, device=q.device)
        _lib.check(_exchange([own], 0, 1, rows, d, splits, epoch, pm, pl, po, out))
        torch.cuda.synchronize()
        H.check_close(H.to_host_f32(out).reshape(b, hq, 1, d), expect, dt, f"single-rank exchange, epoch {epoch}")
    assert _status(own) == 0

    # epoch = 0: the kernel counts the steps itself (identical launch parameters every step, as a graph replay needs)
    counted = _make_buffer(1, rows, d)
    for step in range(3):
        pm, pl, po, splits = ops.decode_partials(q, k, v, num_splits=4)
        out = torch.empty((rows, d), dtype=q.dtype, device=q.device)
        _lib.check(_exchange([counted], 0, 1, rows, d, splits, 0, pm, pl, po, out))
        torch.cuda.synchronize()
        H.check_close(H.to_host_f32(out).reshape(b, hq, 1, d), expect, dt, f"single-rank exchange, counted step {step}")
    assert _status(counted) == 0
    _lib.check(_lib.lib().sca_peer_buffer_destroy(counted))

    # head dims 64 and 256 (two columns per thread at 256)
    for d2, seed in ((64, 80), (256, 90)):
        qb2, qd2 = H.normal_inputs((1, 8, 1, d2), seed, ol.DT_BF16)
        kb2, kd2 = H.normal_inputs((1, 2, 700, d2), seed + 1, ol.DT_BF16)
        vb2, vd2 = H.normal_inputs((1, 2, 700, d2), seed + 2, ol.DT_BF16)
        q2, k2, v2 = (H.to_device(x, ol.DT_BF16) for x in (qb2, kb2, vb2))
        buf = _make_buffer(1, 8, d2)
        pm, pl, po, splits = ops.decode_partials(q2, k2, v2, num_splits=3)
        out2 = torch.empty((8, d2), dtype=q2.dtype, device=q2.device)
        _lib.check(_exchange([buf], 0, 1, 8, d2, splits, 1, pm, pl, po, out2))
        torch.cuda.synchronize()
        H.check_close(H.to_host_f32(out2).reshape(1, 8, 1, d2), ol.attention_f64(qd2, kd2, vd2, causal=True), ol.DT_BF16,
                      f"single-rank exchange D={d2}")
        _lib.check(_lib.lib().sca_peer_buffer_destroy(buf))

    # rank 1 never publishes: the wait is bounded and reports through the status word
    mine, ghost = _make_buffer(2, rows, d), _make_buffer(2, rows, d)
    pm, pl, po, splits = ops.decode_partials(q, k, v, num_splits=4)
    out = torch.empty((rows, d), dtype=q.dtype, device=q.device)
    _lib.check(_exchange([mine, ghost], 0, 2, rows, d, splits, 1, pm, pl, po, out))
    torch.cuda.synchronize()
    assert _status(mine) == 1                      # the step (epoch) that gave up
    assert torch.isnan(out.float()).all()          # no stale values pass as a result
    _lib.check(_lib.lib().sca_peer_exchange_clear(mine))
    assert _status(mine) == 0
    # the context is intact: the ordinary operator still works afterwards
    again = ops.decode_attention(q, k, v)
    torch.cuda.synchronize()
    H.check_close(H.to_host_f32(again), expect, dt, "decode after a timed-out exchange")
    for buf in (own, mine, ghost):
        _lib.check(_lib.lib().sca_peer_buffer_destroy(buf))

    # argument checks
    assert _lib.lib().sca_peer_buffer_bytes(0, rows, d) == -1
    assert _lib.lib().sca_peer_buffer_bytes(_lib.PEER_MAX_RANKS + 1, rows, d) == -1
