"""The allocation-free decode entry point, exercised through the C ABI.

Some users of this library cannot obtain device memory around a decode step: they run while a stream
is being captured, or inside a server that has already given all free GPU memory to its own pool, or
under a rule that nothing is allocated after start-up. For them sca_launch_decode_splitk_static keeps
the split-K partials in a fixed 16 MiB array inside the library. This test calls it twice in a row
(the second call finds the first call's data in the shared array) and requires the same output as the
regular entry point, which gets its scratch from the caller. It lives in a file pytest collects last,
so a failure here cannot hide the result of any other test when the run stops at the first failure.
"""
import ctypes as C

import numpy as np
import pytest

import helpers as H
import oracle_lib as ol

pytestmark = pytest.mark.gpu


def _params(q, k, v, out, splits, ws):
    from scicompute_attention_b200 import _lib, ops
    b, hq, _, d = q.shape
    _, hkv, skv, _ = k.shape
    p = _lib.DecodeFwdParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    base = b * hq * splits
    if ws is not None:
        p.partial_m, p.partial_l, p.partial_o = ws.data_ptr(), ws.data_ptr() + 4 * base, ws.data_ptr() + 8 * base
    p.batch, p.num_heads, p.num_kv_heads, p.seq_kv, p.head_dim, p.num_splits = b, hq, hkv, skv, d, splits
    p.q_stride = _lib.DecodeStrides(hq * d, d, d)
    p.k_stride = _lib.DecodeStrides(hkv * skv * d, skv * d, d)
    p.v_stride = p.k_stride
    p.o_stride = _lib.DecodeStrides(hq * d, d, d)
    p.scale = ops.effective_scale(None, d)
    p.dtype = ops.dtype_id(q.dtype)
    return p


def test_static_scratch_decode_matches_the_regular_entry_point_twice():
    import torch
    from scicompute_attention_b200 import _lib
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    dt = ol.DT_BF16
    cases = [(2, 32, 8, 1500, 128, 4, 90000), (3, 8, 2, 700, 64, 7, 90001)]
    for b, hq, hkv, skv, d, splits, seed in cases:
        qb, qd = H.normal_inputs((b, hq, 1, d), seed, dt)
        kb, kd = H.normal_inputs((b, hkv, skv, d), seed + 1, dt)
        vb, vd = H.normal_inputs((b, hkv, skv, d), seed + 2, dt)
        q, k, v = H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt)
        ws = torch.empty(b * hq * splits * (2 + d), dtype=torch.float32, device="cuda")
        ref_out = torch.zeros((b, hq, 1, d), dtype=q.dtype, device="cuda")
        p = _params(q, k, v, ref_out, splits, ws)
        _lib.check(lib.sca_launch_decode_splitk(C.byref(p), stream))
        expect64 = ol.attention_f64(qd, kd, vd, causal=True)
        H.check_close(H.to_host_f32(ref_out), expect64, dt, "regular entry point")
        for call in range(2):
            out = torch.zeros_like(ref_out)
            ps = _params(q, k, v, out, splits, None)  # no caller scratch at all
            _lib.check(lib.sca_launch_decode_splitk_static(C.byref(ps), stream))
            torch.cuda.synchronize()
            got, want = H.to_host_f32(out), H.to_host_f32(ref_out)
            assert np.abs(got - want).max() <= H.MAX_ABS[dt], f"call {call}: differs from the regular entry point"
            H.check_close(got, expect64, dt, f"static scratch, call {call}")


def test_static_scratch_rejects_requests_beyond_its_fixed_size():
    import torch
    from scicompute_attention_b200 import _lib
    lib = _lib.lib()
    d = 128
    q = torch.zeros((1, 8, 1, d), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((1, 8, 64, d), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(q)
    p = _params(q, k, k, out, 16, None)
    p.batch = 4096  # 4096 * 8 * 16 * 130 floats > 4 Mi floats
    rc = lib.sca_launch_decode_splitk_static(C.byref(p), torch.cuda.current_stream().cuda_stream)
    assert rc == 4
    msg = lib.sca_last_error().decode()
    assert "exceeds the built-in scratch" in msg and "4194304" in msg
