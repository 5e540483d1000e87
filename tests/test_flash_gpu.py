"""Flash prefill parity on the GPU, through the C ABI, against the FP64 oracle. Cases mirror the
reference's tests/kernel/test_flash_correctness.cu: both 16-bit dtypes x causal x head dims at S=128,
ragged sequence lengths around the tile edges, GQA with S_q != S_kv under the bottom-right causal
mask, the log-sum-exp output, and the fp32 rejection; plus BSHD inputs and unit-variance inputs in
the headline head geometry."""
import numpy as np
import pytest

import helpers as H
import oracle_lib as ol

pytestmark = pytest.mark.gpu

HEAD_DIMS = (32, 64, 96, 128, 160, 192, 256)


def run_flash(dt, b, hq, hkv, sq, skv, d, causal, seed, layout="bhsd", normal=False, lse=False, scale=None):
    import torch
    from scicompute_attention_b200 import ops
    gen = H.normal_inputs if normal else H.uniform_inputs
    qb, qd = gen((b, hq, sq, d), seed, dt)
    kb, kd = gen((b, hkv, skv, d), seed + 101, dt)
    vb, vd = gen((b, hkv, skv, d), seed + 202, dt)
    q, k, v = H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt)
    if layout == "bshd":
        q, k, v = (t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v))
    res = ops.flash_attention(q, k, v, causal=causal, layout=layout, return_lse=lse, scale=scale)
    torch.cuda.synchronize()
    out = res[0] if lse else res
    tag = f"flash dt={dt} causal={causal} B={b} Hq={hq} Hkv={hkv} Sq={sq} Skv={skv} D={d} seed={seed} {layout}"
    if lse:
        expect, elog = ol.attention_f64(qd, kd, vd, causal=causal, scale=scale or 0.0, want_lse=True)
        got = res[1].cpu().numpy().astype(np.float64)
        assert got.shape == elog.shape
        assert np.abs(got - elog).max() <= 1e-2, tag + " LSE"
    else:
        expect = ol.attention_f64(qd, kd, vd, causal=causal, scale=scale or 0.0)
    assert tuple(out.shape) == (b, hq, sq, d)
    H.check_close(H.to_host_f32(out), expect, dt, tag)


def test_single_tile_non_causal():
    run_flash(ol.DT_BF16, 1, 1, 1, 128, 128, 128, False, 60000)
    run_flash(ol.DT_F16, 1, 2, 2, 128, 128, 128, False, 60001)


def test_dtypes_causal_head_dims_at_128():
    seed = 61000
    for dt in (ol.DT_F16, ol.DT_BF16):
        for causal in (False, True):
            for d in HEAD_DIMS:
                run_flash(dt, 1, 4, 4, 128, 128, d, causal, seed)
                seed += 1


def test_sequence_lengths_around_tile_edges():
    seed = 62000
    for s in (1, 7, 63, 64, 65, 127, 128, 129, 255, 256, 257, 1024):
        for causal in (False, True):
            run_flash(ol.DT_F16, 1, 2, 2, s, s, 128, causal, seed)
            seed += 1


def test_gqa_with_different_q_and_kv_lengths():
    seed = 63000
    for group in (1, 2, 4, 8):
        run_flash(ol.DT_BF16, 2, 2 * group, 2, 96, 160, 64, True, seed)
        run_flash(ol.DT_F16, 1, 2 * group, 2, 300, 700, 128, True, seed + 50)
        seed += 1


def test_log_sum_exp_output():
    run_flash(ol.DT_F16, 1, 4, 2, 200, 330, 128, True, 64000, lse=True)
    run_flash(ol.DT_BF16, 2, 2, 2, 128, 128, 64, False, 64001, lse=True)


def test_bshd_layout_and_custom_scale():
    run_flash(ol.DT_BF16, 2, 4, 2, 260, 260, 128, True, 65000, layout="bshd")
    run_flash(ol.DT_F16, 1, 4, 4, 192, 192, 64, False, 65001, layout="bshd", scale=0.2)


def test_unit_variance_inputs_qwen_head_geometry():
    # headline geometry (H_q=32, H_kv=8, D=128, causal) at a length the FP64 oracle finishes quickly
    run_flash(ol.DT_BF16, 1, 32, 8, 512, 512, 128, True, 66000, normal=True)
    run_flash(ol.DT_F16, 1, 8, 2, 1024, 1024, 128, True, 66001, normal=True)


def test_long_rows_exercise_the_lazy_rescale():
    # logits with a large spread so that the running max moves by more than the rescale threshold
    import torch
    from scicompute_attention_b200 import ops
    dt, b, h, s, d = ol.DT_BF16, 1, 2, 640, 128
    qb, qd = H.uniform_inputs((b, h, s, d), 67000, dt, -6.0, 6.0)
    kb, kd = H.uniform_inputs((b, h, s, d), 67001, dt, -6.0, 6.0)
    vb, vd = H.uniform_inputs((b, h, s, d), 67002, dt)
    out = ops.flash_attention(H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt), causal=False)
    H.check_close(H.to_host_f32(out), ol.attention_f64(qd, kd, vd), dt, "large-spread logits")


def test_flash_status_is_clean_after_normal_launches():
    """Every wait in the kernel is bounded; sca_flash_status reports a launch that gave up. Healthy launches leave 0."""
    import torch
    from scicompute_attention_b200 import ops
    ops.flash_status()  # drop whatever an earlier process phase left
    run_flash(ol.DT_BF16, 1, 4, 2, 333, 333, 128, True, 51000)
    torch.cuda.synchronize()
    assert ops.flash_status() == 0


def test_fp32_is_rejected_with_a_pointer_to_the_reference_backends():
    import torch
    from scicompute_attention_b200 import _lib, ops
    q = torch.zeros(1, 2, 16, 64, dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.ScaError) as e:
        ops.flash_attention(q, q, q)
    assert "naive" in str(e.value)


def test_simt_reference_backend_matches_oracle_including_fp32():
    import torch
    from scicompute_attention_b200 import ops
    for dt, sq, skv, d, causal in ((ol.DT_F32, 40, 72, 64, True), (ol.DT_F16, 33, 33, 96, False),
                                   (ol.DT_BF16, 17, 129, 128, True)):
        qb, qd = H.uniform_inputs((1, 4, sq, d), 68000, dt)
        kb, kd = H.uniform_inputs((1, 2, skv, d), 68001, dt)
        vb, vd = H.uniform_inputs((1, 2, skv, d), 68002, dt)
        expect, elog = ol.attention_f64(qd, kd, vd, causal=causal, want_lse=True)
        for name, fn in (("simt", ops.simt_attention), ("naive", ops.naive_attention)):
            out, lse = fn(H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt), causal=causal, return_lse=True)
            H.check_close(H.to_host_f32(out), expect, dt, f"{name} dt={dt}")
            assert np.abs(lse.cpu().numpy() - elog).max() <= 1e-3, name


def test_packed_variable_length_batches_in_one_launch():
    """Ragged batches through sca_launch_flash_varlen: every sequence must equal the oracle on that sequence alone
    (rows of a neighbouring sequence that a tile load drags in must not leak into the result)."""
    import torch
    from scicompute_attention_b200 import ops
    cases = [
        (ol.DT_F16, 128, 8, 2, True, [1, 63, 128, 129, 300, 17, 1000], None),
        (ol.DT_BF16, 128, 32, 8, True, [512, 5, 256, 257], None),
        (ol.DT_F16, 64, 4, 4, False, [40, 256, 3, 700], [90, 256, 64, 701]),
        (ol.DT_BF16, 256, 4, 2, True, [130, 64, 1, 250], [200, 64, 5, 250]),
        (ol.DT_F16, 96, 6, 3, True, [77, 200], None),
    ]
    seed = 69000
    for dt, d, hq, hkv, causal, q_lens, kv_lens in cases:
        kv_lens = kv_lens or q_lens
        cu_q = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
        cu_kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
        # unit-variance logits; V uniform in [-1, 1] so that |out| < 1 and the bf16 output rounding (half an ulp is
        # 7.8e-3 in [2, 4)) cannot reach the 8e-3 bound by itself
        qb, qd = H.normal_inputs((int(cu_q[-1]), hq, d), seed, dt)
        kb, kd = H.normal_inputs((int(cu_kv[-1]), hkv, d), seed + 1, dt)
        vb, vd = H.uniform_inputs((int(cu_kv[-1]), hkv, d), seed + 2, dt)
        out = ops.flash_attention_varlen(H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt), cu_q, cu_kv,
                                         causal=causal)
        torch.cuda.synchronize()
        got = H.to_host_f32(out)
        for s in range(len(q_lens)):
            qs = qd[cu_q[s]:cu_q[s + 1]].transpose(1, 0, 2)[None]
            ks = kd[cu_kv[s]:cu_kv[s + 1]].transpose(1, 0, 2)[None]
            vs = vd[cu_kv[s]:cu_kv[s + 1]].transpose(1, 0, 2)[None]
            expect = ol.attention_f64(qs, ks, vs, causal=causal)
            H.check_close(got[cu_q[s]:cu_q[s + 1]].transpose(1, 0, 2)[None], expect, dt,
                          f"varlen dt={dt} D={d} seq {s} S_q={q_lens[s]} S_kv={kv_lens[s]} causal={causal}")
        seed += 10
    # argument checks: a causal sequence with fewer keys than queries, and offsets that do not end at the totals
    q = torch.zeros(8, 2, 64, dtype=torch.float16, device="cuda")
    from scicompute_attention_b200 import _lib
    with pytest.raises(_lib.ScaError):
        ops.flash_attention_varlen(q, q[:6].contiguous(), q[:6].contiguous(), [0, 8], [0, 6], causal=True)
    with pytest.raises(_lib.ScaError):
        ops.flash_attention_varlen(q, q, q, [0, 7], [0, 8])
