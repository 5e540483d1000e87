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
        out, lse = ops.simt_attention(H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt), causal=causal,
                                      return_lse=True)
        expect, elog = ol.attention_f64(qd, kd, vd, causal=causal, want_lse=True)
        H.check_close(H.to_host_f32(out), expect, dt, f"simt dt={dt}")
        assert np.abs(lse.cpu().numpy() - elog).max() <= 1e-3
