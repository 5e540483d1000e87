"""Split-K decode parity on the GPU, through the C ABI, against the FP64 oracle. Cases mirror the
reference's tests/kernel/test_decode_correctness.cu (split counts x lengths, GQA groups, every head
dim, bf16) and add BSHD layout, fp32, ragged seq_lens and unit-variance inputs."""
import numpy as np
import pytest

import helpers as H
import oracle_lib as ol

pytestmark = pytest.mark.gpu


def run_decode(dt, hq, hkv, skv, d, splits, seed, batch=1, layout="bhsd", normal=False, scale=None):
    import torch
    from scicompute_attention_b200 import ops
    gen = H.normal_inputs if normal else H.uniform_inputs
    qb, qd = gen((batch, hq, 1, d), seed, dt)
    kb, kd = gen((batch, hkv, skv, d), seed + 101, dt)
    vb, vd = gen((batch, hkv, skv, d), seed + 202, dt)
    q, k, v = H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt)
    if layout == "bshd":
        q, k, v = (t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v))
    out, stats = ops.decode_attention(q, k, v, num_splits=splits, layout=layout, scale=scale, return_stats=True)
    torch.cuda.synchronize()
    expect = ol.attention_f64(qd, kd, vd, causal=True, scale=scale or 0.0)
    tag = f"decode dt={dt} B={batch} Hq={hq} Hkv={hkv} Skv={skv} D={d} splits={splits} seed={seed} {layout}"
    H.check_close(H.to_host_f32(out), expect, dt, tag)
    assert tuple(out.shape) == (batch, hq, 1, d)
    if splits > 0:
        assert stats["num_splits"] == splits
    assert stats["workspace_bytes"] > 0


def test_every_split_count_matches_reference():
    seed = 70000
    for splits in (1, 2, 3, 4, 8, 16):
        for skv in (1, 127, 1024, 4096):
            run_decode(ol.DT_F16, 8, 8, skv, 128, splits, seed)
            seed += 1


def test_grouped_query_attention_across_split_counts():
    seed = 71000
    for group in (1, 2, 4, 8):
        for splits in (1, 4, 16):
            run_decode(ol.DT_F16, 8 * group, 8, 2048, 128, splits, seed)
            seed += 1


def test_bf16_and_every_head_dim():
    seed = 72000
    for d in (32, 64, 96, 128, 160, 192, 256):
        run_decode(ol.DT_BF16, 4, 2, 512, d, 4, seed)
        seed += 1


def test_wide_groups_use_both_row_halves_and_head_chunks():
    # group 16 fills all 16 fragment rows, group 32 needs two head chunks per kv head
    run_decode(ol.DT_BF16, 16, 1, 777, 128, 3, 73000)
    run_decode(ol.DT_F16, 32, 1, 300, 64, 2, 73001)
    run_decode(ol.DT_BF16, 24, 2, 513, 128, 0, 73002)


def test_batched_bshd_layout_and_auto_splits():
    run_decode(ol.DT_BF16, 8, 2, 1500, 128, 0, 74000, batch=3, layout="bshd")
    run_decode(ol.DT_F16, 8, 8, 333, 64, 0, 74001, batch=2, layout="bshd")


def test_unit_variance_inputs_qwen_shape():
    # the headline decode shape (H_q=32, H_kv=8, D=128), N(0,1) inputs, reduced batch and length
    run_decode(ol.DT_BF16, 32, 8, 4096, 128, 0, 75000, batch=2, normal=True)
    run_decode(ol.DT_F16, 32, 8, 2048, 128, 8, 75001, batch=1, normal=True)


def test_custom_scale_and_fp32_path():
    run_decode(ol.DT_F16, 8, 4, 640, 128, 4, 76000, scale=0.05)
    run_decode(ol.DT_F32, 4, 2, 384, 64, 4, 76001)
    run_decode(ol.DT_F32, 8, 8, 1024, 128, 1, 76002)


def test_ragged_seq_lens_and_empty_sequence():
    import torch
    from scicompute_attention_b200 import ops
    dt, b, hq, hkv, skv, d = ol.DT_BF16, 4, 8, 2, 900, 128
    qb, qd = H.uniform_inputs((b, hq, 1, d), 77000, dt)
    kb, kd = H.uniform_inputs((b, hkv, skv, d), 77001, dt)
    vb, vd = H.uniform_inputs((b, hkv, skv, d), 77002, dt)
    lens = np.array([900, 1, 0, 517], dtype=np.int32)
    out = ops.decode_attention(H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt), num_splits=5,
                               seq_lens=torch.from_numpy(lens).cuda())
    got = H.to_host_f32(out)
    for i, n in enumerate(lens):
        if n == 0:
            assert (got[i] == 0).all()  # nothing visible: output 0, as for a fully masked row
            continue
        expect = ol.attention_f64(qd[i:i + 1], kd[i:i + 1, :, :n], vd[i:i + 1, :, :n], causal=True)
        H.check_close(got[i:i + 1], expect, dt, f"ragged seq {i} len {n}")


def test_seq_lens_beyond_the_kv_extent_are_clamped():
    """A device length larger than S_kv must not read past the K/V tensors: the result is that of the full extent."""
    import torch
    from scicompute_attention_b200 import ops
    dt, b, hq, hkv, skv, d = ol.DT_F16, 2, 8, 2, 300, 64
    qb, qd = H.uniform_inputs((b, hq, 1, d), 77100, dt)
    kb, kd = H.uniform_inputs((b, hkv, skv, d), 77101, dt)
    vb, vd = H.uniform_inputs((b, hkv, skv, d), 77102, dt)
    q, k, v = H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt)
    lens = torch.tensor([skv + 1000, 123], dtype=torch.int32, device="cuda")
    out = ops.decode_attention(q, k, v, num_splits=3, seq_lens=lens)
    clamped = ops.decode_attention(q, k, v, num_splits=3, seq_lens=torch.tensor([skv, 123], dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    assert torch.equal(out, clamped)
    H.check_close(H.to_host_f32(out)[:1], ol.attention_f64(qd[:1], kd[:1], vd[:1], causal=True), dt, "clamped length")


def test_multi_token_queries_are_rejected():
    import torch
    from scicompute_attention_b200 import _lib, ops
    q = torch.zeros(1, 2, 4, 64, dtype=torch.float16, device="cuda")
    k = torch.zeros(1, 2, 64, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(_lib.ScaError) as e:
        ops.decode_attention(q, k, k)
    assert e.value.code == 5 and "flash" in str(e.value)


def test_sequence_split_merge_matches_unsplit():
    """KV axis cut into 3 uneven shards (one of them empty): per-shard triples merged by the same
    kernel the multi-GPU path uses after its all-gather."""
    import torch
    from scicompute_attention_b200 import ops
    dt, b, hq, hkv, skv, d = ol.DT_BF16, 2, 8, 2, 1100, 128
    qb, qd = H.normal_inputs((b, hq, 1, d), 78000, dt)
    kb, kd = H.normal_inputs((b, hkv, skv, d), 78001, dt)
    vb, vd = H.normal_inputs((b, hkv, skv, d), 78002, dt)
    q, k, v = H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt)
    cuts = [(0, 600), (600, 1100)]
    parts = [ops.decode_triples(q, k[:, :, a:z].contiguous(), v[:, :, a:z].contiguous(), num_splits=3)
             for a, z in cuts]
    empty = torch.zeros_like(parts[0])
    empty[:, 0] = float("-inf")
    gathered = torch.stack(parts + [empty])
    out = ops.merge_triples(gathered, q.dtype).view(b, hq, 1, d)
    expect = ol.attention_f64(qd, kd, vd, causal=True)
    H.check_close(H.to_host_f32(out), expect, dt, "sequence-split merge")
