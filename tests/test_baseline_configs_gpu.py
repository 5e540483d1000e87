"""The five headline configurations at their FULL sizes, on the GPU, through the C ABI.

The FP64 oracle cannot redo a whole 4096-token prefill of 128 heads in a test, so each case checks
  * sampled units against the oracle (the bottom-right aligned causal mask makes "query rows r0..r1 against the
    keys 0..r1" a self-contained oracle problem; for decode a unit is one sequence or one (batch, kv head)), and
  * size-independent properties over the WHOLE output: V = 1 gives O = 1 in every row (the row sums normalise),
    the first causal row is V[0], different split counts agree, paged equals contiguous on the gathered cache.
Inputs are seeded iid N(0,1) generated on the device and cast to the storage type; the oracle sees the same
dequantised values.
  C1 fp16 B=1 H=8 D=128 S=1024 non-causal           C2 bf16/fp16 B=4 Hq=32 Hkv=8 D=128 S=4096 causal
  C3 bf16 B=128 S_kv=4096 split-K decode             C4 256 sequences U[512, 8192], 16-token pages, 160k-block pool
  C5 bf16 B=8 S_kv=131072 (+ D in {64, 256} at S_kv=32768)
"""
import numpy as np
import pytest

import helpers as H
import oracle_lib as ol

pytestmark = pytest.mark.gpu

HQ, HKV, D = 32, 8, 128
GROUP = HQ // HKV


def _randn(shape, seed, dtype, device="cuda"):
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(dtype)


def _dt(dtype):
    import torch
    return {torch.float16: ol.DT_F16, torch.bfloat16: ol.DT_BF16}[dtype]


def _f32(t):
    return H.to_host_f32(t)


def test_c1_reference_runnable_case():
    import torch
    from scicompute_attention_b200 import ops
    q, k, v = (_randn((1, 8, 1024, 128), s, torch.float16) for s in (0, 1, 2))
    out = ops.flash_attention(q, k, v, causal=False)
    torch.cuda.synchronize()
    H.check_close(_f32(out), ol.attention_f64(_f32(q), _f32(k), _f32(v), causal=False), ol.DT_F16, "C1")


@pytest.mark.parametrize("dtype_name", ["bfloat16", "float16"])
def test_c2_prefill_full_size(dtype_name):
    import torch
    from scicompute_attention_b200 import ops
    dtype = getattr(torch, dtype_name)
    b, s = 4, 4096
    q = _randn((b, HQ, s, D), 10, dtype)
    k = _randn((b, HKV, s, D), 11, dtype)
    v = _randn((b, HKV, s, D), 12, dtype)
    out = ops.flash_attention(q, k, v, causal=True)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    # first causal row sees only key 0
    first = out[:, :, 0, :].float()
    v0 = v[:, :, 0, :].float().repeat_interleave(GROUP, dim=1)
    assert (first - v0).abs().max().item() <= H.MAX_ABS[_dt(dtype)]
    # sampled row windows against the oracle: 16 rows ending at r1, all heads of a few (batch, kv head) units
    rng = np.random.default_rng(5)
    for r1 in (16, 129, 1000, 2048, 3333, 4096):
        bi = int(rng.integers(0, b))
        kv = int(rng.integers(0, HKV))
        hs = slice(kv * GROUP, (kv + 1) * GROUP)
        qs = _f32(q[bi:bi + 1, hs, r1 - 16:r1])
        ks = _f32(k[bi:bi + 1, kv:kv + 1, :r1])
        vs = _f32(v[bi:bi + 1, kv:kv + 1, :r1])
        expect = ol.attention_f64(qs, ks, vs, causal=True)
        H.check_close(_f32(out[bi:bi + 1, hs, r1 - 16:r1]), expect, _dt(dtype), f"C2 rows {r1 - 16}..{r1} b={bi} kv={kv}")
    # V = 1: every output element is 1 (up to the rounding of P and of the result)
    ones = torch.ones_like(v)
    out1 = ops.flash_attention(q, k, ones, causal=True)
    torch.cuda.synchronize()
    assert (out1.float() - 1.0).abs().max().item() <= H.MAX_ABS[_dt(dtype)]


@pytest.mark.parametrize("dtype_name", ["bfloat16", "float16"])
def test_c2_prefill_whole_output_against_the_oracle(dtype_name):
    """Every element of the full C2 output (4 x 32 heads x 4096 causal rows) against the FP64 oracle on all host
    threads - about half a minute of host work per dtype."""
    import os

    import torch
    from scicompute_attention_b200 import ops
    dtype = getattr(torch, dtype_name)
    b, s = 4, 4096
    q = _randn((b, HQ, s, D), 10, dtype)
    k = _randn((b, HKV, s, D), 11, dtype)
    v = _randn((b, HKV, s, D), 12, dtype)
    out = ops.flash_attention(q, k, v, causal=True)
    torch.cuda.synchronize()
    threads = os.cpu_count() or 1
    for bi in range(b):  # one batch element at a time keeps the FP64 copies small
        expect = ol.attention_f64(_f32(q[bi:bi + 1]), _f32(k[bi:bi + 1]), _f32(v[bi:bi + 1]), causal=True, threads=threads)
        H.check_close(_f32(out[bi:bi + 1]), expect, _dt(dtype), f"C2 whole output, batch {bi}, {dtype_name}")


def test_c3_split_k_decode_full_size():
    import torch
    from scicompute_attention_b200 import ops
    b, skv = 128, 4096
    q = _randn((b, HQ, 1, D), 20, torch.bfloat16)
    k = _randn((b, HKV, skv, D), 21, torch.bfloat16)
    v = _randn((b, HKV, skv, D), 22, torch.bfloat16)
    out = ops.decode_attention(q, k, v)
    torch.cuda.synchronize()
    for bi in (0, 37, 127):
        expect = ol.attention_f64(_f32(q[bi:bi + 1]), _f32(k[bi:bi + 1]), _f32(v[bi:bi + 1]), causal=True)
        H.check_close(_f32(out[bi:bi + 1]), expect, ol.DT_BF16, f"C3 sequence {bi}")
    # the split count is a scheduling choice: 1, 4 and 16 splits agree with the automatic choice
    for splits in (1, 4, 16):
        other = ops.decode_attention(q, k, v, num_splits=splits)
        torch.cuda.synchronize()
        assert (other.float() - out.float()).abs().max().item() <= H.MAX_ABS[ol.DT_BF16]
    out1 = ops.decode_attention(q, k, torch.ones_like(v))
    torch.cuda.synchronize()
    assert (out1.float() - 1.0).abs().max().item() <= H.MAX_ABS[ol.DT_BF16]


def test_c4_paged_decode_full_size():
    import torch
    from scicompute_attention_b200 import ops
    nseq, bs, nblk = 256, 16, 160000
    rng = np.random.default_rng(30)
    lens = rng.integers(512, 8193, size=nseq).astype(np.int64)
    # LIFO allocator after a seeded shuffle of the free-list order: every allocation pops from the back
    order = np.arange(nblk, dtype=np.int32)
    rng.shuffle(order)
    free = list(order)
    table = np.full((nseq, nblk), -1, dtype=np.int32)
    for s in range(nseq):
        for j in range(-(-(int(lens[s]) + 1) // bs)):
            table[s, j] = free.pop()
    assert len(set(table[table >= 0].tolist())) == int((table >= 0).sum())  # no block is mapped twice
    page_table = torch.from_numpy(table).cuda()
    seq_lens = torch.from_numpy((lens + 1).astype(np.int32)).cuda()
    k_pool = _randn((nblk, bs, HKV, D), 31, torch.bfloat16)
    v_pool = _randn((nblk, bs, HKV, D), 32, torch.bfloat16)
    q = _randn((nseq, HQ, 1, D), 33, torch.bfloat16)
    k_new = _randn((nseq, HKV, D), 34, torch.bfloat16)
    v_new = _randn((nseq, HKV, D), 35, torch.bfloat16)
    ops.kv_append_batched(k_pool, v_pool, k_new, v_new, page_table, seq_lens)
    out = ops.paged_attention(q, k_pool, v_pool, page_table, seq_lens, block_size=bs, typical_len=int(lens.mean()) + 1)
    torch.cuda.synchronize()
    # the appended token sits where ComputeSlotMapping says: last position of each sequence, bit-exact
    for s in (0, 100, 255):
        pos = int(lens[s])
        blk, off = int(table[s, pos // bs]), pos % bs
        assert torch.equal(k_pool[blk, off], k_new[s]) and torch.equal(v_pool[blk, off], v_new[s])
    # sampled sequences: gather their pages into a contiguous cache; oracle and the contiguous kernel must both agree
    for s in (3, 77, 200, int(np.argmax(lens)), int(np.argmin(lens))):
        n = int(lens[s]) + 1
        pages = torch.from_numpy(table[s, :-(-n // bs)].astype(np.int64)).cuda()
        ks = k_pool[pages].reshape(-1, HKV, D)[:n].permute(1, 0, 2).unsqueeze(0).contiguous()
        vs = v_pool[pages].reshape(-1, HKV, D)[:n].permute(1, 0, 2).unsqueeze(0).contiguous()
        expect = ol.attention_f64(_f32(q[s:s + 1]), _f32(ks), _f32(vs), causal=True)
        H.check_close(_f32(out[s:s + 1]), expect, ol.DT_BF16, f"C4 sequence {s} ({n} tokens)")
        dense = ops.decode_attention(q[s:s + 1], ks, vs)
        torch.cuda.synchronize()
        assert (dense.float() - out[s:s + 1].float()).abs().max().item() <= H.MAX_ABS[ol.DT_BF16]


@pytest.mark.parametrize("d,skv,batch", [(128, 131072, 8), (64, 32768, 8), (256, 32768, 8)])
def test_c5_long_context_decode_full_size(d, skv, batch):
    import torch
    from scicompute_attention_b200 import multi_gpu as mg, ops
    q = _randn((batch, HQ, 1, d), 40 + d, torch.bfloat16)
    k = _randn((batch, HKV, skv, d), 41 + d, torch.bfloat16)
    v = _randn((batch, HKV, skv, d), 42 + d, torch.bfloat16)
    out = ops.decode_attention(q, k, v)
    torch.cuda.synchronize()
    for bi, kv in ((0, 0), (batch - 1, HKV - 1)):
        hs = slice(kv * GROUP, (kv + 1) * GROUP)
        expect = ol.attention_f64(_f32(q[bi:bi + 1, hs]), _f32(k[bi:bi + 1, kv:kv + 1]), _f32(v[bi:bi + 1, kv:kv + 1]),
                                  causal=True)
        H.check_close(_f32(out[bi:bi + 1, hs]), expect, ol.DT_BF16, f"C5 D={d} b={bi} kv={kv}")
    # the sequence split used across GPUs, emulated on one: per-slice triples merged by the rank-merge kernel
    world = 8
    triples = []
    for r in range(world):
        lo, hi = mg.kv_range_for_rank(skv, r, world)
        triples.append(ops.decode_triples(q, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous()))
    merged = ops.merge_triples(torch.stack(triples), q.dtype)
    torch.cuda.synchronize()
    assert (merged.float().reshape(batch, HQ, 1, d) - out.float()).abs().max().item() <= H.MAX_ABS[ol.DT_BF16]
