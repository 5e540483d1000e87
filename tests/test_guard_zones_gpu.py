"""Kernels write only where they are told to, and leave their inputs alone.

The memory checker of the CUDA toolkit is not available on the machines these tests run on, so the same question is
asked with guard zones: every buffer a kernel writes (outputs, log-sum-exp, split-K partials, KV pools, gather
targets) is carved out of a larger allocation whose surroundings hold a byte pattern, at ragged sizes where an
off-by-one tile would spill (sequence lengths around the 64 / 128 tile edges, padded head dims, first and last block
of a pool). After the kernel the pattern must be intact, the inputs bit-identical, and the result still equal to the
FP64 oracle. Calls go through the C ABI (ctypes) so that outputs and scratch can be placed by the test."""
import ctypes as C

import numpy as np
import pytest

import helpers as H
import oracle_lib as ol

pytestmark = pytest.mark.gpu

GUARD = 4096  # bytes on each side
PATTERN = 0xA5


class Guarded:
    """A device tensor of `shape` inside an allocation with GUARD bytes of PATTERN before and after it."""

    def __init__(self, shape, dtype, fill=None):
        import torch
        self.torch = torch
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        self.n = n
        self.raw = torch.full((GUARD + n + GUARD,), PATTERN, dtype=torch.uint8, device="cuda")
        self.tensor = self.raw[GUARD:GUARD + n].view(dtype).view(shape)
        if fill is not None:
            self.tensor.copy_(fill)

    def intact(self):
        front = self.raw[:GUARD]
        back = self.raw[GUARD + self.n:]
        return bool((front == PATTERN).all()) and bool((back == PATTERN).all())


def _snapshot(*tensors):
    return [t.clone() for t in tensors]


def _unchanged(before, *tensors):
    import torch
    return all(torch.equal(a.view(torch.uint8), b.view(torch.uint8)) for a, b in zip(before, tensors))


def test_prefill_output_and_lse_stay_inside_their_buffers():
    import torch
    from scicompute_attention_b200 import ops
    seed = 91000
    for dt in (ol.DT_F16, ol.DT_BF16):
        for (hq, hkv, sq, skv, d, causal) in ((2, 2, 129, 129, 128, True), (4, 2, 65, 257, 96, True), (2, 1, 127, 63, 32, False),
                                              (2, 2, 1, 130, 160, True), (3, 3, 255, 255, 64, True), (2, 2, 129, 191, 256, False)):
            qb, qd = H.uniform_inputs((1, hq, sq, d), seed, dt)
            kb, kd = H.uniform_inputs((1, hkv, skv, d), seed + 1, dt)
            vb, vd = H.uniform_inputs((1, hkv, skv, d), seed + 2, dt)
            q, k, v = H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt)
            before = _snapshot(q, k, v)
            out = Guarded((1, hq, sq, d), H.torch_dtype(dt))
            lse = Guarded((1, hq, sq), torch.float32)
            ops.flash_attention(q, k, v, causal=causal, return_lse=True, out=out.tensor, lse=lse.tensor)
            torch.cuda.synchronize()
            tag = f"prefill guard dt={dt} Hq={hq} Hkv={hkv} Sq={sq} Skv={skv} D={d} causal={causal}"
            assert out.intact() and lse.intact(), tag + ": wrote outside the output / lse"
            assert _unchanged(before, q, k, v), tag + ": inputs modified"
            H.check_close(H.to_host_f32(out.tensor), ol.attention_f64(qd, kd, vd, causal=causal), dt, tag)
            seed += 10


def _decode_params(lib_mod, q, k, v, out, ws, base, splits, seq_lens=None, page_table=None, block_size=0, max_blocks=0,
                   num_kv_blocks=0, seq_kv=0):
    from scicompute_attention_b200 import ops
    from scicompute_attention_b200._lib import DecodeFwdParams, DecodeStrides
    b, hq, _, d = q.shape
    p = DecodeFwdParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.partial_m = ws.data_ptr()
    p.partial_l = ws.data_ptr() + 4 * base
    p.partial_o = ws.data_ptr() + 8 * base
    p.batch, p.num_heads, p.head_dim, p.num_splits = b, hq, d, splits
    p.q_stride = DecodeStrides(hq * d, d, d)
    p.o_stride = DecodeStrides(hq * d, d, d)
    p.scale = ops.effective_scale(None, d)
    p.dtype = ops.dtype_id(q.dtype)
    if page_table is None:
        hkv, skv = k.shape[1], k.shape[2]
        p.num_kv_heads, p.seq_kv = hkv, skv
        p.k_stride = DecodeStrides(hkv * skv * d, skv * d, d)
        p.v_stride = p.k_stride
        p.page_table = None
    else:
        hkv = k.shape[2]
        p.num_kv_heads, p.seq_kv = hkv, seq_kv
        p.k_stride = DecodeStrides(0, d, hkv * d)
        p.v_stride = p.k_stride
        p.page_table = page_table.data_ptr()
        p.block_size, p.max_blocks_per_seq, p.num_kv_blocks = block_size, max_blocks, num_kv_blocks
    p.seq_lens = seq_lens.data_ptr() if seq_lens is not None else None
    return p


def test_decode_output_and_partials_stay_inside_their_buffers():
    import torch
    from scicompute_attention_b200 import _lib
    lib = _lib.lib()
    seed = 92000
    for dt in (ol.DT_F16, ol.DT_BF16):
        for (b, hq, hkv, skv, d, splits) in ((1, 4, 2, 129, 128, 3), (3, 8, 2, 1000, 64, 7), (2, 6, 6, 65, 256, 1), (5, 32, 8, 700, 128, 16)):
            qb, qd = H.uniform_inputs((b, hq, 1, d), seed, dt)
            kb, kd = H.uniform_inputs((b, hkv, skv, d), seed + 1, dt)
            vb, vd = H.uniform_inputs((b, hkv, skv, d), seed + 2, dt)
            q, k, v = H.to_device(qb, dt), H.to_device(kb, dt), H.to_device(vb, dt)
            lens_host = np.array([skv - (i * 37) % skv for i in range(b)], dtype=np.int32)
            lens = torch.from_numpy(lens_host).cuda()
            before = _snapshot(q, k, v, lens)
            base = b * hq * splits
            out = Guarded((b, hq, 1, d), H.torch_dtype(dt))
            ws = Guarded((base * (2 + d),), torch.float32)
            p = _decode_params(_lib, q, k, v, out.tensor, ws.tensor, base, splits, seq_lens=lens)
            _lib.check(lib.sca_launch_decode_splitk(C.byref(p), None))
            torch.cuda.synchronize()
            tag = f"decode guard dt={dt} B={b} Hq={hq} Hkv={hkv} Skv={skv} D={d} splits={splits}"
            assert out.intact() and ws.intact(), tag + ": wrote outside the output / partial scratch"
            assert _unchanged(before, q, k, v, lens), tag + ": inputs modified"
            expect = np.zeros((b, hq, 1, d))
            for i in range(b):
                n = int(lens_host[i])
                expect[i] = ol.attention_f64(qd[i:i + 1], kd[i:i + 1, :, :n], vd[i:i + 1, :, :n], causal=True)[0]
            H.check_close(H.to_host_f32(out.tensor), expect, dt, tag)
            seed += 10


def test_kv_pool_kernels_touch_only_the_addressed_blocks():
    import torch
    from scicompute_attention_b200 import ops
    rng = np.random.default_rng(93)
    for dt in (torch.float16, torch.bfloat16):
        for (blocks, bs, hkv, d) in ((6, 16, 2, 128), (5, 8, 3, 64), (4, 32, 1, 96)):
            pool_k = Guarded((blocks, bs, hkv, d), dt)
            pool_v = Guarded((blocks, bs, hkv, d), dt)
            pool_k.tensor.zero_()
            pool_v.tensor.zero_()
            # append into the first and the last block, ragged token count
            n = bs + 3
            slots_host = np.concatenate([np.arange(0, bs), (blocks - 1) * bs + np.arange(bs - 3, bs)]).astype(np.int32)
            assert slots_host.shape[0] == n
            k_new = torch.randn((n, hkv, d), device="cuda").to(dt)
            v_new = torch.randn((n, hkv, d), device="cuda").to(dt)
            slots = torch.from_numpy(slots_host).cuda()
            before = _snapshot(k_new, v_new, slots)
            ops.kv_append(pool_k.tensor, pool_v.tensor, k_new, v_new, slots)
            torch.cuda.synchronize()
            tag = f"kv guard dt={dt} blocks={blocks} bs={bs} Hkv={hkv} D={d}"
            assert pool_k.intact() and pool_v.intact(), tag + ": append wrote outside the pool"
            assert _unchanged(before, k_new, v_new, slots), tag + ": append modified its inputs"
            flat_k = pool_k.tensor.view(blocks * bs, hkv, d)
            assert torch.equal(flat_k[slots.long()], k_new)
            untouched = np.setdiff1d(np.arange(blocks * bs), slots_host)
            assert bool((flat_k[torch.from_numpy(untouched).cuda()] == 0).all()), tag + ": append touched other slots"
            # gather into a guarded target, ids in shuffled order
            ids_host = rng.permutation(blocks).astype(np.int32)[: blocks - 1]
            ids = torch.from_numpy(ids_host).cuda()
            from scicompute_attention_b200 import _lib
            target = Guarded((len(ids_host), bs, hkv, d), dt)
            shape = _lib.KvCacheShape(blocks, bs, hkv, d)
            _lib.check(_lib.lib().sca_launch_kv_gather(pool_k.tensor.data_ptr(), ids.data_ptr(), len(ids_host),
                                                       target.tensor.data_ptr(), C.byref(shape), 2, None))
            torch.cuda.synchronize()
            assert target.intact(), tag + ": gather wrote outside its target"
            assert torch.equal(target.tensor, pool_k.tensor[ids.long()])
            # reset the last block only
            last = torch.tensor([blocks - 1], dtype=torch.int32, device="cuda")
            keep = pool_k.tensor[: blocks - 1].clone()
            ops.kv_reset(pool_k.tensor, pool_v.tensor, last)
            torch.cuda.synchronize()
            assert pool_k.intact() and pool_v.intact(), tag + ": reset wrote outside the pool"
            assert bool((pool_k.tensor[blocks - 1] == 0).all()) and torch.equal(pool_k.tensor[: blocks - 1], keep)


def test_batched_append_and_paged_decode_with_guarded_pool_and_scratch():
    import torch
    from scicompute_attention_b200 import _lib, ops
    lib = _lib.lib()
    dt_t, dt = torch.bfloat16, ol.DT_BF16
    nseq, hq, hkv, d, bs, max_blocks = 3, 8, 2, 128, 16, 5
    blocks = nseq * max_blocks
    rng = np.random.default_rng(94)
    lens_host = np.array([15, 16, 47], dtype=np.int32)           # next token lands at a page edge for two of them
    table_host = rng.permutation(blocks).astype(np.int32).reshape(nseq, max_blocks)
    kb, kd = H.uniform_inputs((blocks * bs, hkv, d), 94001, dt)
    vb, vd = H.uniform_inputs((blocks * bs, hkv, d), 94002, dt)
    pool_k = Guarded((blocks, bs, hkv, d), dt_t, fill=H.to_device(kb, dt).view(blocks, bs, hkv, d))
    pool_v = Guarded((blocks, bs, hkv, d), dt_t, fill=H.to_device(vb, dt).view(blocks, bs, hkv, d))
    table = torch.from_numpy(table_host).cuda()
    nb, nd = H.uniform_inputs((nseq, hkv, d), 94003, dt)
    k_new = H.to_device(nb, dt)
    v_new = H.to_device(nb, dt)
    lens_after = torch.from_numpy(lens_host + 1).cuda()   # the kernel takes the lengths that include the new token
    ops.kv_append_batched(pool_k.tensor, pool_v.tensor, k_new, v_new, table, lens_after)
    torch.cuda.synchronize()
    assert pool_k.intact() and pool_v.intact(), "batched append wrote outside the pool"
    for s in range(nseq):
        pos = int(lens_host[s])
        slot = int(table_host[s, pos // bs]) * bs + pos % bs
        assert torch.equal(pool_k.tensor.view(blocks * bs, hkv, d)[slot], k_new[s])
        kd[slot], vd[slot] = nd[s], nd[s]
    qb, qd = H.uniform_inputs((nseq, hq, 1, d), 94004, dt)
    q = H.to_device(qb, dt)
    splits = 4
    base = nseq * hq * splits
    out = Guarded((nseq, hq, 1, d), dt_t)
    ws = Guarded((base * (2 + d),), torch.float32)
    p = _decode_params(_lib, q, pool_k.tensor, pool_v.tensor, out.tensor, ws.tensor, base, splits, seq_lens=lens_after,
                       page_table=table, block_size=bs, max_blocks=max_blocks, num_kv_blocks=blocks, seq_kv=max_blocks * bs)
    _lib.check(lib.sca_launch_decode_splitk_paged(C.byref(p), None))
    torch.cuda.synchronize()
    assert out.intact() and ws.intact(), "paged decode wrote outside the output / partial scratch"
    expect = np.zeros((nseq, hq, 1, d))
    for s in range(nseq):
        n = int(lens_host[s]) + 1
        rows = [int(table_host[s, t // bs]) * bs + t % bs for t in range(n)]
        ks = kd[rows].transpose(1, 0, 2)[None]
        vs = vd[rows].transpose(1, 0, 2)[None]
        expect[s] = ol.attention_f64(qd[s:s + 1], ks, vs, causal=True)[0]
    H.check_close(H.to_host_f32(out.tensor), expect, dt, "paged decode with guarded pool")
