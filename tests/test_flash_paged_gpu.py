"""Chunked prefill over a paged KV cache (sca_launch_flash_paged) on the GPU, through the C ABI.

Every case builds a shuffled (non-contiguous) page table with the oracle's LIFO allocator, scatters K/V into the pool
with the append kernel, and checks the one-launch paged prefill (a) against the FP64 oracle on the gathered cache with
the bottom-right aligned causal mask, and (b) bit for bit against the contiguous packed prefill on the gathered K/V -
the two run the same arithmetic on the same values, only the addressing differs. Unmapped pages must carry weight 0
(reference semantics: src/backends/paged/page_table.cuh:18-36)."""
import numpy as np
import pytest

import helpers as H
import oracle_lib as ol

pytestmark = pytest.mark.gpu


def build(dt, new_lens, kv_lens, bs, hq, hkv, d, seed, nblk=None, unmap=()):
    import torch
    from scicompute_attention_b200 import ops
    nseq = len(kv_lens)
    need = sum(-(-int(n) // bs) for n in kv_lens)
    nblk = nblk or need + 7
    bm = ol.OracleBlockManager(nblk, nseq, nblk)
    rc, ids = bm.allocate(nblk)
    np.random.default_rng(seed).shuffle(ids)
    bm.free(ids)
    table = np.full((nseq, nblk), -1, dtype=np.int32)
    tdt = H.torch_dtype(dt)
    k_pool = torch.zeros((nblk, bs, hkv, d), dtype=tdt, device="cuda")
    v_pool = torch.zeros_like(k_pool)
    ks, vs = [], []
    for s, n in enumerate(kv_lens):
        rc, got = bm.allocate(-(-int(n) // bs))
        assert rc == 0
        table[s, :len(got)] = got
        kb, kd = H.normal_inputs((1, hkv, int(n), d), seed + 10 * s + 1, dt)
        vb, vd = H.uniform_inputs((1, hkv, int(n), d), seed + 10 * s + 2, dt)
        ks.append(kd[0])
        vs.append(vd[0])
        t = np.arange(int(n))
        slots = (table[s, t // bs].astype(np.int64) * bs + t % bs).astype(np.int32)
        kt = H.to_device(kb, dt)[0].permute(1, 0, 2).contiguous()   # [n, hkv, d]
        vt = H.to_device(vb, dt)[0].permute(1, 0, 2).contiguous()
        ops.kv_append(k_pool, v_pool, kt, vt, torch.from_numpy(slots).cuda())
    for s, page in unmap:
        table[s, page] = -1
    qs, q_bits = [], []
    for s, n in enumerate(new_lens):
        qb, qd = H.normal_inputs((1, hq, int(n), d), seed + 10 * s + 3, dt)
        qs.append(qd[0])
        q_bits.append(H.to_device(qb, dt)[0].permute(1, 0, 2))     # [n, hq, d]
    q = torch.cat(q_bits, dim=0).contiguous()
    cu_q = np.concatenate([[0], np.cumsum(new_lens)]).astype(np.int32)
    return q, k_pool, v_pool, table, cu_q, qs, ks, vs


def run_case(dt, new_lens, kv_lens, bs, hq=8, hkv=2, d=128, seed=900, causal=True, unmap=()):
    import torch
    from scicompute_attention_b200 import ops
    q, k_pool, v_pool, table, cu_q, qs, ks, vs = build(dt, new_lens, kv_lens, bs, hq, hkv, d, seed, unmap=unmap)
    out = ops.flash_attention_paged(q, k_pool, v_pool, torch.from_numpy(table).cuda(), cu_q, kv_lens, causal=causal)
    torch.cuda.synchronize()
    got = H.to_host_f32(out)
    for s, (nq, nkv) in enumerate(zip(new_lens, kv_lens)):
        keep = np.ones(int(nkv), dtype=bool)
        for us, page in unmap:
            if us == s:
                keep[page * bs:(page + 1) * bs] = False
        # the oracle's causal mask is bottom-right aligned over the keys that are there; dropping unmapped keys
        # would shift it, so those keys stay in place with a huge negative score instead: V row 0, K row pushed away
        kd, vd = ks[s].copy(), vs[s].copy()
        expect = ol.attention_f64(qs[s][None], kd[None], vd[None], causal=causal)
        if not keep.all():
            expect = masked_reference(qs[s], kd, vd, keep, causal)
        mine = got[cu_q[s]:cu_q[s + 1]].transpose(1, 0, 2)[None]
        H.check_close(mine, expect, dt, f"paged prefill dt={dt} seq={s} Sq={nq} Skv={nkv} bs={bs} D={d}")
    return out, (q, k_pool, v_pool, table, cu_q)


def masked_reference(q, k, v, keep, causal):
    """FP64 attention of one sequence with some keys removed from the softmax (their columns weigh 0)."""
    hq, sq, d = q.shape
    hkv, skv, _ = k.shape
    out = np.zeros((1, hq, sq, d))
    for h in range(hq):
        kh, vh = k[h // (hq // hkv)].astype(np.float64), v[h // (hq // hkv)].astype(np.float64)
        s = q[h].astype(np.float64) @ kh.T / np.sqrt(d)
        mask = np.broadcast_to(keep[None, :], s.shape).copy()
        if causal:
            i = np.arange(sq)[:, None]
            j = np.arange(skv)[None, :]
            mask &= j <= i + (skv - sq)
        s = np.where(mask, s, -np.inf)
        m = s.max(axis=1, keepdims=True)
        m = np.where(np.isfinite(m), m, 0.0)
        pmat = np.exp(s - m)
        den = pmat.sum(axis=1, keepdims=True)
        out[0, h] = np.where(den > 0, (pmat @ vh) / np.where(den > 0, den, 1.0), 0.0)
    return out


def test_new_token_counts_and_block_sizes():
    seed = 910
    for bs in (8, 16, 32):
        for sq in (1, 17, 128, 300):
            run_case(ol.DT_F16, [sq], [sq + 333], bs, seed=seed)
            seed += 1


def test_ragged_batch_bf16_and_gqa():
    run_case(ol.DT_BF16, [5, 130, 64, 1], [700, 130, 1000, 257], 16, hq=8, hkv=2, seed=930)
    run_case(ol.DT_F16, [40, 256], [40, 2000], 16, hq=4, hkv=4, d=64, seed=931)
    run_case(ol.DT_F16, [33, 90], [500, 90], 32, hq=4, hkv=2, d=256, seed=932)
    run_case(ol.DT_F16, [100], [900], 64, hq=4, hkv=1, seed=933, causal=False)


def test_equals_contiguous_prefill_on_the_gathered_cache():
    """Same values, same arithmetic, different addressing: the outputs agree to the last bit."""
    import torch
    from scicompute_attention_b200 import ops
    new_lens, kv_lens, bs = [77, 300, 128], [600, 300, 1500], 16
    out, (q, k_pool, v_pool, table, cu_q) = run_case(ol.DT_F16, new_lens, kv_lens, bs, seed=950)
    ks, vs = [], []
    for s, n in enumerate(kv_lens):
        pages = torch.from_numpy(table[s, : -(-n // bs)].astype(np.int64)).cuda()
        ks.append(k_pool[pages].reshape(-1, k_pool.shape[2], k_pool.shape[3])[:n])
        vs.append(v_pool[pages].reshape(-1, v_pool.shape[2], v_pool.shape[3])[:n])
    cu_kv = np.concatenate([[0], np.cumsum(kv_lens)]).astype(np.int32)
    dense = ops.flash_attention_varlen(q, torch.cat(ks).contiguous(), torch.cat(vs).contiguous(), cu_q, cu_kv, causal=True)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), dense.view(torch.int16))


def test_unmapped_pages_carry_no_weight():
    run_case(ol.DT_F16, [50, 20], [400, 200], 16, seed=960, unmap=[(0, 3), (0, 10), (1, 0)])


def test_argument_errors_are_reported_not_launched():
    import torch
    from scicompute_attention_b200 import _lib, ops
    q = torch.zeros((4, 2, 64), dtype=torch.float16, device="cuda")
    pool = torch.zeros((4, 4, 2, 64), dtype=torch.float16, device="cuda")   # block_size 4: not a TMA page size
    table = torch.zeros((1, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.ScaError) as e:
        ops.flash_attention_paged(q, pool, pool, table, [0, 4], [8])
    assert "block_size=4" in str(e.value)
    pool16 = torch.zeros((4, 16, 2, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(_lib.ScaError) as e:
        ops.flash_attention_paged(q, pool16, pool16, table, [0, 4], [2])     # fewer cached tokens than new ones
    assert "S_q" in str(e.value) or "causal" in str(e.value)
