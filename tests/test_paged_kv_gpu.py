"""KV-cache kernels and paged decode on the GPU, through the C ABI.

Integer/byte work (slot placement, pool contents, reset, gather) must be bit-exact against
oracle/kv_oracle.c; the attention output is checked against the FP64 oracle walking the same page
table. Cases mirror tests/kv/test_kv_cache.cpp (append -> gather -> reset round trip, block sizes
{1,8,16,32,64}) and tests/kernel/test_paged_correctness.cu (block sizes {1,8,16,32} at S_kv=257,
GQA x {33,129,512}) and add shuffled (non-contiguous) page tables, unmapped pages and ragged lengths."""
import numpy as np
import pytest

import helpers as H
import oracle_lib as ol

pytestmark = pytest.mark.gpu


def _pool_bytes(nblk, bs, hkv, d, elem):
    return nblk * bs * hkv * d * elem


def test_append_gather_reset_round_trip_all_block_sizes():
    import torch
    from scicompute_attention_b200 import ops
    for dt, elem in ((ol.DT_F16, 2), (ol.DT_F32, 4)):
        for bs in (1, 8, 16, 32, 64):
            nblk, hkv, d, ntok = 8, 2, 64, 3 * bs + 1
            rng = np.random.default_rng(1000 + bs)
            k_new = rng.integers(0, 256, size=(ntok, hkv, d * elem), dtype=np.uint8)
            v_new = rng.integers(0, 256, size=(ntok, hkv, d * elem), dtype=np.uint8)
            slots = rng.permutation(nblk * bs)[:ntok].astype(np.int32)
            slots[0] = -1                      # "do not store"
            if ntok > 2:
                slots[2] = nblk * bs + 5       # block out of range: skipped
            ek = np.zeros(_pool_bytes(nblk, bs, hkv, d, elem), np.uint8)
            ev = np.zeros_like(ek)
            ol.oracle().oracle_kv_append(ek, ev, k_new.reshape(-1), v_new.reshape(-1), slots, ntok, nblk, bs, hkv, d, elem)

            tdt = H.torch_dtype(dt)
            lk = torch.zeros((nblk, bs, hkv, d), dtype=tdt, device="cuda")
            lv = torch.zeros_like(lk)
            kn = torch.from_numpy(k_new).cuda().view(tdt).view(ntok, hkv, d)
            vn = torch.from_numpy(v_new).cuda().view(tdt).view(ntok, hkv, d)
            ops.kv_append(lk, lv, kn, vn, torch.from_numpy(slots).cuda())
            assert np.array_equal(lk.view(torch.uint8).cpu().numpy().reshape(-1), ek), (dt, bs)
            assert np.array_equal(lv.view(torch.uint8).cpu().numpy().reshape(-1), ev), (dt, bs)

            ids = np.array([1, 0, -1, nblk, 5], dtype=np.int32)  # includes invalid ids -> zeros
            per_block = bs * hkv * d * elem
            eg = np.empty(ids.size * per_block, np.uint8)
            ol.oracle().oracle_kv_gather(ek, ids, ids.size, eg, nblk, bs, hkv, d, elem)
            got = ops.kv_gather(lk, torch.from_numpy(ids).cuda())
            assert np.array_equal(got.view(torch.uint8).cpu().numpy().reshape(-1), eg)

            ol.oracle().oracle_kv_reset(ek, ev, ids, ids.size, nblk, bs, hkv, d, elem)
            ops.kv_reset(lk, lv, torch.from_numpy(ids).cuda())
            assert np.array_equal(lk.view(torch.uint8).cpu().numpy().reshape(-1), ek)
            assert np.array_equal(lv.view(torch.uint8).cpu().numpy().reshape(-1), ev)


def test_block_id_lists_in_host_memory_are_staged_not_dereferenced():
    """The reference's PagedKVCache::ResetSeq passes KVCache::Reset the ids of a std::vector
    (src/kv_cache/paged_kv_cache.cpp:150-156). Reset and gather must give the same bytes for a list in pageable or
    pinned host memory as for the same list on the device - and must never read a host address from a kernel."""
    import ctypes as C

    import torch
    from scicompute_attention_b200 import _lib, ops
    nblk, bs, hkv, d = 6, 8, 2, 64
    rng = np.random.default_rng(7)
    lk = torch.from_numpy(rng.integers(1, 255, size=(nblk, bs, hkv, d * 2), dtype=np.uint8)).cuda().view(torch.float16)
    lv = torch.from_numpy(rng.integers(1, 255, size=(nblk, bs, hkv, d * 2), dtype=np.uint8)).cuda().view(torch.float16)
    lk = lk.view(nblk, bs, hkv, d)
    lv = lv.view(nblk, bs, hkv, d)
    ids = np.array([4, 1, -1, nblk], dtype=np.int32)
    shape = _lib.KvCacheShape(nblk, bs, hkv, d)
    want_gather = ops.kv_gather(lk, torch.from_numpy(ids).cuda())
    for kind in ("pageable", "pinned"):
        host = torch.from_numpy(ids.copy())
        if kind == "pinned":
            host = host.pin_memory()
        out = torch.empty_like(want_gather)
        _lib.check(_lib.lib().sca_launch_kv_gather(lk.data_ptr(), host.data_ptr(), ids.size, out.data_ptr(),
                                                   C.byref(shape), 2, None))
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.uint8), want_gather.view(torch.uint8)), kind
        k2, v2 = lk.clone(), lv.clone()
        k3, v3 = lk.clone(), lv.clone()
        ops.kv_reset(k2, v2, torch.from_numpy(ids).cuda())
        _lib.check(_lib.lib().sca_launch_kv_reset_block(k3.data_ptr(), v3.data_ptr(), host.data_ptr(), ids.size,
                                                        C.byref(shape), 2, None))
        torch.cuda.synchronize()
        assert torch.equal(k2.view(torch.uint8), k3.view(torch.uint8)) and torch.equal(v2.view(torch.uint8), v3.view(torch.uint8)), kind
        assert int(k3[4].view(torch.uint8).max()) == 0 and int(k3[1].view(torch.uint8).max()) == 0
        assert int(k3[0].view(torch.uint8).min()) > 0


def build_paged_case(dt, lens, bs, hkv, d, nblk, seed, shuffle=True, unmap=()):
    """Allocates pages through the oracle's LIFO allocator after a seeded shuffle of its free list,
    fills K/V for every sequence, and returns host-side truth."""
    nseq = len(lens)
    max_blocks = nblk
    bm = ol.OracleBlockManager(nblk, nseq, max_blocks)
    if shuffle:
        rc, ids = bm.allocate(nblk)
        assert rc == 0 and np.array_equal(ids, np.arange(nblk))
        np.random.default_rng(seed).shuffle(ids)
        bm.free(ids)
    slots_all = []
    for s, n in enumerate(lens):
        need = -(-int(n) // bs)
        if need > 0:
            rc, got = bm.allocate(need)
            assert rc == 0
            assert bm.append_to_table(s, got) == 0
        rc, slots, _ = ol.slot_mapping(bm.table()[s], 0, int(n), bs, max_blocks) if n > 0 else (0, np.empty(0, np.int32), -1)
        assert rc == 0
        slots_all.append(slots.copy())
    table = bm.table()
    total = int(sum(lens))
    kb, kd = H.normal_inputs((total, hkv, d), seed + 1, dt)
    vb, vd = H.normal_inputs((total, hkv, d), seed + 2, dt)
    slots = np.concatenate(slots_all) if total else np.empty(0, np.int32)
    k_pool = np.zeros((nblk * bs, hkv, d), np.float32)
    v_pool = np.zeros_like(k_pool)
    k_pool[slots] = kd
    v_pool[slots] = vd
    for (s, logical) in unmap:
        table[s, logical] = -1
    return dict(table=table, slots=slots, kb=kb, vb=vb, k_pool=k_pool.reshape(nblk, bs, hkv, d),
                v_pool=v_pool.reshape(nblk, bs, hkv, d), bm=bm)


def run_paged(dt, lens, bs, hq, hkv, d, nblk, seed, splits=0, shuffle=True, unmap=(), use_lens=True):
    import torch
    from scicompute_attention_b200 import ops
    case = build_paged_case(dt, lens, bs, hkv, d, nblk, seed, shuffle, unmap)
    nseq = len(lens)
    tdt = H.torch_dtype(dt)
    lk = torch.zeros((nblk, bs, hkv, d), dtype=tdt, device="cuda")
    lv = torch.zeros_like(lk)
    if case["slots"].size:
        ops.kv_append(lk, lv, H.to_device(case["kb"], dt), H.to_device(case["vb"], dt),
                      torch.from_numpy(case["slots"]).cuda())
    # pool contents are bit-exact images of the oracle's pool
    kbits, _ = ol.encode(case["k_pool"], dt)
    assert torch.equal(lk.cpu().view(torch.int16 if dt != ol.DT_F32 else tdt),
                       torch.from_numpy(kbits.view(np.int16) if dt != ol.DT_F32 else kbits).view(nblk, bs, hkv, d))
    qb, qd = H.normal_inputs((nseq, hq, 1, d), seed + 3, dt)
    lens_np = np.asarray(lens, dtype=np.int32)
    out = ops.paged_attention(H.to_device(qb, dt), lk, lv, torch.from_numpy(case["table"]).cuda(),
                              torch.from_numpy(lens_np).cuda() if use_lens else None, block_size=bs,
                              num_splits=splits, typical_len=int(np.mean(lens)) if len(lens) else 0)
    expect = ol.paged_decode_f64(qd[:, :, 0, :], case["k_pool"], case["v_pool"], case["table"],
                                 lens_np if use_lens else None, bs)
    H.check_close(H.to_host_f32(out)[:, :, 0, :], expect, dt,
                  f"paged dt={dt} lens={list(lens)[:6]} bs={bs} Hq={hq} Hkv={hkv} D={d} splits={splits}")
    if dt != ol.DT_F32 and nseq > 1:
        # the scheduling hint (longest first) changes which thread block does what, never the result
        order = torch.from_numpy(np.argsort(-lens_np, kind="stable").astype(np.int32)).cuda()
        hinted = ops.paged_attention(H.to_device(qb, dt), lk, lv, torch.from_numpy(case["table"]).cuda(),
                                     torch.from_numpy(lens_np).cuda() if use_lens else None, block_size=bs,
                                     num_splits=splits, typical_len=int(np.mean(lens)), seq_order=order)
        assert torch.equal(hinted, out)


def test_block_sizes_at_257_tokens():
    for i, bs in enumerate((1, 8, 16, 32)):
        nblk = -(-257 // bs) + 3
        run_paged(ol.DT_F16, [257], bs, 8, 8, 128, nblk, 80000 + i, splits=4)


def test_gqa_groups_and_lengths():
    seed = 81000
    for group in (1, 2, 4, 8):
        for n in (33, 129, 512):
            run_paged(ol.DT_BF16, [n], 16, 4 * group, 4, 64, 40, seed, splits=3)
            seed += 1


def test_multi_sequence_ragged_shuffled_tables():
    lens = [700, 1, 16, 17, 255, 1024, 333]
    run_paged(ol.DT_BF16, lens, 16, 32, 8, 128, 200, 82000)            # Qwen3-4B head geometry
    run_paged(ol.DT_F16, lens, 16, 8, 2, 128, 200, 82001, splits=16)
    run_paged(ol.DT_F32, [100, 37], 8, 4, 2, 64, 32, 82002, splits=2)


def test_unmapped_pages_get_weight_zero():
    # holes in the table (-1) inside the visible range: those tokens are skipped, as in the reference
    run_paged(ol.DT_BF16, [200, 90], 16, 8, 2, 128, 40, 83000, splits=2, unmap=((0, 3), (0, 7), (1, 0)))


def test_without_seq_lens_scans_the_mapped_range():
    # seq_lens == NULL: every position of max_blocks * block_size is scanned, -1 pages end the data
    run_paged(ol.DT_F16, [64, 128], 16, 4, 2, 64, 12, 84000, splits=2, use_lens=False, shuffle=False)


def test_batched_append_matches_slot_mapping_per_sequence():
    import torch
    from scicompute_attention_b200 import ops
    dt, bs, hkv, d, nblk = ol.DT_BF16, 16, 8, 128, 64
    lens = [15, 16, 31, 1, 100]
    case = build_paged_case(dt, lens, bs, hkv, d, nblk, 85000)
    bm = case["bm"]
    nseq = len(lens)
    # grow every sequence by one token: allocate when the last page is full (PagedKVCache::AppendTokens rule)
    new_lens = np.array(lens, np.int32) + 1
    for s, n in enumerate(lens):
        need = -(-(n + 1) // bs) - (-(-n // bs))
        if need > 0:
            rc, got = bm.allocate(need)
            assert rc == 0 and bm.append_to_table(s, got) == 0
    table = bm.table()
    expect_slots = np.array([ol.slot_mapping(table[s], lens[s], 1, bs, nblk)[1][0] for s in range(nseq)], np.int32)
    kb, _ = H.normal_inputs((nseq, hkv, d), 85001, dt)
    vb, _ = H.normal_inputs((nseq, hkv, d), 85002, dt)
    tdt = H.torch_dtype(dt)
    a_k = torch.zeros((nblk, bs, hkv, d), dtype=tdt, device="cuda"); a_v = torch.zeros_like(a_k)
    b_k = torch.zeros_like(a_k); b_v = torch.zeros_like(a_k)
    ops.kv_append(a_k, a_v, H.to_device(kb, dt), H.to_device(vb, dt), torch.from_numpy(expect_slots).cuda())
    ops.kv_append_batched(b_k, b_v, H.to_device(kb, dt), H.to_device(vb, dt), torch.from_numpy(table).cuda(),
                          torch.from_numpy(new_lens).cuda())
    assert torch.equal(a_k.view(torch.int16), b_k.view(torch.int16))
    assert torch.equal(a_v.view(torch.int16), b_v.view(torch.int16))
    assert int((a_k.view(torch.int16) != 0).any(dim=-1).sum()) > 0
