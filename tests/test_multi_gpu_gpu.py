"""Sequence-split decode on two real GPUs; the result must match the FP64 oracle on the unsplit sequence.
Two exchanges are covered: (1) each rank runs the CUDA triples operator on its KV slice, NCCL all-gathers the
triples, each rank merges on the device; (2) the single kernel that merges, stores the triples into the peer's
mapped buffer over NVLink, waits (bounded) and merges - several steps in a row, one rank without tokens in one of
them, and the status word must stay 0. In-switch reduction is switched off (NCCL_NVLS_ENABLE=0); the peer path uses
plain stores. One process per GPU. Skipped when fewer than two GPUs are visible."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    here = os.path.dirname(os.path.abspath(__file__))
    for p in (os.path.dirname(here), here, os.path.join(os.path.dirname(here), "oracle")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch
    import torch.distributed as dist

    import helpers as H
    import oracle_lib as ol
    from scicompute_attention_b200 import multi_gpu as mg

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    dt, b, hq, hkv, skv, d = ol.DT_BF16, 2, 32, 8, 3001, 128
    qb, qd = H.normal_inputs((b, hq, 1, d), 11, dt)
    kb, kd = H.normal_inputs((b, hkv, skv, d), 12, dt)
    vb, vd = H.normal_inputs((b, hkv, skv, d), 13, dt)
    lo, hi = mg.kv_range_for_rank(skv, rank, world)
    q = H.to_device(qb, dt, f"cuda:{rank}")
    k = H.to_device(np.ascontiguousarray(kb[:, :, lo:hi]), dt, f"cuda:{rank}")
    v = H.to_device(np.ascontiguousarray(vb[:, :, lo:hi]), dt, f"cuda:{rank}")
    out = mg.sequence_split_decode(q, k, v)
    torch.cuda.synchronize()
    expect = ol.attention_f64(qd, kd, vd, causal=True)
    H.check_close(H.to_host_f32(out).reshape(b, hq, 1, d), expect, dt, f"sequence-split decode rank {rank}")

    # the same through the library's own bounded NCCL communicator (C ABI sca_mgpu_*): identical bits, because the
    # same triples are merged by the same kernel
    comm = mg.MgpuComm(rank, world, timeout_ms=20000)
    out_c = mg.sequence_split_decode(q, k, v, comm=comm)
    torch.cuda.synchronize()
    assert torch.equal(out_c.view(torch.int16), out.view(torch.int16))
    mine = torch.full((4, 6), float(rank), dtype=torch.float32, device=f"cuda:{rank}")
    both = comm.allgather_triples(mine)          # bounded completion wait inside the call
    assert [float(both[r].mean()) for r in range(world)] == [float(r) for r in range(world)]
    comm.close()

    # the same through the peer-memory kernel, three steps with different keys (both buffer halves get reused)
    px = mg.PeerExchange(b * hq, d, f"cuda:{rank}")
    for step in range(3):
        kb2, kd2 = H.normal_inputs((b, hkv, skv, d), 20 + step, dt)
        k2 = H.to_device(np.ascontiguousarray(kb2[:, :, lo:hi]), dt, f"cuda:{rank}")
        out2 = px.decode(q, k2, v)
        torch.cuda.synchronize()
        H.check_close(H.to_host_f32(out2).reshape(b, hq, 1, d), ol.attention_f64(qd, kd2, vd, causal=True), dt,
                      f"peer exchange step {step} rank {rank}")
    # a sequence shorter than the world size leaves the last rank without tokens
    lo1, hi1 = mg.kv_range_for_rank(1, rank, world)
    k1 = H.to_device(np.ascontiguousarray(kb[:, :, lo1:hi1]), dt, f"cuda:{rank}")
    v1 = H.to_device(np.ascontiguousarray(vb[:, :, lo1:hi1]), dt, f"cuda:{rank}")
    out3 = px.decode(q, k1, v1)
    torch.cuda.synchronize()
    H.check_close(H.to_host_f32(out3).reshape(b, hq, 1, d), ol.attention_f64(qd, kd[:, :, :1], vd[:, :, :1], causal=True),
                  dt, f"peer exchange, one token, rank {rank}")
    # the same step captured in a CUDA graph and replayed on new keys (the kernel counts the epochs itself)
    kb4, kd4 = H.normal_inputs((b, hkv, skv, d), 30, dt)
    k_static = H.to_device(np.ascontiguousarray(kb4[:, :, lo:hi]), dt, f"cuda:{rank}")
    graph, out4 = px.capture(q, k_static, v)
    for step in range(2):
        kb5, kd5 = H.normal_inputs((b, hkv, skv, d), 31 + step, dt)
        k_static.copy_(H.to_device(np.ascontiguousarray(kb5[:, :, lo:hi]), dt, f"cuda:{rank}"))
        graph.replay()
        torch.cuda.synchronize()
        H.check_close(H.to_host_f32(out4).reshape(b, hq, 1, d), ol.attention_f64(qd, kd5, vd, causal=True), dt,
                      f"peer exchange, graph replay {step}, rank {rank}")
    assert px.status() == 0
    px.close()
    with open(os.path.join(result_dir, f"ok{rank}"), "w") as f:
        f.write("ok")
    dist.barrier()
    dist.destroy_process_group()


def test_a_rank_that_never_joins_gives_a_timeout_status_not_a_hang():
    """Real NCCL, one process, one GPU: rank 0 of a 2-rank communicator whose rank 1 does not exist. The wait is on
    the host (communicator set-up never completes); after the limit the library aborts and returns SCA_TIMEOUT."""
    import ctypes as C
    import time

    import torch
    from scicompute_attention_b200 import _lib
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    l = _lib.lib()
    ident = C.create_string_buffer(_lib.MGPU_ID_BYTES)
    _lib.check(l.sca_mgpu_unique_id(ident))
    comm = C.c_void_p()
    t0 = time.time()
    rc = l.sca_mgpu_init(ident.raw, 0, 2, 1500, C.byref(comm))
    took = time.time() - t0
    assert rc == 500 and comm.value is None, (rc, l.sca_last_error())
    assert 1.4 <= took < 30.0 and b"aborted" in l.sca_last_error()
    # the device is still fine
    assert float(torch.ones(8, device="cuda").sum()) == 8.0


def test_sequence_split_decode_over_nccl_and_over_peer_memory(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))
