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
