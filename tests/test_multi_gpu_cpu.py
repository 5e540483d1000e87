"""Host-side logic of the multi-GPU paths, on CPU: shard plans, and the sequence-split decode plumbing
(local triples -> all-gather -> merge) run as two gloo ranks with FP64 stand-ins for the two CUDA
operators. One rank holds an empty slice in the second case."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as ol
from scicompute_attention_b200 import multi_gpu as mg


def test_shard_plans():
    assert mg.units_for_rank(32, 3, 8) == [3, 11, 19, 27]
    assert sorted(sum((mg.units_for_rank(10, r, 4) for r in range(4)), [])) == list(range(10))
    assert len(mg.prefill_units(4, 8)) == 32 and mg.prefill_units(4, 8)[9] == (1, 1)
    for total, world in ((131072, 8), (10, 4), (3, 8), (0, 2)):
        ranges = [mg.kv_range_for_rank(total, r, world) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        sizes = mg.shard_sizes(total, world)
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        mg.units_for_rank(4, 4, 4)


def _host_triples(q, k, v):
    """FP64 (m, l, O) per (batch, head) of one KV slice: the contract of the decode-triples operator."""
    b, hq, _, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    qn, kn, vn = q.double().numpy(), k.double().numpy(), v.double().numpy()
    out = np.zeros((b * hq, 2 + d))
    for bi in range(b):
        for h in range(hq):
            s = kn[bi, h // group] @ qn[bi, h, 0] / np.sqrt(d)
            m = s.max()
            w = np.exp(s - m)
            out[bi * hq + h, 0], out[bi * hq + h, 1] = m, w.sum()
            out[bi * hq + h, 2:] = w @ vn[bi, h // group]
    return torch.from_numpy(out).float()


def _host_merge(gathered):
    g = gathered.double().numpy()
    ranks, rows, width = g.shape
    out = np.zeros((rows, width - 2))
    for r in range(rows):
        m = np.ascontiguousarray(g[:, r, 0])
        l = np.ascontiguousarray(g[:, r, 1])
        o = np.ascontiguousarray(g[:, r, 2:])
        ol.oracle().oracle_merge_parts_f64(m, l, o.reshape(-1), ranks, width - 2, out[r])
    return torch.from_numpy(out)


def _worker(rank, world, port, skv, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    b, hq, hkv, d = 2, 4, 2, 32
    q = torch.randn(b, hq, 1, d)
    k = torch.randn(b, hkv, skv, d)
    v = torch.randn(b, hkv, skv, d)
    lo, hi = mg.kv_range_for_rank(skv, rank, world)
    out = mg.sequence_split_decode(q, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous(),
                                   triples_fn=_host_triples, merge_fn=_host_merge)
    expect = ol.attention_f64(q.numpy(), k.numpy(), v.numpy(), causal=True)
    err = np.abs(out.numpy().reshape(b, hq, 1, d) - expect).max()
    with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
        f.write(repr(float(err)))
    dist.barrier()
    dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("skv", [37, 1])  # with 1 token the second rank's slice is empty
def test_sequence_split_decode_over_two_gloo_ranks(tmp_path, skv):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), skv, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err = float(open(tmp_path / f"rank{r}.txt").read())
        assert err < 1e-5, (r, err)   # the stand-in triples travel as fp32
