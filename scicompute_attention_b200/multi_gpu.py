"""Multi-GPU partitioning of the attention hot path: one process per GPU, torch.distributed (NCCL over
NVLink / NVSwitch) as plumbing.

Two schemes, as the workload dictates:
  * independent units - (batch x kv-head-group) for prefill, sequences for decode / paged decode - are
    dealt round-robin to ranks and need no data-path collective at all;
  * long-context decode splits the KV SEQUENCE across ranks: every rank reduces its slice to one
    unnormalised (m, l, O[D]) triple per (batch, head), one small all-gather moves the triples
    (B * H_q * (2 + D) floats per rank), and every rank merges them with the same max-rescaled rule the
    split-K merge kernel uses.
No kernel here reads a peer's memory; every TMA load is a plain per-CTA load; the only cross-GPU traffic is the
all-gather.
"""
from __future__ import annotations

from typing import Callable, Sequence


def units_for_rank(num_units: int, rank: int, world: int) -> list[int]:
    """Round-robin ownership of independent units: rank g of G takes g, g + G, g + 2G, ..."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank={rank} world={world}")
    return list(range(rank, num_units, world))


def prefill_units(batch: int, kv_heads: int) -> list[tuple[int, int]]:
    """The independent units of a GQA prefill: (batch index, kv head); a unit owns the kv head's K/V and
    the `group` query heads that read it."""
    return [(b, h) for b in range(batch) for h in range(kv_heads)]


def kv_range_for_rank(seq_kv: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous token range [lo, hi) of the KV sequence held by `rank` (sizes differ by at most 1;
    trailing ranks may be empty when seq_kv < world)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"rank={rank} world={world}")
    base, extra = divmod(seq_kv, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def sequence_split_decode(q, k_shard, v_shard, *, group=None, scale=None, num_splits: int = 0,
                          triples_fn: Callable | None = None, merge_fn: Callable | None = None,
                          empty_triples_fn: Callable | None = None):
    """Decode attention with the KV sequence sharded over the ranks of `group`.

    q [B, H_q, 1, D] is replicated; k_shard / v_shard [B, H_kv, S_local, D] hold this rank's token range
    (S_local may be 0). Returns the normalised output [B * H_q, D] on every rank.
    `triples_fn`, `merge_fn` and `empty_triples_fn` default to the CUDA operators; the CPU tests of the
    plumbing inject host implementations.
    """
    import torch
    import torch.distributed as dist

    if triples_fn is None or merge_fn is None:
        from . import ops
        triples_fn = triples_fn or (lambda q_, k_, v_: ops.decode_triples(q_, k_, v_, scale=scale, num_splits=num_splits))
        merge_fn = merge_fn or (lambda gathered: ops.merge_triples(gathered, q.dtype))
    b, hq, _, d = q.shape
    if k_shard.shape[2] > 0:
        mine = triples_fn(q, k_shard, v_shard)
    elif empty_triples_fn is not None:
        mine = empty_triples_fn(q)
    else:
        # a rank without tokens contributes m = -inf, l = 0, O = 0 and is skipped by the merge
        mine = torch.zeros((b * hq, 2 + d), dtype=torch.float32, device=q.device)
        mine[:, 0] = float("-inf")
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if world == 1:
        gathered = mine.unsqueeze(0)
    else:
        rows, width = mine.shape
        flat = torch.empty((world * rows, width), dtype=mine.dtype, device=mine.device)  # rank-major concatenation
        dist.all_gather_into_tensor(flat, mine.contiguous(), group=group)
        gathered = flat.view(world, rows, width)
    return merge_fn(gathered)


def shard_sizes(total: int, world: int) -> Sequence[int]:
    return [kv_range_for_rank(total, r, world)[1] - kv_range_for_rank(total, r, world)[0] for r in range(world)]
