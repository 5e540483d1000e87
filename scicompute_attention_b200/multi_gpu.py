"""Multi-GPU partitioning of the attention hot path: one process per GPU, torch.distributed (NCCL over
NVLink / NVSwitch) as plumbing.

Two schemes, as the workload dictates:
  * independent units - (batch x kv-head-group) for prefill, sequences for decode / paged decode - are
    dealt round-robin to ranks and need no data-path collective at all;
  * long-context decode splits the KV SEQUENCE across ranks: every rank reduces its slice to one
    unnormalised (m, l, O[D]) triple per (batch, head), one small all-gather moves the triples
    (B * H_q * (2 + D) floats per rank), and every rank merges them with the same max-rescaled rule the
    split-K merge kernel uses.
Two ways to move the triples: `sequence_split_decode` uses one NCCL all-gather between two kernels;
`PeerExchange` maps one small buffer per rank into every peer (CUDA IPC) and lets ONE kernel merge the
local splits, store the triples into all peers over NVLink, wait (bounded) for theirs and do the final
merge - no library collective on the data path. Every TMA load in the package is a plain per-CTA load of
local memory; peers are only touched by plain stores from that kernel.
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


class MgpuComm:
    """The library's own NCCL communicator (sca_mgpu_*): non-blocking, every wait for other ranks bounded by
    `timeout_ms`, after which the communicator is aborted and the call raises ScaError(code 500) instead of hanging.

    Collective constructor: rank 0 makes the 128-byte id and `share_id(id_or_None) -> id` hands it to everybody (by
    default through torch.distributed's object broadcast, i.e. over the host side of the process group)."""

    def __init__(self, rank: int, world: int, *, timeout_ms: int = 10000, share_id: Callable | None = None):
        import ctypes as C
        from . import _lib
        self._lib, self._C = _lib, C
        self.rank, self.world, self.timeout_ms = rank, world, timeout_ms
        l = _lib.lib()
        ident = None
        if rank == 0:
            buf = C.create_string_buffer(_lib.MGPU_ID_BYTES)
            _lib.check(l.sca_mgpu_unique_id(buf))
            ident = bytes(buf.raw)
        if share_id is None:
            import torch.distributed as dist
            box = [ident]
            dist.broadcast_object_list(box, src=0)
            ident = box[0]
        else:
            ident = share_id(ident)
        handle = C.c_void_p()
        _lib.check(l.sca_mgpu_init(ident, rank, world, timeout_ms, C.byref(handle)))
        self._comm = handle

    def allgather_triples(self, mine, *, stream=None, timeout_ms: int | None = None):
        """mine fp32 [rows, width] on the device -> [world, rows, width], rank-major. timeout_ms <= 0: enqueue only."""
        import torch
        from . import ops
        rows, width = mine.shape
        out = torch.empty((self.world, rows, width), dtype=torch.float32, device=mine.device)
        limit = self.timeout_ms if timeout_ms is None else timeout_ms
        self._lib.check(self._lib.lib().sca_mgpu_allgather_triples(self._comm, mine.contiguous().data_ptr(), out.data_ptr(),
                                                                   rows * width, ops._stream_ptr(stream), limit))
        return out

    def abort(self):
        self._lib.check(self._lib.lib().sca_mgpu_abort(self._comm))

    def close(self):
        if self._comm is not None:
            self._lib.check(self._lib.lib().sca_mgpu_destroy(self._comm))
            self._comm = None


def sequence_split_decode(q, k_shard, v_shard, *, group=None, scale=None, num_splits: int = 0,
                          triples_fn: Callable | None = None, merge_fn: Callable | None = None,
                          empty_triples_fn: Callable | None = None, comm: "MgpuComm | None" = None):
    """Decode attention with the KV sequence sharded over the ranks of `group`.

    q [B, H_q, 1, D] is replicated; k_shard / v_shard [B, H_kv, S_local, D] hold this rank's token range
    (S_local may be 0). Returns the normalised output [B * H_q, D] on every rank. The triples travel through `comm`
    (the library's bounded NCCL communicator, MgpuComm) when one is given, else through torch.distributed.
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
    if comm is not None:
        # the library's own communicator: enqueue only (the merge kernel follows on the same stream)
        gathered = comm.allgather_triples(mine, timeout_ms=0) if comm.world > 1 else mine.unsqueeze(0)
    elif world == 1:
        gathered = mine.unsqueeze(0)
    else:
        rows, width = mine.shape
        flat = torch.empty((world * rows, width), dtype=mine.dtype, device=mine.device)  # rank-major concatenation
        dist.all_gather_into_tensor(flat, mine.contiguous(), group=group)
        gathered = flat.view(world, rows, width)
    return merge_fn(gathered)


def shard_sizes(total: int, world: int) -> Sequence[int]:
    return [kv_range_for_rank(total, r, world)[1] - kv_range_for_rank(total, r, world)[0] for r in range(world)]


class PeerExchange:
    """Sequence-split decode whose cross-GPU step is one kernel over peer memory.

    Collective constructor: every rank of `group` builds it with the same (rows = B * H_q, head_dim).
    It allocates this rank's exchange buffer, all-gathers the 64-byte IPC handles (host side, once) and
    maps the peers' buffers. `decode` then costs two launches: the split-K partial kernel on this rank's
    KV shard and the fused merge / exchange / merge kernel. One process per GPU is required.
    """

    def __init__(self, rows: int, head_dim: int, device, group=None):
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import _lib
        self._lib = _lib
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > _lib.PEER_MAX_RANKS:
            raise ValueError(f"at most {_lib.PEER_MAX_RANKS} ranks")
        self.rows, self.head_dim, self.device = rows, head_dim, torch.device(device)
        l = _lib.lib()
        nbytes = l.sca_peer_buffer_bytes(self.world, rows, head_dim)
        if nbytes < 0:
            raise ValueError("invalid exchange geometry")
        with torch.cuda.device(self.device):
            own = C.c_void_p()
            handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
            _lib.check(l.sca_peer_buffer_create(nbytes, C.byref(own), handle))
            self._own = own.value
            mine = torch.tensor(list(handle.raw), dtype=torch.uint8, device=self.device)
            everyone = torch.empty((self.world, _lib.PEER_HANDLE_BYTES), dtype=torch.uint8, device=self.device)
            dist.all_gather_into_tensor(everyone.view(-1), mine, group=group)
            handles = everyone.cpu().numpy()
            self._peers = []
            for r in range(self.world):
                if r == self.rank:
                    self._peers.append(self._own)
                    continue
                ptr = C.c_void_p()
                _lib.check(l.sca_peer_buffer_open(bytes(handles[r].tobytes()), C.byref(ptr)))
                self._peers.append(ptr.value)
            torch.cuda.synchronize(self.device)
        dist.barrier(group=group)  # every buffer is zeroed and mapped before the first kernel stores into it

    def decode(self, q, k_shard, v_shard, *, scale=None, num_splits: int = 0, stream=None):
        """q [B, H_q, 1, D] replicated, k_shard / v_shard [B, H_kv, S_local, D] (S_local may be 0).
        Returns the normalised output [B * H_q, D] on every rank."""
        import ctypes as C
        import torch
        from . import ops
        _lib = self._lib
        b, hq, _, d = q.shape
        if b * hq != self.rows or d != self.head_dim:
            raise ValueError("geometry differs from the one the exchange was built for")
        if k_shard.shape[2] > 0:
            pm, pl, po, splits = ops.decode_partials(q, k_shard, v_shard, scale=scale, num_splits=num_splits,
                                                     stream=stream)
        else:
            # a rank without tokens contributes m = -inf, l = 0, O = 0 and is skipped by the merge
            splits = 1
            ws = torch.zeros(self.rows * (2 + d), dtype=torch.float32, device=q.device)
            ws[: self.rows] = float("-inf")
            pm, pl, po = ws[: self.rows], ws[self.rows: 2 * self.rows], ws[2 * self.rows:]
        out = torch.empty((self.rows, d), dtype=q.dtype, device=q.device)
        x = _lib.SeqSplitExchange()
        for r, ptr in enumerate(self._peers):
            x.peer_buffers[r] = ptr
        x.rank, x.world = self.rank, self.world
        x.rows, x.head_dim, x.num_splits = self.rows, d, splits
        x.epoch = 0  # the kernel counts the steps in the buffer: identical parameters every step (graph replay)
        x.partial_m, x.partial_l, x.partial_o = pm.data_ptr(), pl.data_ptr(), po.data_ptr()
        x.out, x.out_dtype = out.data_ptr(), ops.dtype_id(q.dtype)
        _lib.check(_lib.lib().sca_launch_seqsplit_exchange(C.byref(x), ops._stream_ptr(stream)))
        return out

    def capture(self, q, k_shard, v_shard, *, scale=None, num_splits: int = 0):
        """Captures one decode step over these (static) tensors - partial kernel + exchange kernel - in a CUDA
        graph. Collective in effect: every rank must capture and later replay the same number of times.
        Returns (graph, out); `graph.replay()` recomputes `out` from the current contents of q / k_shard / v_shard."""
        import torch
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up outside the capture: scratch pool, kernel attributes
                self.decode(q, k_shard, v_shard, scale=scale, num_splits=num_splits, stream=side)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                out = self.decode(q, k_shard, v_shard, scale=scale, num_splits=num_splits, stream=side)
        torch.cuda.current_stream(self.device).wait_stream(side)
        return graph, out

    def status(self) -> int:
        """0, or the step (from 1) of the first launch that gave up waiting for a peer; that launch wrote NaN instead
        of a result. Synchronises the device. Call it at the cadence results are consumed - after every step when
        each output is used at once, after a batch of graph replays otherwise."""
        import ctypes as C
        value = C.c_int32(0)
        self._lib.check(self._lib.lib().sca_peer_exchange_status(self._own, C.byref(value)))
        return int(value.value)

    def check(self) -> None:
        """Raises when a step since the last check gave up waiting for a peer, and clears the record."""
        step = self.status()
        if step != 0:
            self._lib.check(self._lib.lib().sca_peer_exchange_clear(self._own))
            raise self._lib.ScaError(500, f"sequence-split exchange: step {step} gave up waiting for a peer; its output is NaN")

    def close(self):
        """Collective: unmaps the peers' buffers, then frees the own one."""
        import torch
        import torch.distributed as dist
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        l = self._lib.lib()
        for r, ptr in enumerate(self._peers):
            if r != self.rank:
                self._lib.check(l.sca_peer_buffer_close(ptr))
        dist.barrier(group=self.group)  # nobody still maps the buffer that is about to be freed
        self._lib.check(l.sca_peer_buffer_destroy(self._own))
        self._own, self._peers = None, []
