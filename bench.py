#!/usr/bin/env python
"""Benchmark of the attention hot path on B200: one JSON line on stdout.

  python bench.py [--gpus N] [--steps K] [--warmup W]      # headline + every other workload ("secondary")
  python bench.py --workload decode|paged|longctx|flash|kvfill ...   # that workload alone (profiling)
  python bench.py --impl reference ...                      # the reference's CPU path on the host cores

A "step" is one pass of the hot path over one batch of seeded synthetic input that is already resident in
HBM. A measurement is `repeats` blocks of K steps; every block is bracketed by barrier + synchronize on both
sides and timed with CUDA events on the launching stream; with N > 1 ranks (one process per GPU, torchrun)
the slowest rank's time counts for every block; `value` is the median block, min and max are reported beside it.

The top-level line is the headline: causal flash prefill of the Qwen3-4B layer shape, every GPU on its own
independent batch ("weak"). `secondary` carries the rest of the metric, each entry with its own roofline,
clocks and end-to-end number:
  flash    the same prefill in fp16 and at head dims 64 / 256                      -> TFLOP/s
  decode   split-K decode, B = 128, S_kv = 4096, bf16                               -> GB/s over K, V, Q, O
  paged    256 sequences, lengths U[512, 8192], 16-token pages, 160k-block pool with a shuffled free
           list; one token appended per sequence, then attended                     -> GB/s over the KV read
  longctx  B = 8, S_kv = 131072 (and D = 64 / 256 at 32768) with the KV SEQUENCE split over the ranks
           ("strong"); the (m, l, O) triples cross NVLink inside one kernel over peer-mapped buffers, and
           through one NCCL all-gather for comparison                               -> GB/s over the whole K/V
  kvfill   prefill-sized append, block reset and block gather of the KV pool        -> GB/s
At N > 1 the batched configurations are ALSO run divided over the ranks as the layer shape shards naturally -
(batch x kv head) units for prefill, sequences for decode / paged decode, rank g of G owning units g, g + G, ... -
and reported as "<name>_strong" entries with "scaling": "strong" (total work fixed, no data-path collective).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D = 32, 8, 128
NOMINAL_HBM_GBS = 8000.0
NOMINAL_TENSOR_TFLOPS = 2250.0
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TENSOR_TFLOPS = 1590.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            j = json.load(f)
        return {"hbm_gbs": float(j["hbm_gbs"]), "tflops": float(j["bf16_tflops"]),
                "tflops_sustained": float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": FALLBACK_HBM_GBS, "tflops": FALLBACK_TENSOR_TFLOPS,
                "tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------------------
# clocks during the timed region (read-only NVML queries)
# --------------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int, period_s: float = 0.001):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
                 "hw_thermal_slowdown": 0x40, "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# --------------------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------------------
class Workload:
    """setup() builds this rank's device tensors, step() runs the hot path once, work_per_step() is the algorithmic
    work of the WHOLE job per step when scaling == "strong" and of one rank otherwise."""
    name = ""
    metric = ""
    unit = ""
    bound = ""
    scaling = "weak"
    dtype_name = "bf16"
    launches_per_step = 0
    default_steps = 20
    traffic_bytes = None
    has_e2e = True
    h2d = d2h = 0

    def setup(self, torch, device, seed, rank, world): ...
    def step(self): ...
    def work_per_step(self): ...
    def config(self): ...
    def e2e_setup(self, torch): ...
    def e2e_step(self): ...
    def cpu_sample(self, threads, impl): return None
    def teardown(self): ...

    def traffic(self):
        return self.traffic_bytes


L2_BYTES = 126e6


def replicas_for(bytes_per_step):
    """How many copies of a step's inputs to rotate through so that consecutive steps never find their data in L2:
    1 when one step already moves more than twice the L2, otherwise enough copies to cover 400 MB."""
    if bytes_per_step >= 2 * L2_BYTES:
        return 1
    return int(-(-400e6 // max(bytes_per_step, 1.0)))


def _units(n, rank, world, strong):
    from scicompute_attention_b200 import multi_gpu
    return multi_gpu.units_for_rank(n, rank, world) if strong else list(range(n))


class FlashWorkload(Workload):
    metric, unit, bound = "flash_prefill_throughput", "TFLOP/s", "tensor"
    launches_per_step = 1
    default_steps = 20

    def __init__(self, dtype_name="bf16", head_dim=128, strong=False, batch=4, seq=4096):
        self.dtype_name, self.d, self.strong, self.B, self.S = dtype_name, head_dim, strong, batch, seq
        self.scaling = "strong" if strong else "weak"
        self.name = f"flash_prefill_causal_B{batch}_S{seq}_Hq{HQ}_Hkv{HKV}_D{head_dim}_{dtype_name}" + ("_strong" if strong else "")
        # dram__bytes_read + dram__bytes_write of flash_fwd_sm100_kernel, ncu capture at B=1 scaled x4
        # (profiles/flash_prefill_c2.md, _d64.md, _d256.md); the output mostly stays in L2 until after the kernel
        captured = {128: 50.43e6 + 3.60e6, 64: 25.22e6 + 0.01e6, 256: 102.76e6 + 27.78e6}  # read + written at B=1
        self.traffic_bytes = captured[head_dim] * batch if not strong else None

    def setup(self, torch, device, seed, rank, world):
        from scicompute_attention_b200 import ops
        self.torch, self.ops = torch, ops
        g = torch.Generator(device=device).manual_seed(seed)
        dt = torch.float16 if self.dtype_name == "fp16" else torch.bfloat16
        # independent units of a GQA prefill: (batch, kv head) with the `group` query heads that read it; the strong
        # variant deals them round-robin to the ranks and runs a rank's share as one batch of single-kv-head problems
        units = _units(self.B * HKV, rank, world, self.strong)
        self.world = world
        self.group = HQ // HKV
        if self.strong:
            self.shape_q, self.shape_kv = (len(units), self.group, self.S, self.d), (len(units), 1, self.S, self.d)
        else:
            self.shape_q, self.shape_kv = (self.B, HQ, self.S, self.d), (self.B, HKV, self.S, self.d)
        nq, nkv = 1, 1
        for n in self.shape_q:
            nq *= n
        for n in self.shape_kv:
            nkv *= n
        self.sets = []
        for _ in range(replicas_for((2 * nq + 2 * nkv) * 2)):  # a rank's share may fit into L2: rotate copies
            q = torch.randn(self.shape_q, generator=g, device=device, dtype=torch.float32).to(dt)
            k = torch.randn(self.shape_kv, generator=g, device=device, dtype=torch.float32).to(dt)
            v = torch.randn(self.shape_kv, generator=g, device=device, dtype=torch.float32).to(dt)
            self.sets.append((q, k, v, torch.empty_like(q)))
        self.q, self.k, self.v, self.out = self.sets[0]
        self.turn = 0

    def step(self):
        q, k, v, out = self.sets[self.turn]
        self.turn = (self.turn + 1) % len(self.sets)
        if q.shape[0] > 0:
            self.ops.flash_attention(q, k, v, causal=True, out=out)

    def work_per_step(self):
        return 4 * self.B * HQ * self.d * (self.S * (self.S + 1) // 2)

    def config(self):
        copies = len(getattr(self, "sets", [None]))
        moved = (2 * self.B * HQ + 2 * self.B * HKV) * self.S * self.d * 2 / (getattr(self, "world", 1) if self.strong else 1)
        return {"workload": self.name, "batch": self.B, "seq_len": self.S, "heads_q": HQ, "heads_kv": HKV,
                "head_dim": self.d, "causal": True,
                "l2_policy": ("%d copies of a rank's share (%.0f MB each) used in rotation: larger than L2 together" % (copies, moved / 1e6))
                if copies > 1 else "inputs + output (%.0f MB per GPU and step) larger than L2" % (moved / 1e6),
                "sharding": "(batch, kv head) units dealt round-robin to the ranks, no collective" if self.strong
                else "every GPU runs the whole configuration on its own inputs, no collective"}

    def e2e_setup(self, torch):
        self.hq = self.q.cpu().pin_memory()
        self.hk = self.k.cpu().pin_memory()
        self.hv = self.v.cpu().pin_memory()
        self.ho = torch.empty(self.q.shape, dtype=self.q.dtype).pin_memory()
        self.h2d = (self.hq.numel() + self.hk.numel() + self.hv.numel()) * 2
        self.d2h = self.ho.numel() * 2
        # pieces of the pipeline: (batch element, slice of its kv heads with the query heads that read them);
        # every piece is one contiguous block of each tensor
        hkv = self.k.shape[1]
        per = max(1, hkv // max(1, min(self.e2e_chunks, hkv)))
        self.e2e_pieces = [(b, h0, min(hkv, h0 + per)) for b in range(self.q.shape[0]) for h0 in range(0, hkv, per)]
        self.e2e_streams = [torch.cuda.Stream() for _ in range(min(8, len(self.e2e_pieces)))]

    e2e_chunks = 2  # kv-head slices per batch element in the host-copy pipeline

    def e2e_step(self):
        # one stream per piece (round-robin): the upload of piece i + 1 overlaps the kernel and the download of
        # piece i (the two copy directions are separate engines); small pieces keep the last download, which
        # nothing overlaps, short. The launching stream joins all of them at the end, so the events around the
        # timed region see the whole step
        torch = self.torch
        cur = torch.cuda.current_stream()
        g = self.q.shape[1] // self.k.shape[1]
        for side in self.e2e_streams:
            side.wait_stream(cur)
        for i, (b, h0, h1) in enumerate(self.e2e_pieces):
            side = self.e2e_streams[i % len(self.e2e_streams)]
            with torch.cuda.stream(side):
                q, o = self.q[b:b + 1, h0 * g:h1 * g], self.out[b:b + 1, h0 * g:h1 * g]
                k, v = self.k[b:b + 1, h0:h1], self.v[b:b + 1, h0:h1]
                q.copy_(self.hq[b:b + 1, h0 * g:h1 * g], non_blocking=True)
                k.copy_(self.hk[b:b + 1, h0:h1], non_blocking=True)
                v.copy_(self.hv[b:b + 1, h0:h1], non_blocking=True)
                self.ops.flash_attention(q, k, v, causal=True, out=o, stream=side)
                self.ho[b:b + 1, h0 * g:h1 * g].copy_(o, non_blocking=True)
        for side in self.e2e_streams:
            cur.wait_stream(side)

    def cpu_sample(self, threads, impl):
        # bounded sample: one (batch 0, head) pair per host thread; the main arm's CPU leg takes whole
        # causal heads (all rows), one step of the reference arm the last 256 query rows (row i attends to
        # i + 1 keys); FLOPs are counted for the sampled rows only
        import numpy as np
        skv = self.q.shape[2]
        sq = skv if impl == "port" else min(256, skv)
        hq_have, hkv_have = self.q.shape[1], self.k.shape[1]
        nh = max(1, min(hq_have, threads))
        q = self.q[:1, :nh, skv - sq:skv].float().cpu().numpy()
        k = self.k[:1, :, :skv].float().cpu().numpy()
        v = self.v[:1, :, :skv].float().cpu().numpy()
        k = np.repeat(k, hq_have // hkv_have, axis=1)[:, :nh]
        v = np.repeat(v, hq_have // hkv_have, axis=1)[:, :nh]
        secs, kind = run_cpu_attention(q, np.ascontiguousarray(k), np.ascontiguousarray(v), True, threads, impl)
        flops = 4 * nh * self.d * sum(skv - sq + i + 1 for i in range(sq))
        return flops, secs, f"{nh} heads x last {sq} query rows of a {skv}-token causal prefix", kind


class DecodeWorkload(Workload):
    metric, unit, bound = "decode_kv_bandwidth", "GB/s", "hbm"
    launches_per_step = 2  # partial + merge
    default_steps = 50

    def __init__(self, strong=False, batch=128, seq=4096):
        self.strong, self.B, self.SKV = strong, batch, seq
        self.scaling = "strong" if strong else "weak"
        self.name = f"splitk_decode_B{batch}_Skv{seq}_Hq{HQ}_Hkv{HKV}_D{D}_bf16" + ("_strong" if strong else "")
        # dram__bytes_read + dram__bytes_write of decode_partial_kernel, ncu capture at B=16 scaled by the batch
        # (profiles/decode_splitk_c3.md); traffic grows in proportion to the batch
        self.traffic_bytes = (268.71e6 + 3.96e6) * batch / 16 if not strong else None

    def setup(self, torch, device, seed, rank, world):
        from scicompute_attention_b200 import ops
        self.torch, self.ops = torch, ops
        nb = len(_units(self.B, rank, world, self.strong))
        g = torch.Generator(device=device).manual_seed(seed)
        self.sets = []
        for _ in range(replicas_for(2 * nb * HKV * self.SKV * D * 2)):
            q = torch.randn((nb, HQ, 1, D), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
            k = torch.randn((nb, HKV, self.SKV, D), generator=g, device=device, dtype=torch.bfloat16)
            v = torch.randn((nb, HKV, self.SKV, D), generator=g, device=device, dtype=torch.bfloat16)
            self.sets.append((q, k, v))
        self.q, self.k, self.v = self.sets[0]
        self.turn = 0
        self.out = None

    def step(self):
        q, k, v = self.sets[self.turn]
        self.turn = (self.turn + 1) % len(self.sets)
        if q.shape[0] > 0:
            self.out = self.ops.decode_attention(q, k, v)

    def work_per_step(self):
        return 2 * self.B * HKV * self.SKV * D * 2 + 2 * self.B * HQ * D * 2

    def config(self):
        mine = 2 * self.k.numel() * 2
        copies = len(getattr(self, "sets", [None]))
        return {"workload": self.name, "batch": self.B, "seq_kv": self.SKV, "heads_q": HQ, "heads_kv": HKV,
                "head_dim": D, "l2_policy": "inputs larger than L2 (%d x %.0f MB per GPU, used in rotation)" % (copies, mine / 1e6),
                "sharding": "sequences dealt round-robin to the ranks, no collective" if self.strong
                else "every GPU runs the whole batch on its own sequences, no collective"}

    def e2e_setup(self, torch):
        self.hq = self.q.cpu().pin_memory()
        self.hk = self.k.cpu().pin_memory()
        self.hv = self.v.cpu().pin_memory()
        self.ho = torch.empty((self.q.shape[0], HQ, 1, D), dtype=torch.bfloat16).pin_memory()
        self.h2d = self.hq.numel() * 2 + self.hk.numel() * 2 + self.hv.numel() * 2
        self.d2h = self.ho.numel() * 2

    def e2e_step(self):
        self.q.copy_(self.hq, non_blocking=True)
        self.k.copy_(self.hk, non_blocking=True)
        self.v.copy_(self.hv, non_blocking=True)
        out = self.ops.decode_attention(self.q, self.k, self.v)
        self.ho.copy_(out, non_blocking=True)

    def cpu_sample(self, threads, impl):
        # CPU leg of the main arm: the whole batch (a second or two of FP64 work on all host threads);
        # one step of the reference arm: eight sequences per host thread of the reference's own routine
        nb = self.q.shape[0] if impl == "port" else max(1, min(self.q.shape[0], 8 * threads))
        q = self.q[:nb].float().cpu().numpy()
        k = self.k[:nb].float().cpu().numpy()
        v = self.v[:nb].float().cpu().numpy()
        secs, kind = run_cpu_attention(q, k, v, True, threads, impl)
        work = 2 * nb * HKV * self.SKV * D * 2 + 2 * nb * HQ * D * 2
        return work, secs, f"{nb} of {self.B} sequences, all heads, full S_kv={self.SKV}", kind


class PagedWorkload(Workload):
    metric, unit, bound = "paged_decode_kv_bandwidth", "GB/s", "hbm"
    launches_per_step = 3  # batched append + partial + merge
    default_steps = 30
    # ncu capture of the paged decode_partial_kernel on 32 sequences: 602.5 MB moved for 597.7 MB of K/V
    # (profiles/paged_decode_c4.md); scaled by the tokens of the full batch
    traffic_ratio = (598.31e6 + 4.20e6) / 597.75e6

    def __init__(self, strong=False, nseq=256, nblk=160000):
        self.strong, self.NSEQ, self.NBLK, self.BS = strong, nseq, nblk, 16
        self.scaling = "strong" if strong else "weak"
        self.name = (f"paged_decode_{nseq}seq_len512-8192_bs16_pool{nblk // 1000}k_Hq{HQ}_Hkv{HKV}_D{D}_bf16"
                     + ("_strong" if strong else ""))

    def setup(self, torch, device, seed, rank, world):
        import numpy as np
        from scicompute_attention_b200 import ops
        self.torch, self.ops, self.np = torch, ops, np
        # the whole job's lengths come from one seed; the strong variant gives rank g sequences g, g + G, ... and a
        # pool of its own of 1/G of the blocks (every rank owns allocator, table and pool, as the sharding says)
        rng = np.random.default_rng(seed if not self.strong else 12345)
        all_lens = rng.integers(512, 8193, size=self.NSEQ).astype(np.int64)
        mine = _units(self.NSEQ, rank, world, self.strong)
        self.all_lens = all_lens
        self.lens = all_lens[mine]
        nseq = len(mine)
        nblk = self.NBLK // world if self.strong else self.NBLK
        self.nblk = nblk
        # LIFO allocator with a seeded shuffle of its free list -> non-contiguous page tables. The
        # allocation order is the reference's: allocate everything, shuffle, free in that order, then
        # every allocation pops from the back (src/kv_cache/block_manager.cpp:25-27,60-62).
        ids = np.arange(nblk, dtype=np.int32)
        np.random.default_rng(seed + 1).shuffle(ids)
        free = list(ids)
        max_blocks = nblk  # table row length = pool size (src/kv_cache/paged_kv_cache.cpp:22-27)
        table = np.full((max(nseq, 1), max_blocks), -1, dtype=np.int32)
        for s in range(nseq):
            need = -(-(int(self.lens[s]) + 1) // self.BS)
            for j in range(need):
                table[s, j] = free.pop()
        self.table_host = table
        self.page_table = torch.from_numpy(table).to(device)
        self.seq_lens = torch.from_numpy((self.lens + 1).astype(np.int32)).to(device)  # includes the new token
        g = torch.Generator(device=device).manual_seed(seed)
        shape = (nblk, self.BS, HKV, D)
        self.k_pool = torch.randn(shape, generator=g, device=device, dtype=torch.bfloat16)
        self.v_pool = torch.randn(shape, generator=g, device=device, dtype=torch.bfloat16)
        self.q = torch.randn((nseq, HQ, 1, D), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        self.k_new = torch.randn((nseq, HKV, D), generator=g, device=device, dtype=torch.bfloat16)
        self.v_new = torch.randn((nseq, HKV, D), generator=g, device=device, dtype=torch.bfloat16)
        self.mean_len = int(self.lens.mean()) + 1 if nseq else 1
        self.longest = int(self.lens.max()) + 1 if nseq else 1

    def step(self):
        if self.q.shape[0] == 0:
            return
        self.ops.kv_append_batched(self.k_pool, self.v_pool, self.k_new, self.v_new, self.page_table, self.seq_lens)
        self.out = self.ops.paged_attention(self.q, self.k_pool, self.v_pool, self.page_table, self.seq_lens,
                                            block_size=self.BS, typical_len=self.mean_len, longest_len=self.longest)

    def _bytes(self, lens):
        toks = int((lens + 1).sum())
        pages = int(sum(-(-(int(n) + 1) // self.BS) for n in lens))
        return toks * (2 * HKV * D * 2) + 2 * len(lens) * HQ * D * 2 + pages * 4 + len(lens) * 4

    def work_per_step(self):
        return self._bytes(self.all_lens if self.strong else self.lens)

    def traffic(self):
        return None if self.strong else float((self.lens + 1).sum()) * 2 * HKV * D * 2 * self.traffic_ratio

    def config(self):
        return {"workload": self.name, "num_seqs": self.NSEQ, "block_size": self.BS, "pool_blocks": self.NBLK,
                "tokens_attended": int(((self.all_lens if self.strong else self.lens) + 1).sum()), "heads_q": HQ,
                "heads_kv": HKV, "head_dim": D,
                "l2_policy": "inputs larger than L2 (%.0f MB of KV read per GPU and step)" % (float((self.lens + 1).sum()) * 4096 / 1e6),
                "sharding": "sequences dealt round-robin to the ranks, every rank with its own pool and page table, no collective"
                if self.strong else "every GPU runs the whole batch on its own pool, no collective"}

    def e2e_setup(self, torch):
        # what a serving loop moves per step: the new tokens' q/k/v up, the attention output down;
        # the KV pool and page table live on the device across steps
        self.hq = self.q.cpu().pin_memory()
        self.hkn = self.k_new.cpu().pin_memory()
        self.hvn = self.v_new.cpu().pin_memory()
        self.ho = torch.empty((self.q.shape[0], HQ, 1, D), dtype=torch.bfloat16).pin_memory()
        self.h2d = (self.hq.numel() + self.hkn.numel() + self.hvn.numel()) * 2
        self.d2h = self.ho.numel() * 2

    def e2e_step(self):
        self.q.copy_(self.hq, non_blocking=True)
        self.k_new.copy_(self.hkn, non_blocking=True)
        self.v_new.copy_(self.hvn, non_blocking=True)
        self.step()
        self.ho.copy_(self.out, non_blocking=True)

    def cpu_sample(self, threads, impl):
        np, torch = self.np, self.torch
        # bounded sample: the first sequences, gathered into contiguous K/V (64 for the main arm's CPU leg,
        # two per host thread for one step of the reference arm)
        ns = max(1, min(self.q.shape[0], 64 if impl == "port" else 2 * threads))
        work = 0
        qs, ks, vs = [], [], []
        for s in range(ns):
            n = int(self.lens[s]) + 1
            pages = torch.from_numpy(self.table_host[s, : -(-n // self.BS)].astype(np.int64)).to(self.k_pool.device)
            k = self.k_pool[pages].reshape(-1, HKV, D)[:n].permute(1, 0, 2).float().cpu().numpy()[None]
            v = self.v_pool[pages].reshape(-1, HKV, D)[:n].permute(1, 0, 2).float().cpu().numpy()[None]
            qs.append(self.q[s:s + 1].float().cpu().numpy())
            ks.append(k)
            vs.append(v)
            work += n * (2 * HKV * D * 2) + 2 * HQ * D * 2
        t0 = time.perf_counter()
        kind = None
        for q, k, v in zip(qs, ks, vs):
            _, kind = run_cpu_attention(q, k, v, True, threads, impl)
        secs = time.perf_counter() - t0
        return work, secs, f"{ns} of {self.NSEQ} sequences (gathered to contiguous K/V), all heads", kind


class LongContextWorkload(Workload):
    """Sequence-split decode: the KV axis is cut into one contiguous slice per rank, every rank reduces its slice to
    (m, l, O) triples, B*H_q*(2+D) floats per rank travel to every peer (stored by the merge kernel into peer-mapped
    buffers, or by one NCCL all-gather), and every rank merges. Total work is fixed: this workload scales "strong"."""
    metric, unit, bound = "longctx_decode_kv_bandwidth", "GB/s", "hbm"
    scaling = "strong"
    default_steps = 300
    B = 8

    def __init__(self, head_dim=128, seq=131072, exchange="peer"):
        self.d, self.SKV, self.exchange = head_dim, seq, exchange
        self.name = f"seqsplit_decode_B8_Skv{seq}_Hq{HQ}_Hkv{HKV}_D{head_dim}_bf16"

    def setup(self, torch, device, seed, rank, world):
        from scicompute_attention_b200 import multi_gpu, ops
        self.torch, self.ops, self.mg = torch, ops, multi_gpu
        self.rank, self.world = rank, world
        if world > 1:
            self.name += "_" + self.exchange
        lo, hi = multi_gpu.kv_range_for_rank(self.SKV, rank, world)
        g = torch.Generator(device=device).manual_seed(1234)  # q is replicated: same seed on every rank
        self.q = torch.randn((self.B, HQ, 1, self.d), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        g2 = torch.Generator(device=device).manual_seed(seed + 77)
        self.sets = []
        for _ in range(replicas_for(2 * self.B * HKV * (hi - lo) * self.d * 2)):  # a small share would sit in L2
            k = torch.randn((self.B, HKV, hi - lo, self.d), generator=g2, device=device, dtype=torch.bfloat16)
            v = torch.randn((self.B, HKV, hi - lo, self.d), generator=g2, device=device, dtype=torch.bfloat16)
            self.sets.append((k, v))
        self.k, self.v = self.sets[0]
        self.turn = 0
        self.px = None
        self.launches_per_step = 2  # partial kernel + merge (1 GPU) / fused merge-exchange-merge kernel
        if world > 1 and self.exchange == "peer":
            self.px = multi_gpu.PeerExchange(self.B * HQ, self.d, device)
            # the whole step (partial kernel + exchange kernel) is one captured graph per K/V copy, replayed in turn
            self.graphs = [self.px.capture(self.q, k, v) for k, v in self.sets]
        elif world > 1:
            self.launches_per_step = 3  # partial, merge to triples, merge over ranks (+ the NCCL all-gather)
            self.comm = multi_gpu.MgpuComm(rank, world)  # the library's own bounded communicator (sca_mgpu_*)

    def step(self):
        k, v = self.sets[self.turn]
        if self.px is not None:
            graph, self.out = self.graphs[self.turn]
            graph.replay()
        elif self.world > 1:
            self.out = self.mg.sequence_split_decode(self.q, k, v, comm=self.comm)
        else:
            self.out = self.ops.decode_attention(self.q, k, v)
        self.turn = (self.turn + 1) % len(self.sets)

    def work_per_step(self):
        # whole job: all ranks together read the full K and V once
        return 2 * self.B * HKV * self.SKV * self.d * 2 + 2 * self.B * HQ * self.d * 2

    def config(self):
        mine = 2 * self.k.numel() * 2
        copies = len(getattr(self, "sets", [None]))
        return {"workload": self.name, "batch": self.B, "seq_kv": self.SKV, "heads_q": HQ, "heads_kv": HKV,
                "head_dim": self.d, "l2_policy": "inputs larger than L2 (%d x %.0f MB per GPU, used in rotation)" % (copies, mine / 1e6),
                "sharding": "KV sequence split across ranks; (m, l, O) triples exchanged " +
                            ("by peer stores inside the merge kernel (captured graph)" if self.px is not None else
                             "by one NCCL all-gather per step (sca_mgpu communicator)" if self.world > 1 else "locally (one rank)")}

    def e2e_setup(self, torch):
        self.hq = self.q.cpu().pin_memory()
        self.ho = torch.empty((self.B * HQ, self.d), dtype=torch.bfloat16).pin_memory()
        self.h2d, self.d2h = self.hq.numel() * 2, self.ho.numel() * 2

    def e2e_step(self):
        # a decode step moves the new query up and the attention output down; the KV cache lives on the devices
        self.q.copy_(self.hq, non_blocking=True)
        self.step()
        self.ho.copy_(self.out.reshape(self.B * HQ, self.d), non_blocking=True)

    def cpu_sample(self, threads, impl):
        nb = 1
        skv = min(16384, self.k.shape[2])
        q = self.q[:nb].float().cpu().numpy()
        k = self.k[:nb, :, :skv].float().cpu().numpy()
        v = self.v[:nb, :, :skv].float().cpu().numpy()
        secs, kind = run_cpu_attention(q, k, v, True, threads, impl)
        work = 2 * nb * HKV * k.shape[2] * self.d * 2 + 2 * nb * HQ * self.d * 2
        return work, secs, f"{nb} of {self.B} sequences, first {k.shape[2]} of {self.SKV} keys, all heads", kind

    def teardown(self):
        if self.px is not None:
            self.graphs = None
            self.px.check()  # raises if some step gave up waiting for a peer
            self.px.close()
            self.px = None
        if getattr(self, "comm", None) is not None:
            self.comm.close()
            self.comm = None


class KvWorkload(Workload):
    """The KV-cache data movement kernels at prefill size: `append` scatters the tokens of a ragged batch
    (lengths U[512, 8192], 256 sequences: about 1.1 M tokens x 4096 B) into a shuffled 160k-block pool, `reset`
    zeroes 10 000 blocks of K and V, `gather` copies 10 000 blocks into a contiguous buffer."""
    unit, bound = "GB/s", "hbm"
    launches_per_step = 1
    default_steps = 10
    has_e2e = False  # these kernels move data that lives on the device on both sides: nothing to bring from the host
    NSEQ, NBLK, BS, NIDS = 256, 160000, 16, 10000

    def __init__(self, op="append"):
        self.op = op
        self.metric = f"kv_{op}_bandwidth"
        self.name = {"append": "kv_append_prefill_fill_256seq_len512-8192_bs16_pool160k",
                     "reset": "kv_reset_10000_blocks_bs16", "gather": "kv_gather_10000_blocks_bs16"}[op] + f"_Hkv{HKV}_D{D}_bf16"

    def setup(self, torch, device, seed, rank, world):
        import numpy as np
        from scicompute_attention_b200 import ops
        self.torch, self.ops = torch, ops
        rng = np.random.default_rng(seed)
        shape = (self.NBLK, self.BS, HKV, D)
        self.k_pool = torch.zeros(shape, device=device, dtype=torch.bfloat16)
        self.v_pool = torch.zeros(shape, device=device, dtype=torch.bfloat16) if self.op != "gather" else None
        perm = rng.permutation(self.NBLK).astype(np.int32)
        if self.op == "append":
            lens = rng.integers(512, 8193, size=self.NSEQ)
            ntok = int(lens.sum())
            nblocks = int(sum(-(-int(n) // self.BS) for n in lens))
            slots = np.empty(ntok, dtype=np.int32)
            at, blk = 0, 0
            for n in lens:  # token t of a sequence goes to its (t // 16)-th block, blocks taken from the shuffled list
                need = -(-int(n) // self.BS)
                ids = perm[blk:blk + need].astype(np.int64)
                t = np.arange(int(n))
                slots[at:at + int(n)] = (ids[t // self.BS] * self.BS + t % self.BS).astype(np.int32)
                at += int(n)
                blk += need
            assert blk == nblocks
            self.ntok = ntok
            self.slots = torch.from_numpy(slots).to(device)
            g = torch.Generator(device=device).manual_seed(seed)
            self.k_new = torch.randn((ntok, HKV, D), generator=g, device=device, dtype=torch.bfloat16)
            self.v_new = torch.randn((ntok, HKV, D), generator=g, device=device, dtype=torch.bfloat16)
        else:
            self.ids = torch.from_numpy(perm[: self.NIDS].copy()).to(device)
            self.gathered = None

    def step(self):
        if self.op == "append":
            self.ops.kv_append(self.k_pool, self.v_pool, self.k_new, self.v_new, self.slots)
        elif self.op == "reset":
            self.ops.kv_reset(self.k_pool, self.v_pool, self.ids)
        else:
            self.gathered = self.ops.kv_gather(self.k_pool, self.ids)

    def work_per_step(self):
        block = self.BS * HKV * D * 2
        if self.op == "append":   # K and V rows read once and written once, plus the slot list
            return self.ntok * (HKV * D * 2) * 2 * 2 + self.ntok * 4
        if self.op == "reset":    # K and V blocks written
            return self.NIDS * block * 2 + self.NIDS * 4
        return self.NIDS * block * 2 + self.NIDS * 4  # gather: one layer read + written

    def config(self):
        return {"workload": self.name, "pool_blocks": self.NBLK, "block_size": self.BS, "heads_kv": HKV, "head_dim": D,
                "l2_policy": "working set larger than L2 (%.0f MB per step)" % (self.work_per_step() / 1e6),
                "sharding": "every GPU on its own pool, no collective"}

def build_workloads(args, world):
    """(primary, [secondary...]) as factories, in run order."""
    single = {
        "flash": lambda: FlashWorkload(args.dtype, head_dim=args.head_dim),
        "decode": lambda: DecodeWorkload(),
        "paged": lambda: PagedWorkload(),
        "longctx": lambda: LongContextWorkload(exchange=args.exchange),
        "kvfill": lambda: KvWorkload("append"),
    }
    if args.workload != "all":
        return single[args.workload], []
    secondary = [
        lambda: FlashWorkload("fp16"),
        lambda: FlashWorkload("bf16", head_dim=64),
        lambda: FlashWorkload("bf16", head_dim=256),
        lambda: DecodeWorkload(),
        lambda: PagedWorkload(),
        lambda: LongContextWorkload(128, 131072, "peer"),
        lambda: LongContextWorkload(64, 32768, "peer"),
        lambda: LongContextWorkload(256, 32768, "peer"),
        lambda: KvWorkload("append"),
        lambda: KvWorkload("reset"),
        lambda: KvWorkload("gather"),
    ]
    if world > 1:
        secondary[5:5] = [lambda: FlashWorkload("bf16", strong=True), lambda: DecodeWorkload(strong=True),
                          lambda: PagedWorkload(strong=True)]
        secondary.insert(9, lambda: LongContextWorkload(128, 131072, "nccl"))
    return single["flash"], secondary


# --------------------------------------------------------------------------------------------------
# CPU legs (the oracle / the reference's own FP64 routine): checker code, timed only here
# --------------------------------------------------------------------------------------------------
def run_cpu_attention(q, k, v, causal, threads, impl):
    """Times the FP64 host attention on (q, k, v); returns (seconds, kind).
    impl == "reference": the reference's own routine (oracle/_ref), one (batch, head) slice per host
    thread; otherwise the plain-C restatement with OpenMP over (batch, head)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_lib as ol
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    B, H, Sq, Dd = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    if impl == "reference" and ol.have_ref():
        lib = ol.ref()
        group = H // Hkv
        jobs = [(b, h) for b in range(B) for h in range(H)]
        outs = [np.zeros((Sq, Dd)) for _ in jobs]

        def work(i):
            b, h = jobs[i]
            lib.ref_attention(np.ascontiguousarray(q[b, h]).reshape(-1), np.ascontiguousarray(k[b, h // group]).reshape(-1),
                              np.ascontiguousarray(v[b, h // group]).reshape(-1), 1, 1, 1, Sq, Skv, Dd, int(causal),
                              outs[i].reshape(-1))

        from concurrent.futures import ThreadPoolExecutor
        t0 = time.perf_counter()
        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(work, range(len(jobs))))
        return time.perf_counter() - t0, "reference"
    t0 = time.perf_counter()
    ol.attention_f64(q, k, v, causal=causal, threads=threads)
    return time.perf_counter() - t0, "port"


# --------------------------------------------------------------------------------------------------
# measurement
# --------------------------------------------------------------------------------------------------
def _stats(values):
    s = sorted(values)
    return {"n": len(s), "min": s[0], "median": s[len(s) // 2], "max": s[-1]}


def pin_to_gpu_numa_node(torch, local_rank):
    """Pinned host buffers are placed by first touch: run this process on the CPUs of the GPU's NUMA node before it
    allocates them. Returns the node, or None when the platform does not say."""
    try:
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = torch.cuda.get_device_properties(local_rank).pci_domain_id
        dev = torch.cuda.get_device_properties(local_rank).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        node = int(open(path).read().strip())
        if node < 0:
            return None
        cpus = []
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus += list(range(int(lo), int(hi or lo) + 1))
        allowed = sorted(set(cpus) & os.sched_getaffinity(0))
        if allowed:
            os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def measure(wl, args, steps, repeats, ctx, with_cpu):
    """Runs one workload: warm-up, `repeats` timed blocks of `steps` steps, the end-to-end leg, optionally the CPU leg."""
    torch, dist, device = ctx["torch"], ctx["dist"], ctx["device"]
    rank, world, local_rank = ctx["rank"], ctx["world"], ctx["local_rank"]
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    wl.setup(torch, device, args.seed + rank, rank, world)
    for _ in range(args.warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    block_ms = []
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record(stream)
        for _ in range(steps):
            wl.step()
        stop.record(stream)
        barrier()
        block_ms.append(start.elapsed_time(stop))
    clocks = sampler.stop()

    # end to end through the public operator with host buffers: pinned H2D of the step's inputs,
    # the step, D2H of its result - all inside the timed region
    e2e_steps = args.e2e_steps or min(steps, 5)
    e2e_ms = []
    if not args.capture and wl.has_e2e:
        wl.e2e_setup(torch)
        wl.e2e_step()
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record(stream)
            for _ in range(e2e_steps):
                wl.e2e_step()
            e1.record(stream)
            barrier()
            e2e_ms.append(e0.elapsed_time(e1) / e2e_steps)

    if world > 1:
        t = torch.tensor(block_ms + (e2e_ms or [0.0]), device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        vals = [float(x) for x in t]
        block_ms, e2e_ms = vals[:repeats], (vals[repeats:] if e2e_ms else [])
    step_ms = _stats([ms / steps for ms in block_ms])
    strong = wl.scaling == "strong"
    work = wl.work_per_step()
    scale = 1e9 if wl.unit == "GB/s" else 1e12
    total = (1 if strong else world)

    def rate(ms):
        return work / (ms * 1e-3) / scale * total

    value = rate(step_ms["median"])
    per_gpu = value / world
    entry = None
    if rank == 0:
        peaks = measured_peaks()
        peak = peaks["hbm_gbs"] if wl.bound == "hbm" else peaks["tflops"]
        nominal = NOMINAL_HBM_GBS if wl.bound == "hbm" else NOMINAL_TENSOR_TFLOPS
        cpu = None
        if with_cpu and not args.capture:
            got = wl.cpu_sample(ctx["threads"], "port")
            if got is not None:
                cw, cs, desc, kind = got
                cpu = {"value": cw / cs / scale, "unit": wl.unit, "cores": ctx["threads"], "kind": kind,
                       "sample": desc + f" ({cs:.1f} s of FP64 host work)"}
        e2e = None
        if e2e_ms:
            med = sorted(e2e_ms)[len(e2e_ms) // 2]
            e2e = {"value": rate(med), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                   "ms_per_step": med, "steps": e2e_steps, "repeats": len(e2e_ms),
                   "host_copy_gbs_per_rank": ((wl.h2d + wl.d2h) / (med * 1e-3) / 1e9) if (wl.h2d + wl.d2h) else 0.0}
        entry = {
            "workload": wl.name, "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "ms_per_step": step_ms["median"], "scaling": wl.scaling,
            "repeats": {"n": repeats, "value_min": rate(step_ms["max"]), "value_median": value, "value_max": rate(step_ms["min"]),
                        "ms_min": step_ms["min"], "ms_median": step_ms["median"], "ms_max": step_ms["max"],
                        "ms_blocks": [round(ms / steps, 5) for ms in block_ms]},
            "dtype": wl.dtype_name, "config": wl.config(),
            "roofline": {"bound": wl.bound, "achieved": per_gpu, "peak": peak, "unit": wl.unit,
                         "frac": per_gpu / peak, "peak_source": peaks["source"],
                         "frac_of_nominal": per_gpu / nominal, "traffic": wl.traffic(),
                         # the median block of a tensor-bound entry runs after the power cap has engaged (see
                         # repeats.ms_blocks): the library GEMM's figure for that state is given beside the burst one
                         **({"peak_sustained": peaks["tflops_sustained"], "frac_of_sustained": per_gpu / peaks["tflops_sustained"],
                             "frac_best_block": rate(step_ms["min"]) / world / peak} if wl.bound == "tensor" else {}),
                         "traffic_unit": "bytes per launch of the dominant kernel (ncu capture, scaled; see profiles/)"},
            "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": wl.launches_per_step * steps * repeats,
            "clocks": clocks,
        }
    barrier()
    wl.teardown()
    return entry


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=10, help="timed blocks of --steps steps; the median block is reported")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "flash", "decode", "paged", "longctx", "kvfill"])
    ap.add_argument("--no-secondary", action="store_true", help="headline only")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed host-side legs (for runs under a profiler)")
    ap.add_argument("--e2e-steps", type=int, default=0, help="0 = min(steps, 5)")
    ap.add_argument("--e2e-chunks", type=int, default=2,
                    help="prefill host-copy leg: kv-head slices per batch element that travel as separate pieces")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"], help="--workload flash only")
    ap.add_argument("--head-dim", type=int, default=128, choices=[64, 128, 256], help="--workload flash only")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="--workload longctx on more than one GPU: how the triples cross NVLink")
    ap.add_argument("--capture", action="store_true",
                    help="profiler-sized variant of the workload (same kernels, a few hundred MB): flash B=1, "
                         "decode B=16, paged 32 sequences in a 20k-block pool; one block, no e2e and CPU legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    threads = os.cpu_count() or 1

    if args.impl == "reference":
        return reference_arm(args, rank, world, threads)

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    node = pin_to_gpu_numa_node(torch, local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = {"torch": torch, "dist": dist, "device": device, "rank": rank, "world": world, "local_rank": local_rank,
           "threads": threads}

    FlashWorkload.e2e_chunks = max(1, args.e2e_chunks)
    primary_factory, secondary_factories = build_workloads(args, world)
    primary = primary_factory()
    repeats = 1 if args.capture else max(1, args.repeats)
    if args.capture:
        if isinstance(primary, FlashWorkload):
            primary.B = 1
        elif isinstance(primary, DecodeWorkload):
            primary.B = 16
        elif isinstance(primary, PagedWorkload):
            primary.NSEQ, primary.NBLK = 32, 20000
        primary.name += "_capture"
        primary.traffic_bytes = None
    head = measure(primary, args, args.steps, repeats, ctx, with_cpu=not args.no_cpu)
    del primary
    gc.collect()
    torch.cuda.empty_cache()

    secondary = []
    if not args.no_secondary and not args.capture:
        cpu_done = set()
        for make in secondary_factories:
            wl = make()
            # one CPU leg per workload family (the headline already carries the prefill one)
            family = type(wl).__name__
            with_cpu = (family in ("DecodeWorkload", "PagedWorkload", "LongContextWorkload") and family not in cpu_done
                        and not args.no_cpu)
            cpu_done.add(family)
            entry = measure(wl, args, wl.default_steps, repeats, ctx, with_cpu=with_cpu)
            if entry is not None:
                secondary.append(entry)
            del wl
            gc.collect()
            torch.cuda.empty_cache()

    if rank == 0:
        line = {
            "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": head["scaling"],
            "vs_baseline": None, "dtype": head["dtype"],
            "data": "synthetic (seeded iid N(0,1), random page tables)",
            "config": head["config"], "repeats": head["repeats"], "roofline": head["roofline"],
            "cpu_baseline": head["cpu_baseline"], "e2e": head["e2e"],
            "gpu_launches": head["gpu_launches"], "clocks": head["clocks"],
            "host": {"numa_node_of_gpu": node, "threads": threads},
            "secondary": secondary,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def reference_arm(args, rank, world, threads):
    """The reference's own CPU implementation of the path on this host's cores. Under torchrun only
    rank 0 works; every step is a bounded sample of the same workload."""
    if rank != 0:
        return
    import numpy as np
    import torch
    name = "flash" if args.workload == "all" else args.workload
    wl = {"flash": lambda: FlashWorkload(args.dtype, head_dim=args.head_dim), "decode": DecodeWorkload, "paged": PagedWorkload,
          "longctx": lambda: LongContextWorkload(exchange=args.exchange), "kvfill": None}[name]
    if wl is None:
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no CPU implementation of the KV kernels"}), flush=True)
        return
    wl = wl()
    # host tensors with the workload's shapes, reduced to the sample the CPU leg consumes
    g = torch.Generator().manual_seed(args.seed)
    if isinstance(wl, FlashWorkload):
        wl.q = torch.randn((1, HQ, wl.S, wl.d), generator=g).to(torch.bfloat16)
        wl.k = torch.randn((1, HKV, wl.S, wl.d), generator=g).to(torch.bfloat16)
        wl.v = torch.randn((1, HKV, wl.S, wl.d), generator=g).to(torch.bfloat16)
    elif isinstance(wl, LongContextWorkload):
        wl.q = torch.randn((1, HQ, 1, wl.d), generator=g).to(torch.bfloat16)
        wl.k = torch.randn((1, HKV, 16384, wl.d), generator=g).to(torch.bfloat16)
        wl.v = torch.randn((1, HKV, 16384, wl.d), generator=g).to(torch.bfloat16)
        wl.px, wl.world = None, 1
    elif isinstance(wl, DecodeWorkload):
        nb = max(1, min(wl.B, 8 * threads))
        wl.q = torch.randn((nb, HQ, 1, D), generator=g).to(torch.bfloat16)
        wl.k = torch.randn((nb, HKV, wl.SKV, D), generator=g).to(torch.bfloat16)
        wl.v = torch.randn((nb, HKV, wl.SKV, D), generator=g).to(torch.bfloat16)
    else:
        rng = np.random.default_rng(args.seed)
        wl.np, wl.torch = np, torch
        wl.lens = wl.all_lens = rng.integers(512, 8193, size=wl.NSEQ).astype(np.int64)
        ns = max(1, min(wl.NSEQ, 2 * threads))
        need = int(sum(-(-(int(n) + 1) // wl.BS) for n in wl.lens[:ns]))
        wl.k_pool = torch.randn((need, wl.BS, HKV, D), generator=g).to(torch.bfloat16)
        wl.v_pool = torch.randn((need, wl.BS, HKV, D), generator=g).to(torch.bfloat16)
        wl.q = torch.randn((ns, HQ, 1, D), generator=g).to(torch.bfloat16)
        table = np.full((ns, need), -1, dtype=np.int32)
        perm = list(rng.permutation(need))
        for s in range(ns):
            for j in range(-(-(int(wl.lens[s]) + 1) // wl.BS)):
                table[s, j] = perm.pop()
        wl.table_host = table
    wl.sets = [None]
    scale = 1e9 if wl.unit == "GB/s" else 1e12
    for _ in range(min(args.warmup, 1)):
        wl.cpu_sample(threads, "reference")
    tot_w, tot_s, desc, kind = 0.0, 0.0, "", "port"
    for _ in range(args.steps):
        w, s, desc, kind = wl.cpu_sample(threads, "reference")
        tot_w += w
        tot_s += s
    value = tot_w / tot_s / scale
    line = {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": tot_s / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic (seeded iid N(0,1))", "config": wl.config(),
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": threads, "kind": kind,
                         "sample": "each step: " + desc},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
