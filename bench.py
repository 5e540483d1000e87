#!/usr/bin/env python
"""Benchmark of the attention hot path on B200: one JSON line on stdout.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload flash|decode|paged]
  python bench.py --impl reference ...      # the reference's CPU path on the host cores

A "step" is one pass of the hot path over one batch of seeded synthetic input that is already
resident in HBM. Timed with CUDA events on the launching stream between barrier + synchronize on
both sides; with N > 1 ranks (one process per GPU) every rank runs the same per-GPU workload on its
own independent sequences (no data-path collective), the slowest rank's time is taken and the
reported value is the work of all ranks divided by it ("weak" scaling).

Workloads (shapes of a Qwen3-4B attention layer: H_q = 32, H_kv = 8, D = 128):
  flash   causal prefill, B = 4, S = 4096, bf16      -> TFLOP/s, FLOPs = 4 B H_q D S (S + 1) / 2
  decode  split-K decode, B = 128, S_kv = 4096, bf16  -> GB/s over bytes(K) + bytes(V) + bytes(Q) + bytes(O)
  paged   256 sequences, lengths U[512, 8192], 16-token pages in a 160k-block pool with a shuffled
          free list; one token appended per sequence, then attended -> GB/s over the KV bytes read
  longctx B = 8, S_kv = 131072 with the KV sequence split over the ranks (strong scaling); the partial
          (m, l, O) triples cross NVLink inside one merge kernel over peer-mapped buffers
          (--exchange nccl: one NCCL all-gather between two kernels) -> GB/s over the whole K/V
"""
from __future__ import annotations

import argparse
import json
import math
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
    name = ""
    metric = ""
    unit = ""
    bound = ""
    launches_per_step = 0

    def setup(self, torch, device, seed): ...
    def step(self): ...
    def work_per_step(self): ...          # algorithmic bytes or flops of one step
    def e2e_setup(self, torch): ...
    def e2e_step(self): ...               # H2D + step + D2H; returns nothing
    def cpu_sample(self, threads, impl): ...  # -> (work_done, seconds, description, kind)

    def traffic(self):
        return getattr(self, "traffic_bytes", None)


class DecodeWorkload(Workload):
    name = "splitk_decode_B128_Skv4096_Hq32_Hkv8_D128_bf16"
    metric, unit, bound = "decode_kv_bandwidth", "GB/s", "hbm"
    launches_per_step = 2  # partial + merge
    B, SKV = 128, 4096
    # dram__bytes_read + dram__bytes_write of decode_partial_kernel, ncu capture at B=16 scaled x8
    # (profiles/decode_splitk_c3.md); traffic grows in proportion to the batch
    traffic_bytes = (268.61e6 + 5.8e6) * 8

    def setup(self, torch, device, seed):
        from scicompute_attention_b200 import ops
        self.torch, self.ops = torch, ops
        g = torch.Generator(device=device).manual_seed(seed)
        self.q = torch.randn((self.B, HQ, 1, D), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        self.k = torch.randn((self.B, HKV, self.SKV, D), generator=g, device=device, dtype=torch.bfloat16)
        self.v = torch.randn((self.B, HKV, self.SKV, D), generator=g, device=device, dtype=torch.bfloat16)
        self.out = None

    def step(self):
        self.out = self.ops.decode_attention(self.q, self.k, self.v)

    def work_per_step(self):
        return 2 * self.B * HKV * self.SKV * D * 2 + 2 * self.B * HQ * D * 2

    def config(self):
        return {"workload": self.name, "batch": self.B, "seq_kv": self.SKV, "heads_q": HQ, "heads_kv": HKV,
                "head_dim": D, "l2_policy": "inputs larger than L2 (2.1 GB per step)",
                "sharding": "independent sequences per GPU, no collective"}

    def e2e_setup(self, torch):
        self.hq = self.q.cpu().pin_memory()
        self.hk = self.k.cpu().pin_memory()
        self.hv = self.v.cpu().pin_memory()
        self.ho = torch.empty((self.B, HQ, 1, D), dtype=torch.bfloat16).pin_memory()
        self.h2d = self.hq.numel() * 2 + self.hk.numel() * 2 + self.hv.numel() * 2
        self.d2h = self.ho.numel() * 2

    def e2e_step(self):
        self.q.copy_(self.hq, non_blocking=True)
        self.k.copy_(self.hk, non_blocking=True)
        self.v.copy_(self.hv, non_blocking=True)
        out = self.ops.decode_attention(self.q, self.k, self.v)
        self.ho.copy_(out, non_blocking=True)

    def cpu_sample(self, threads, impl):
        import numpy as np
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
    name = "paged_decode_256seq_len512-8192_bs16_pool160k_Hq32_Hkv8_D128_bf16"
    metric, unit, bound = "paged_decode_kv_bandwidth", "GB/s", "hbm"
    launches_per_step = 3  # batched append + partial + merge
    NSEQ, BS, NBLK = 256, 16, 160000
    # ncu capture of the paged decode_partial_kernel on 32 sequences: 606.3 MB moved for 597.7 MB of K/V
    # (profiles/paged_decode_c4.md); scaled by the tokens of the full batch in roofline()
    traffic_ratio = (598.10e6 + 8.21e6) / 597.75e6

    def setup(self, torch, device, seed):
        import numpy as np
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        from scicompute_attention_b200 import ops
        self.torch, self.ops, self.np = torch, ops, np
        rng = np.random.default_rng(seed)
        self.lens = rng.integers(512, 8193, size=self.NSEQ).astype(np.int64)
        # LIFO allocator with a seeded shuffle of its free list -> non-contiguous page tables. The
        # allocation order is the reference's: allocate everything, shuffle, free in that order, then
        # every allocation pops from the back (src/kv_cache/block_manager.cpp:25-27,60-62).
        ids = np.arange(self.NBLK, dtype=np.int32)
        rng.shuffle(ids)
        free = list(ids)  # freed in this order; allocation pops from the back
        max_blocks = self.NBLK  # table row length = pool size (src/kv_cache/paged_kv_cache.cpp:22-27)
        table = np.full((self.NSEQ, max_blocks), -1, dtype=np.int32)
        for s in range(self.NSEQ):
            need = -(-(int(self.lens[s]) + 1) // self.BS)
            for j in range(need):
                table[s, j] = free.pop()
        self.table_host = table
        self.page_table = torch.from_numpy(table).to(device)
        self.seq_lens = torch.from_numpy((self.lens + 1).astype(np.int32)).to(device)  # includes the new token
        g = torch.Generator(device=device).manual_seed(seed)
        shape = (self.NBLK, self.BS, HKV, D)
        self.k_pool = torch.randn(shape, generator=g, device=device, dtype=torch.bfloat16)
        self.v_pool = torch.randn(shape, generator=g, device=device, dtype=torch.bfloat16)
        self.q = torch.randn((self.NSEQ, HQ, 1, D), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        self.k_new = torch.randn((self.NSEQ, HKV, D), generator=g, device=device, dtype=torch.bfloat16)
        self.v_new = torch.randn((self.NSEQ, HKV, D), generator=g, device=device, dtype=torch.bfloat16)
        self.mean_len = int(self.lens.mean()) + 1
        # scheduling hint: longest sequences first (the host knows the lengths of its batch)
        self.seq_order = torch.from_numpy(np.argsort(-self.lens, kind="stable").astype(np.int32)).to(device)

    def step(self):
        self.ops.kv_append_batched(self.k_pool, self.v_pool, self.k_new, self.v_new, self.page_table, self.seq_lens)
        self.out = self.ops.paged_attention(self.q, self.k_pool, self.v_pool, self.page_table, self.seq_lens,
                                            block_size=self.BS, typical_len=self.mean_len, seq_order=self.seq_order)

    def work_per_step(self):
        toks = int((self.lens + 1).sum())
        pages = int(sum(-(-(int(n) + 1) // self.BS) for n in self.lens))
        return toks * (2 * HKV * D * 2) + 2 * self.NSEQ * HQ * D * 2 + pages * 4 + self.NSEQ * 4

    def traffic(self):
        return float((self.lens + 1).sum()) * 2 * HKV * D * 2 * self.traffic_ratio

    def config(self):
        return {"workload": self.name, "num_seqs": self.NSEQ, "block_size": self.BS, "pool_blocks": self.NBLK,
                "tokens_attended": int((self.lens + 1).sum()), "heads_q": HQ, "heads_kv": HKV, "head_dim": D,
                "l2_policy": "inputs larger than L2 (4.6 GB of KV read per step)",
                "sharding": "independent sequences and pools per GPU, no collective"}

    def e2e_setup(self, torch):
        # what a serving loop moves per step: the new tokens' q/k/v up, the attention output down;
        # the KV pool and page table live on the device across steps
        self.hq = self.q.cpu().pin_memory()
        self.hkn = self.k_new.cpu().pin_memory()
        self.hvn = self.v_new.cpu().pin_memory()
        self.ho = torch.empty((self.NSEQ, HQ, 1, D), dtype=torch.bfloat16).pin_memory()
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


class FlashWorkload(Workload):
    name = "flash_prefill_causal_B4_S4096_Hq32_Hkv8_D128_bf16"
    metric, unit, bound = "flash_prefill_throughput", "TFLOP/s", "tensor"
    launches_per_step = 1
    B, S = 4, 4096
    # dram__bytes_read + dram__bytes_write of flash_fwd_sm100_kernel, ncu capture at B=1 scaled x4
    # (profiles/flash_prefill_c2.md); the output mostly stays in L2 until after the kernel
    traffic_bytes = (50.41e6 + 2.9e6) * 4
    dtype_name = "bf16"  # --dtype fp16 runs the same configuration in half precision

    def setup(self, torch, device, seed):
        from scicompute_attention_b200 import ops
        self.torch, self.ops = torch, ops
        g = torch.Generator(device=device).manual_seed(seed)
        dt = torch.float16 if self.dtype_name == "fp16" else torch.bfloat16
        self.q = torch.randn((self.B, HQ, self.S, D), generator=g, device=device, dtype=torch.float32).to(dt)
        self.k = torch.randn((self.B, HKV, self.S, D), generator=g, device=device, dtype=torch.float32).to(dt)
        self.v = torch.randn((self.B, HKV, self.S, D), generator=g, device=device, dtype=torch.float32).to(dt)
        self.out = torch.empty_like(self.q)
        # 256 MiB scratch written between steps would flush L2; inputs + output (320 MiB) already exceed it
        self.flush = None

    def step(self):
        self.ops.flash_attention(self.q, self.k, self.v, causal=True, out=self.out)

    def work_per_step(self):
        return 4 * self.B * HQ * D * (self.S * (self.S + 1) // 2)

    def config(self):
        return {"workload": self.name.replace("bf16", self.dtype_name), "batch": self.B, "seq_len": self.S, "heads_q": HQ,
                "heads_kv": HKV, "head_dim": D, "causal": True,
                "l2_policy": "inputs + output (335 MB per step) larger than L2",
                "sharding": "independent (batch, kv-head group) units per GPU, no collective"}

    def e2e_setup(self, torch):
        self.hq = self.q.cpu().pin_memory()
        self.hk = self.k.cpu().pin_memory()
        self.hv = self.v.cpu().pin_memory()
        self.ho = torch.empty(self.q.shape, dtype=self.q.dtype).pin_memory()
        self.h2d = (self.hq.numel() + self.hk.numel() + self.hv.numel()) * 2
        self.d2h = self.ho.numel() * 2
        self.e2e_streams = [torch.cuda.Stream() for _ in range(self.B)]

    def e2e_step(self):
        # one stream per batch element: the upload of prompt b + 1 overlaps the kernel and the download of prompt b
        # (the two copy directions are separate engines); the launching stream joins all of them at the end, so the
        # events around the timed region see the whole step
        torch = self.torch
        cur = torch.cuda.current_stream()
        for b in range(self.B):
            side = self.e2e_streams[b]
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                self.q[b:b + 1].copy_(self.hq[b:b + 1], non_blocking=True)
                self.k[b:b + 1].copy_(self.hk[b:b + 1], non_blocking=True)
                self.v[b:b + 1].copy_(self.hv[b:b + 1], non_blocking=True)
                self.ops.flash_attention(self.q[b:b + 1], self.k[b:b + 1], self.v[b:b + 1], causal=True,
                                         out=self.out[b:b + 1], stream=side)
                self.ho[b:b + 1].copy_(self.out[b:b + 1], non_blocking=True)
        for side in self.e2e_streams:
            cur.wait_stream(side)

    def cpu_sample(self, threads, impl):
        # bounded sample: one (batch 0, head) pair per host thread; the main arm's CPU leg takes whole
        # causal heads (all 4096 rows), one step of the reference arm the last 256 query rows (rows i attend to
        # i + 1 keys); FLOPs are counted for the sampled rows only
        import numpy as np
        skv = self.q.shape[2]
        sq = skv if impl == "port" else min(256, skv)
        nh = max(1, min(HQ, threads))
        q = self.q[:1, :nh, skv - sq:skv].float().cpu().numpy()
        k = self.k[:1, :HKV, :skv].float().cpu().numpy()
        v = self.v[:1, :HKV, :skv].float().cpu().numpy()
        k = np.repeat(k, HQ // HKV, axis=1)[:, :nh]
        v = np.repeat(v, HQ // HKV, axis=1)[:, :nh]
        secs, kind = run_cpu_attention(q, np.ascontiguousarray(k), np.ascontiguousarray(v), True, threads, impl)
        flops = 4 * nh * D * sum(skv - sq + i + 1 for i in range(sq))
        return flops, secs, f"{nh} heads x last {sq} query rows of a {skv}-token causal prefix", kind


class LongContextWorkload(Workload):
    """Sequence-split decode: B = 8, S_kv = 131072; the KV axis is cut into one contiguous slice per rank,
    every rank reduces its slice to (m, l, O) triples, B*H_q*(2+D) floats per rank travel to every peer
    (stored by the merge kernel into peer-mapped buffers, or by one NCCL all-gather), and every rank merges.
    Total work is fixed, so this workload scales "strong"."""
    name = "seqsplit_decode_B8_Skv131072_Hq32_Hkv8_D128_bf16"
    metric, unit, bound = "longctx_decode_kv_bandwidth", "GB/s", "hbm"
    launches_per_step = 2  # partial kernel + fused merge / exchange / merge (3 plus the all-gather with --exchange nccl)
    scaling = "strong"
    B, SKV = 8, 131072
    traffic_bytes = None
    exchange = "peer"

    def setup(self, torch, device, seed):
        import torch.distributed as dist
        from scicompute_attention_b200 import multi_gpu, ops
        self.torch, self.ops, self.mg = torch, ops, multi_gpu
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        lo, hi = multi_gpu.kv_range_for_rank(self.SKV, self.rank, self.world)
        g = torch.Generator(device=device).manual_seed(1234)  # q is replicated: same seed on every rank
        self.q = torch.randn((self.B, HQ, 1, D), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        g2 = torch.Generator(device=device).manual_seed(seed + 77)
        self.k = torch.randn((self.B, HKV, hi - lo, D), generator=g2, device=device, dtype=torch.bfloat16)
        self.v = torch.randn((self.B, HKV, hi - lo, D), generator=g2, device=device, dtype=torch.bfloat16)
        self.px = None
        if self.world > 1 and self.exchange == "peer":
            self.px = multi_gpu.PeerExchange(self.B * HQ, D, device)
            # the whole step (partial kernel + exchange kernel) is one captured graph, replayed every step
            self.graph, self.out = self.px.capture(self.q, self.k, self.v)
        else:
            self.launches_per_step = 3

    def step(self):
        if self.px is not None:
            self.graph.replay()
        else:
            self.out = self.mg.sequence_split_decode(self.q, self.k, self.v)

    def work_per_step(self):
        # whole job: all ranks together read the full K and V once
        return 2 * self.B * HKV * self.SKV * D * 2 + 2 * self.B * HQ * D * 2

    def config(self):
        return {"workload": self.name, "batch": self.B, "seq_kv": self.SKV, "heads_q": HQ, "heads_kv": HKV,
                "head_dim": D, "l2_policy": "inputs larger than L2 (4.3 GB over all ranks)",
                "sharding": "KV sequence split across ranks; (m, l, O) triples exchanged " +
                            ("by peer stores inside the merge kernel" if self.px is not None else
                             "by one NCCL all-gather per step" if self.world > 1 else "locally (one rank)")}

    def e2e_setup(self, torch):
        self.hq = self.q.cpu().pin_memory()
        self.ho = torch.empty((self.B * HQ, D), dtype=torch.bfloat16).pin_memory()
        self.h2d, self.d2h = self.hq.numel() * 2, self.ho.numel() * 2

    def e2e_step(self):
        # a decode step moves the new query up and the attention output down; the KV cache lives on the devices
        self.q.copy_(self.hq, non_blocking=True)
        self.step()
        self.ho.copy_(self.out, non_blocking=True)

    def cpu_sample(self, threads, impl):
        nb = 1
        skv = 16384
        q = self.q[:nb].float().cpu().numpy()
        k = self.k[:nb, :, :skv].float().cpu().numpy()
        v = self.v[:nb, :, :skv].float().cpu().numpy()
        secs, kind = run_cpu_attention(q, k, v, True, threads, impl)
        work = 2 * nb * HKV * k.shape[2] * D * 2 + 2 * nb * HQ * D * 2
        return work, secs, f"{nb} of {self.B} sequences, first {k.shape[2]} of {self.SKV} keys, all heads", kind


WORKLOADS = {"flash": FlashWorkload, "decode": DecodeWorkload, "paged": PagedWorkload, "longctx": LongContextWorkload}
DEFAULT_WORKLOAD = "flash"


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
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=0, help="0 = min(steps, 5)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"], help="flash workload only")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="longctx on more than one GPU: how the triples cross NVLink")
    ap.add_argument("--capture", action="store_true",
                    help="profiler-sized variant of the workload (same kernels, a few hundred MB): flash B=1, "
                         "decode B=16, paged 32 sequences in a 20k-block pool; skips the e2e and CPU legs")
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
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    LongContextWorkload.exchange = args.exchange
    FlashWorkload.dtype_name = args.dtype
    wl = WORKLOADS[args.workload]()
    if args.capture:
        if isinstance(wl, FlashWorkload):
            wl.B = 1
        elif isinstance(wl, DecodeWorkload):
            wl.B = 16
        else:
            wl.NSEQ, wl.NBLK = 32, 20000
        wl.name += "_capture"
    wl.setup(torch, device, args.seed + rank)
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    start.record(stream)
    for _ in range(args.steps):
        wl.step()
    stop.record(stream)
    barrier()
    clocks = sampler.stop()
    ms_total = start.elapsed_time(stop)

    # end to end through the public operator with host buffers: pinned H2D of the step's inputs,
    # the step, D2H of its result - all inside the timed region
    e2e_steps = args.e2e_steps or min(args.steps, 5)
    e2e_ms = None
    wl.h2d = wl.d2h = 0
    if not args.capture:
        wl.e2e_setup(torch)
        wl.e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            wl.e2e_step()
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps

    if world > 1:
        t = torch.tensor([ms_total, e2e_ms or 0.0], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms = float(t[0]), (float(t[1]) if e2e_ms is not None else None)
    ms_step = ms_total / args.steps
    work = wl.work_per_step()
    scale = 1e9 if wl.unit == "GB/s" else 1e12
    strong = getattr(wl, "scaling", "weak") == "strong"   # strong: `work` is already the whole job
    value = work / (ms_step * 1e-3) / scale * (1 if strong else world)
    per_gpu = value / world
    e2e_value = (work / (e2e_ms * 1e-3) / scale * (1 if strong else world)) if e2e_ms else None

    if rank == 0:
        peaks = measured_peaks()
        peak = peaks["hbm_gbs"] if wl.bound == "hbm" else peaks["tflops"]
        nominal = NOMINAL_HBM_GBS if wl.bound == "hbm" else NOMINAL_TENSOR_TFLOPS
        cpu = None
        if not args.capture:
            cw, cs, desc, kind = wl.cpu_sample(threads, "port")
            cpu = {"value": cw / cs / scale, "unit": wl.unit, "cores": threads, "kind": kind,
                   "sample": desc + f" ({cs:.1f} s of FP64 host work)"}
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": getattr(wl, "scaling", "weak"),
            "vs_baseline": None, "dtype": getattr(wl, "dtype_name", "bf16"),
            "data": "synthetic (seeded iid N(0,1), random page tables)",
            "config": wl.config(),
            "roofline": {"bound": wl.bound, "achieved": per_gpu, "peak": peak, "unit": wl.unit,
                         "frac": per_gpu / peak, "peak_source": peaks["source"],
                         "frac_of_nominal": per_gpu / nominal, "traffic": wl.traffic(),
                         "traffic_unit": "bytes per launch of the dominant kernel (ncu capture, scaled; see profiles/)"},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": wl.launches_per_step * args.steps,
            "clocks": clocks,
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

    class _HostTorchShim:
        """The CPU arm needs the workload's tensors but no GPU: build them with torch on the host."""

    import torch
    LongContextWorkload.exchange = args.exchange
    FlashWorkload.dtype_name = args.dtype
    wl = WORKLOADS[args.workload]()
    # host tensors with the workload's shapes, reduced to the sample the CPU leg consumes
    g = torch.Generator().manual_seed(args.seed)
    if isinstance(wl, FlashWorkload):
        wl.q = torch.randn((1, HQ, wl.S, D), generator=g).to(torch.bfloat16)
        wl.k = torch.randn((1, HKV, wl.S, D), generator=g).to(torch.bfloat16)
        wl.v = torch.randn((1, HKV, wl.S, D), generator=g).to(torch.bfloat16)
    elif isinstance(wl, LongContextWorkload):
        wl.q = torch.randn((1, HQ, 1, D), generator=g).to(torch.bfloat16)
        wl.k = torch.randn((1, HKV, 16384, D), generator=g).to(torch.bfloat16)
        wl.v = torch.randn((1, HKV, 16384, D), generator=g).to(torch.bfloat16)
    elif isinstance(wl, DecodeWorkload):
        nb = max(1, min(wl.B, 8 * threads))
        wl.q = torch.randn((nb, HQ, 1, D), generator=g).to(torch.bfloat16)
        wl.k = torch.randn((nb, HKV, wl.SKV, D), generator=g).to(torch.bfloat16)
        wl.v = torch.randn((nb, HKV, wl.SKV, D), generator=g).to(torch.bfloat16)
    else:
        rng = np.random.default_rng(args.seed)
        wl.np, wl.torch = np, torch
        wl.lens = rng.integers(512, 8193, size=wl.NSEQ).astype(np.int64)
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
