"""Measures where the backends cross over on this GPU, for the thresholds of the dispatch table
(reference: tools/dispatch_threshold_sweep.py and src/runtime/dispatch_table.inc:30-37).

Two questions, Qwen3-4B head geometry (H_q = 32, H_kv = 8, D = 128, fp16):
  * seq_q = 1: from which seq_kv on is the split-K decode kernel faster than the prefill kernel run on one query
    row (`decode_min_seq_kv`)?
  * prefill: up to which seq_kv is the plain SIMT kernel (the naive / tiled backends) faster than the tensor-core
    flash kernel (`tiled_max_seq_kv`)?
Prints one table per question and the crossover it found; `--emit-inc` prints the initialiser of a thresholds
struct with the measured values. The shipped table keeps the reference's thresholds (the dispatch decisions are
pinned against the reference's own); this tool documents what the hardware would prefer.

    python -m scicompute_attention_b200.dispatch_sweep [--batch B] [--emit-inc]
"""
from __future__ import annotations

import argparse


def _time(fn, iters=20):
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1000.0  # microseconds


def sweep(batch: int):
    import torch
    from . import ops
    hq, hkv, d = 32, 8, 128
    dev = "cuda"
    rows_decode, rows_prefill = [], []
    for skv in (16, 32, 64, 128, 256, 512, 1024, 2048, 4096):
        q = torch.randn(batch, hq, 1, d, device=dev).half()
        k = torch.randn(batch, hkv, skv, d, device=dev).half()
        v = torch.randn(batch, hkv, skv, d, device=dev).half()
        t_dec = _time(lambda: ops.decode_attention(q, k, v))
        t_fla = _time(lambda: ops.flash_attention(q, k, v, causal=True))
        rows_decode.append((skv, t_dec, t_fla))
    for s in (16, 32, 64, 128, 256, 512):
        q = torch.randn(batch, hq, s, d, device=dev).half()
        k = torch.randn(batch, hkv, s, d, device=dev).half()
        v = torch.randn(batch, hkv, s, d, device=dev).half()
        t_simt = _time(lambda: ops.simt_attention(q, k, v, causal=True), iters=5)
        t_fla = _time(lambda: ops.flash_attention(q, k, v, causal=True))
        rows_prefill.append((s, t_simt, t_fla))
    return rows_decode, rows_prefill


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--emit-inc", action="store_true")
    args = ap.parse_args()
    rows_decode, rows_prefill = sweep(args.batch)
    print(f"seq_q = 1, batch {args.batch}: microseconds per call")
    print("  seq_kv   decode    flash")
    decode_min = None
    for skv, t_dec, t_fla in rows_decode:
        print(f"  {skv:6d} {t_dec:8.1f} {t_fla:8.1f}")
        if decode_min is None and t_dec <= t_fla:
            decode_min = skv
    print(f"prefill (seq_q = seq_kv, causal), batch {args.batch}: microseconds per call")
    print("  seq      simt     flash")
    tiled_max = 0
    for s, t_simt, t_fla in rows_prefill:
        print(f"  {s:6d} {t_simt:8.1f} {t_fla:8.1f}")
        if t_simt <= t_fla:
            tiled_max = s
    print(f"decode is the faster choice from seq_kv = {decode_min} on; the SIMT kernel is the faster choice up to seq_kv = {tiled_max}")
    if args.emit_inc:
        print("// measured on this GPU by scicompute_attention_b200.dispatch_sweep")
        print(f"{{/* decode_max_seq_q */ 1, /* decode_min_seq_kv */ {decode_min or 0}, /* tiled_max_seq_kv */ {tiled_max}, "
              "/* min_tokens_per_split */ 256, /* max_splits */ 64, /* revision */ \"b200-measured\"}")


if __name__ == "__main__":
    main()
