"""The decode kernel's equal-share schedule, restated on the host and checked for the properties the kernel relies on.

decode_partial_kernel (csrc/kernels/decode.cu) gives CTA c the steps [c * per_cta, (c + 1) * per_cta) of the
sequence-major list of 64-token steps of all (sequence, kv head, head chunk) units, with
per_cta = max(ceil(total / ctas), ceil(longest / (slots - 1))). The model below follows the kernel's index
arithmetic line by line; the properties: every step of every unit is covered exactly once, every piece of a unit
lands in a slot below `slots`, the slots a unit uses are 0 .. used-1 with `used` as the kernel computes it (the rest
is marked empty by the CTA that holds the unit's first step), and the host-side slot heuristic is large enough that
the balance term, not the slot term, decides per_cta."""
import numpy as np

from scicompute_attention_b200 import ops

STEP = ops.DECODE_STEP_TOKENS


def kernel_schedule(lens, units_per_seq, slots, ctas):
    steps = [max(1, -(-int(n) // STEP)) for n in lens]
    total = sum(steps) * units_per_seq
    longest = max(steps)
    per_cta = max(-(-total // ctas), -(-longest // (slots - 1)))
    before = np.concatenate([[0], np.cumsum(steps)])
    pieces = []   # (cta, sequence, unit, first step, last step (exclusive), slot)
    marked = {}   # (sequence, unit) -> first unused slot, as written by MarkUnusedSlots
    for cta in range(ctas):
        begin = cta * per_cta
        if begin >= total:
            break
        end = min(begin + per_cta, total)
        want = begin // units_per_seq
        b = int(np.searchsorted(before, want, side="right") - 1)
        pos = begin
        while pos < end:
            in_seq = pos - units_per_seq * int(before[b])
            gi, t0 = divmod(in_seq, steps[b])
            unit_start = units_per_seq * int(before[b]) + gi * steps[b]
            t1 = min(steps[b], t0 + (end - pos))
            slot = cta - unit_start // per_cta
            if t0 == 0:
                marked[(b, gi)] = (unit_start + steps[b] - 1) // per_cta - unit_start // per_cta + 1
            pieces.append((cta, b, gi, t0, t1, slot))
            pos += t1 - t0
            if t1 == steps[b] and gi == units_per_seq - 1 and pos < end:
                b += 1
    return steps, per_cta, pieces, marked


def check(lens, units_per_seq, slots, ctas):
    steps, per_cta, pieces, marked = kernel_schedule(lens, units_per_seq, slots, ctas)
    covered = {}
    used = {}
    for cta, b, gi, t0, t1, slot in pieces:
        assert 0 <= slot < slots, (lens, slots, ctas, slot)
        assert t0 < t1 <= steps[b]
        for t in range(t0, t1):
            assert (b, gi, t) not in covered
            covered[(b, gi, t)] = cta
        used.setdefault((b, gi), []).append(slot)
    assert len(covered) == sum(steps) * units_per_seq
    for key, got in used.items():
        assert sorted(got) == list(range(len(got))), (key, got)      # slots 0 .. n-1, each once
        assert marked[key] == len(got), (key, marked[key], got)      # the rest is what gets marked empty
    return per_cta


def test_every_step_is_covered_once_and_slots_stay_in_range():
    rng = np.random.default_rng(5)
    for _ in range(300):
        nseq = int(rng.integers(1, 40))
        lens = rng.integers(0, 9000, size=nseq)
        if rng.random() < 0.3:
            lens[rng.integers(0, nseq)] = 0
        units = int(rng.integers(1, 9))
        slots = int(rng.integers(2, 20))
        ctas = int(rng.choice([1, 3, 37, 148, 296]))
        check(lens, units, slots, ctas)


def test_baseline_shapes_are_balanced_by_the_automatic_slot_count():
    """With the automatic slot count the share per CTA is the balanced one (ceil(total / ctas)), not one inflated by
    too few slots - at the full configurations and at one GPU's share of them on 8 GPUs."""
    sms = 148
    for batch, seq in ((128, 4096), (16, 4096), (8, 131072), (8, 16384), (8, 32768), (1, 131072)):
        units = 8
        slots = ops.splits_for(seq, batch, 8, 4, sms)
        per_cta = check([seq] * batch, units, slots, 2 * sms)
        total = batch * units * -(-seq // STEP)
        assert per_cta == -(-total // (2 * sms)), (batch, seq, slots, per_cta)
    rng = np.random.default_rng(0)
    for nseq in (256, 32):
        lens = rng.integers(512, 8193, size=nseq) + 1
        slots = ops.paged_splits_for(int(lens.mean()), nseq, 8, 4, sms)
        per_cta = check(lens, 8, slots, 2 * sms)
        total = 8 * sum(-(-int(n) // STEP) for n in lens)
        assert per_cta == -(-total // (2 * sms))
