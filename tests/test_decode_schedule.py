"""The decode kernel's equal-share schedule, restated on the host and checked for the properties the kernel relies on.

decode_partial_kernel (csrc/kernels/decode.cu) ties every CTA to one (kv head, head chunk) column; the CTAs of a column
split its list of 64-token steps (sequence after sequence) into contiguous shares of
per_cta = max(ceil(total / sharers), ceil(longest / (slots - 1))) steps. The model below follows the kernel's index
arithmetic line by line; the properties: every step of every sequence is covered exactly once, every piece of a
sequence lands in a slot below `slots`, the slots a sequence uses are 0 .. used-1 with `used` as the kernel computes it
(the rest is marked empty by the CTA that holds the sequence's first step), and the host-side slot heuristic is large
enough that the balance term, not the slot term, decides per_cta."""
import numpy as np

from scicompute_attention_b200 import ops

STEP = ops.DECODE_STEP_TOKENS


def column_schedule(lens, slots, sharers, uniform):
    """Shares of one column: list of (share, sequence, first step, last step (exclusive), slot) and the marks."""
    steps = [max(1, -(-int(n) // STEP)) for n in lens]
    total, longest = sum(steps), max(steps)
    per_cta = -(-total // sharers)
    floor_steps = -(-longest // (slots - 1)) if slots > 1 else total
    per_cta = max(per_cta, floor_steps)
    if slots == 1 and uniform:
        per_cta = -(-per_cta // steps[0]) * steps[0]
    before = np.concatenate([[0], np.cumsum(steps)])
    pieces, marked = [], {}
    for share in range(sharers):
        begin = share * per_cta
        if begin >= total:
            break
        end = min(begin + per_cta, total)
        b = int(np.searchsorted(before, begin, side="right") - 1)
        pos = begin
        while pos < end:
            t0 = pos - int(before[b])
            t1 = min(steps[b], t0 + (end - pos))
            slot = share - int(before[b]) // per_cta
            if t0 == 0:
                marked[b] = (int(before[b]) + steps[b] - 1) // per_cta - int(before[b]) // per_cta + 1
            pieces.append((share, b, t0, t1, slot))
            pos += t1 - t0
            if t1 == steps[b] and pos < end:
                b += 1
    return steps, per_cta, pieces, marked


def check(lens, slots, sharers, uniform=False):
    steps, per_cta, pieces, marked = column_schedule(lens, slots, sharers, uniform)
    covered, used = {}, {}
    for share, b, t0, t1, slot in pieces:
        assert 0 <= slot < slots, (list(lens), slots, sharers, slot)
        assert t0 < t1 <= steps[b]
        for t in range(t0, t1):
            assert (b, t) not in covered
            covered[(b, t)] = share
        used.setdefault(b, []).append(slot)
    assert len(covered) == sum(steps)
    for b, got in used.items():
        assert sorted(got) == list(range(len(got))), (b, got)   # slots 0 .. n-1, each once
        assert marked[b] == len(got), (b, marked[b], got)       # the rest is what gets marked empty
    return per_cta


def test_every_step_is_covered_once_and_slots_stay_in_range():
    rng = np.random.default_rng(5)
    for _ in range(400):
        nseq = int(rng.integers(1, 40))
        lens = rng.integers(0, 9000, size=nseq)
        if rng.random() < 0.3:
            lens[rng.integers(0, nseq)] = 0
        check(lens, int(rng.integers(2, 20)), int(rng.choice([1, 2, 9, 37, 74])))
    for seq in (1, 63, 64, 65, 4096, 5000):
        for batch in (1, 3, 128):
            for slots in (1, 2, 7):
                check([seq] * batch, slots, int(rng.choice([1, 4, 37])), uniform=True)
    check(rng.integers(0, 3000, size=9), 1, 37)   # one slot, ragged: the column goes to its first CTA


def test_baseline_shapes_are_balanced_by_the_automatic_slot_count():
    """With the automatic slot count the share per CTA is the balanced one (ceil(total / sharers)), not one inflated
    by too few slots - at the full configurations and at one GPU's share of them on 8 GPUs."""
    sms, columns = 148, 8
    sharers = 2 * sms // columns
    for batch, seq in ((128, 4096), (16, 4096), (8, 131072), (8, 16384), (8, 32768), (1, 131072)):
        slots = ops.splits_for(seq, batch, 8, 4, sms)
        per_cta = check([seq] * batch, slots, sharers, uniform=True)
        assert per_cta == -(-batch * -(-seq // STEP) // sharers), (batch, seq, slots, per_cta)
    rng = np.random.default_rng(0)
    for nseq in (256, 32):
        lens = rng.integers(512, 8193, size=nseq) + 1
        slots = ops.paged_splits_for(int(lens.mean()), nseq, 8, 4, sms, int(lens.max()))
        per_cta = check(lens, slots, sharers)
        assert per_cta == -(-sum(-(-int(n) // STEP) for n in lens) // sharers)
