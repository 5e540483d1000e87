"""Shared pieces of the parity tests: seeded inputs, device staging and the acceptance bounds.

Bounds (stated by the build target): output max-abs <= 2e-3 for fp16 and <= 8e-3 for bf16 against the
FP64 oracle on the same dequantised inputs, relative L2 <= 1e-3. A correctly rounded bf16 result
already has a relative L2 of ~1.7e-3 on unit-variance inputs, so for bf16 the 1e-3 budget is applied
on top of that rounding floor, which each test computes by rounding the oracle itself to bf16.
fp32 (reference-level backends only) keeps the reference's own bound of 1e-4 max-abs.
"""
from __future__ import annotations

import numpy as np

import oracle_lib as ol

MAX_ABS = {ol.DT_F16: 2e-3, ol.DT_BF16: 8e-3, ol.DT_F32: 1e-4}
REL_L2 = 1e-3


def torch_dtype(dt):
    import torch
    return {ol.DT_F32: torch.float32, ol.DT_F16: torch.float16, ol.DT_BF16: torch.bfloat16}[dt]


def uniform_inputs(shape, seed, dt, low=-1.0, high=1.0):
    """xorshift32 uniform values as in the reference's tests -> (storage bits, dequantised float32)."""
    vals = ol.random_floats(int(np.prod(shape)), seed, low, high).reshape(shape)
    return ol.encode(vals, dt)


def normal_inputs(shape, seed, dt):
    """iid N(0,1) in fp32 from a seed, then cast (the distribution the headline configs use)."""
    rng = np.random.Generator(np.random.Philox(seed))
    vals = rng.standard_normal(size=shape, dtype=np.float32)
    return ol.encode(vals, dt)


def to_device(bits, dt, device="cuda"):
    import torch
    if dt == ol.DT_F32:
        return torch.from_numpy(np.ascontiguousarray(bits)).to(device)
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device)
    return t.view(torch_dtype(dt))


def to_host_f32(t):
    import torch
    return t.detach().to(torch.float32).cpu().numpy()


def round_like(values64, dt):
    """Round an FP64 oracle result to the storage dtype (round-to-nearest-even) and back."""
    if dt == ol.DT_F32:
        return values64.astype(np.float32).astype(np.float64)
    _, deq = ol.encode(values64.astype(np.float32), dt)
    return deq.astype(np.float64)


def check_close(got_f32, expect64, dt, tag=""):
    got = np.asarray(got_f32, dtype=np.float64)
    assert got.shape == expect64.shape, (got.shape, expect64.shape, tag)
    assert np.isfinite(got).all(), f"non-finite output {tag}"
    diff = np.abs(got - expect64)
    max_abs = float(diff.max()) if diff.size else 0.0
    denom = float(np.sqrt((expect64 ** 2).sum()))
    rel = float(np.sqrt((diff ** 2).sum())) / denom if denom > 0 else 0.0
    floor = 0.0
    if dt != ol.DT_F32 and denom > 0:
        floor = float(np.sqrt(((round_like(expect64, dt) - expect64) ** 2).sum())) / denom
    assert max_abs <= MAX_ABS[dt], f"max_abs={max_abs:.3e} > {MAX_ABS[dt]:.1e} {tag}"
    # The 1e-3 bound is on the value BEFORE the final store. A correctly rounded bf16 result alone is 1.7e-3 away
    # from the FP64 one on unit-variance data, and that rounding error is independent of the error made before the
    # store, so the two add in quadrature: rel^2 <= floor^2 + (1e-3)^2. (fp16's floor, 2e-4, hardly matters.)
    budget = float(np.sqrt(REL_L2 ** 2 + floor ** 2))
    assert rel <= budget, f"rel_l2={rel:.3e} > {budget:.3e} (rounding floor {floor:.3e}) {tag}"
    return max_abs, rel


def error_before_store(rel, floor):
    """Relative L2 error of the value before its final rounding, from the measured total and the rounding floor."""
    return float(np.sqrt(max(rel * rel - floor * floor, 0.0)))
