"""Integer rescale parameters for seeded workloads.

The TFLite/TOSA "quantize multiplier" rule with scale32 = true: a real scale r
becomes (multiplier, shift) with r = multiplier * 2**-shift and
multiplier in [2**30, 2**31). The reference's fixtures carry integers of exactly
this form (e.g. multiplier 2003370132 / shift 39 in
tests/testdata/gen_ops/conv2d_8x8.mlir).
"""
from __future__ import annotations

import math

import numpy as np


def quantize_multiplier(real: float) -> tuple[int, int]:
    if real == 0.0:
        return 0, 2
    q, e = math.frexp(real)
    m = int(math.floor(q * (1 << 31) + 0.5))
    if m == (1 << 31):
        m //= 2
        e += 1
    s = 31 - e
    if s > 62:
        m >>= s - 62
        s = 62
    if s < 2:
        raise ValueError(f"scale {real} too large for a scale32 rescale")
    return m, s


def quantize_multipliers(reals) -> tuple[np.ndarray, np.ndarray]:
    ms = [quantize_multiplier(float(r)) for r in np.atleast_1d(reals)]
    return (np.array([m for m, _ in ms], np.int32), np.array([s for _, s in ms], np.int8))


def relu6_clamp(out_scale: float, out_zp: int) -> tuple[int, int]:
    """Quantised-domain clamp range of a folded ReLU6."""
    lo = max(-128, out_zp)
    hi = min(127, out_zp + int(round(6.0 / out_scale)))
    return lo, hi


def add_rescale_params(s0: float, s1: float, s_out: float, input_shift: int = 20):
    """Input/output rescales of a quantized add as the TFLite->TOSA legalisation
    forms them (two i8->i32 rescales with a 2**20 left shift folded in, one
    i32->i8 rescale; form visible in tests/testdata/tosa_ops/add-single-rescale.mlir)."""
    max2 = 2.0 * max(s0, s1)
    m0 = quantize_multiplier((1 << input_shift) * s0 / max2)
    m1 = quantize_multiplier((1 << input_shift) * s1 / max2)
    mo = quantize_multiplier(max2 / (s_out * (1 << input_shift)))
    return m0, m1, mo
