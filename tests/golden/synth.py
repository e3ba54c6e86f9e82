"""Bit-stable synthetic BF16 inputs for the golden fixtures.

Everything here is integer arithmetic on hashed indices, so the same seed gives
the same bit patterns on every machine, NumPy build and CPU (no libm, no
floating-point RNG).  Exponents are drawn from small probability tables that
imitate the binade occupancy of common value distributions; sign and mantissa
bits are uniform.  The fixtures store a digest of each input so a silent change
here is caught.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return x ^ (x >> np.uint64(31))


# Exponent offset -> weight out of 65536.  "normal" follows |N(0,1)| binades:
# P(2^e <= |z| < 2^(e+1)) for e = 2 .. -12, the remainder going to e = -13.
_NORMAL = {2: 4, 1: 2978, 0: 17813, -1: 19672, -2: 12152, -3: 6414, -4: 3258, -5: 1634,
           -6: 818, -7: 409, -8: 205, -9: 102, -10: 51, -11: 26, -12: 0}
_LAPLACE = {3: 1, 2: 1178, 1: 7669, 0: 15257, -1: 15637, -2: 11280, -3: 6741, -4: 3678, -5: 1921,
            -6: 982, -7: 496, -8: 249, -9: 125, -10: 63, -11: 31, -12: 0}


def _thresholds(table: dict[int, int]):
    offsets = sorted(table, reverse=True)
    weights = np.array([table[o] for o in offsets], dtype=np.int64)
    weights[-1] = 65536 - weights[:-1].sum()
    assert weights[-1] >= 0
    return np.array(offsets, dtype=np.int64), np.cumsum(weights)


def synth_bf16(n: int, seed: int, kind: str = "normal", base_exponent: int = 0) -> np.ndarray:
    """Return ``n`` BF16 bit patterns as int16.

    kind: ``normal`` / ``laplace`` (binade tables above, centred on
    ``base_exponent``), ``wide`` (exponents uniform over 24 binades: overflows
    every lane budget), ``sparse`` (half exact +0.0, else ``normal``),
    ``outliers`` (``laplace`` with 1 in 1024 values pushed up 7 binades),
    ``ones`` (all 1.0), ``zeros`` (all +0.0).
    """
    idx = np.arange(n, dtype=np.uint64) + (np.uint64(seed) << np.uint64(40))
    h = _splitmix64(idx)
    h2 = _splitmix64(h)
    low = (h & np.uint64(0xFF)).astype(np.int64)          # sign + 7 mantissa bits
    u16 = ((h >> np.uint64(8)) & np.uint64(0xFFFF)).astype(np.int64)
    if kind == "ones":
        return np.full(n, 0x3F80, np.uint16).view(np.int16)
    if kind == "zeros":
        return np.zeros(n, np.int16)
    if kind == "wide":
        offset = (u16 % 24) - 12
    else:
        table = _LAPLACE if kind in ("laplace", "outliers") else _NORMAL
        offsets, cumulative = _thresholds(table)
        offset = offsets[np.searchsorted(cumulative, u16, side="right")]
        if kind == "outliers":
            bump = ((h2 >> np.uint64(20)) & np.uint64(1023)) == 0
            offset = offset + 7 * bump
    exponent = np.clip(127 + base_exponent + offset, 1, 254)
    bits = ((low & 0x80) << 8) | (exponent << 7) | (low & 0x7F)
    if kind == "sparse":
        zero = ((h2 >> np.uint64(33)) & np.uint64(1)) == 1
        bits = np.where(zero, 0, bits)
    return bits.astype(np.uint16).view(np.int16)


def synth_exact_scale(n: int, seed: int) -> np.ndarray:
    """BF16 powers of two 2^k, k in [-2, 2], with random sign: multiplying or
    adding through them never rounds, so fused-op results do not depend on the
    rounding mode of whatever computes them."""
    idx = np.arange(n, dtype=np.uint64) + (np.uint64(seed) << np.uint64(40))
    h = _splitmix64(idx)
    k = (h % np.uint64(5)).astype(np.int64) - 2
    sign = ((h >> np.uint64(17)) & np.uint64(1)).astype(np.int64)
    bits = (sign << 15) | ((127 + k) << 7)
    return bits.astype(np.uint16).view(np.int16)
