"""Normal deviates from a counter: the same bits on the host and on the device.

A tensor's values are a pure function of (key, element index): Philox4x32-10 (Salmon et al., SC11;
the generator the reference's sampler uses, helios/crates/helios-hal/src/sampler_reference.rs:67-84)
turns the counter ``index // 2`` into four 32-bit words, the first two become the uniforms of a
Box-Muller transform, and elements ``2c`` and ``2c + 1`` are its cosine and its sine branch.  The
transform is written with additions, multiplications, divisions and square roots in 64-bit floating
point only, in a fixed order and with nothing fused: every one of them is correctly rounded by IEEE 754
on the host (numpy) and on the device (``__dadd_rn`` and its kin in ``csrc/random_normal.cu``), so
the two agree bit for bit.  The logarithm and the cosine and sine are series whose coefficients are
computed here once and handed to the kernel, so that both sides use the same numbers:

* ``ln u = e ln 2 + 2 s (1 + s^2/3 + s^4/5 + ...)`` with ``u = m 2^e``, ``m`` in [sqrt(1/2), sqrt(2))
  and ``s = (m - 1)/(m + 1)``, so ``|s| < 0.172`` and nine terms leave an error below 1e-15;
* ``cos`` and ``sin`` of an angle in [0, pi/2) by their Taylor series to the 22nd and 23rd power
  (the quadrant comes from the uniform's two leading bits).
"""
from __future__ import annotations

import ctypes
import hashlib
import math

import numpy as np

LN_TERMS = 9
TRIG_TERMS = 12
LN2 = float.fromhex("0x1.62e42fefa39efp-1")
HALF_PI = float.fromhex("0x1.921fb54442d18p+0")
SQRT_HALF = float.fromhex("0x1.6a09e667f3bcdp-1")
LN_COEFFS = tuple(1.0 / (2 * k + 1) for k in range(LN_TERMS))


def _taylor(first: int) -> tuple[float, ...]:
    """(-1)^k / (first + 2k)! for k = 0 .. TRIG_TERMS - 1."""
    return tuple((-1.0) ** k / math.factorial(first + 2 * k) for k in range(TRIG_TERMS))


COS_COEFFS = _taylor(0)
SIN_COEFFS = _taylor(1)


class Constants(ctypes.Structure):
    """What the device kernel is given by value, so that it evaluates the very series of this file."""

    _fields_ = [("ln", ctypes.c_double * LN_TERMS), ("cos", ctypes.c_double * TRIG_TERMS), ("sin", ctypes.c_double * TRIG_TERMS),
                ("ln2", ctypes.c_double), ("half_pi", ctypes.c_double), ("sqrt_half", ctypes.c_double)]


def constants() -> Constants:
    return Constants((ctypes.c_double * LN_TERMS)(*LN_COEFFS), (ctypes.c_double * TRIG_TERMS)(*COS_COEFFS),
                     (ctypes.c_double * TRIG_TERMS)(*SIN_COEFFS), LN2, HALF_PI, SQRT_HALF)


def tensor_key(seed: int, name: str) -> tuple[int, int]:
    """The Philox key of one tensor: 64 bits of SHA-256 over ``"<seed>:<name>"``, so that a tensor's values depend on
    the seed and on its own name only."""
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:4], "little"), int.from_bytes(digest[4:8], "little")


def philox4x32_10(counter_lo: np.ndarray, counter_hi: np.ndarray, key: tuple[int, int]) -> tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    """Philox4x32-10 of the counters (lo, hi, 0, 0), vectorised: four uint64 arrays holding 32-bit words."""
    mask = np.uint64(0xFFFFFFFF)
    c0, c1 = counter_lo.astype(np.uint64), counter_hi.astype(np.uint64)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = key
    for round_index in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        c0, c1, c2, c3 = (p1 >> np.uint64(32)) ^ c1 ^ np.uint64(k0), p1 & mask, (p0 >> np.uint64(32)) ^ c3 ^ np.uint64(k1), p0 & mask
        if round_index < 9:
            k0, k1 = (k0 + 0x9E3779B9) & 0xFFFFFFFF, (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return c0, c1, c2, c3


def _series(x2: np.ndarray, coeffs) -> np.ndarray:
    """c[0] + x2 (c[1] + x2 (c[2] + ...)), one multiplication and one addition per term, innermost first."""
    acc = np.full_like(x2, coeffs[-1])
    for c in reversed(coeffs[:-1]):
        acc = acc * x2 + c  # numpy rounds the product, then the sum: nothing is fused
    return acc


def standard_normal_pairs(first_pair: int, pairs: int, key: tuple[int, int]) -> tuple[np.ndarray, np.ndarray]:
    """The cosine and sine branches (float64) for the counters first_pair .. first_pair + pairs - 1."""
    counters = np.arange(first_pair, first_pair + pairs, dtype=np.uint64)
    w0, w1, _, _ = philox4x32_10(counters & np.uint64(0xFFFFFFFF), counters >> np.uint64(32), key)
    # u1 = (w0 + 1/2) / 2^32 in (0, 1): never 0, so its logarithm is finite
    u1 = (w0.astype(np.float64) + 0.5) * 2.0 ** -32
    m, e = np.frexp(u1)  # u1 = m 2^e with m in [1/2, 1): exact
    low = m < SQRT_HALF
    m = np.where(low, m * 2.0, m)
    e = np.where(low, e - 1, e).astype(np.float64)
    s = (m - 1.0) / (m + 1.0)
    log_u1 = e * LN2 + (2.0 * s) * _series(s * s, LN_COEFFS)
    radius = np.sqrt(-2.0 * log_u1)
    # the angle 2 pi w1 / 2^32 = (quadrant + r) pi / 2 with r in [0, 1)
    quadrant = (w1 >> np.uint64(30)).astype(np.int64)
    r = (w1 & np.uint64(0x3FFFFFFF)).astype(np.float64) * 2.0 ** -30
    phi = r * HALF_PI
    phi2 = phi * phi
    c = _series(phi2, COS_COEFFS)
    sn = phi * _series(phi2, SIN_COEFFS)
    cos_t = np.where(quadrant == 0, c, np.where(quadrant == 1, -sn, np.where(quadrant == 2, -c, sn)))
    sin_t = np.where(quadrant == 0, sn, np.where(quadrant == 1, c, np.where(quadrant == 2, -sn, -c)))
    return radius * cos_t, radius * sin_t


def normal_float32(count: int, key: tuple[int, int], std: float, mean: float = 0.0, chunk: int = 1 << 14) -> np.ndarray:
    """``count`` values mean + std z, z standard normal, rounded once from float64 to float32 (in chunks of pairs that stay
    in the processor's cache: the intermediate arrays are many)."""
    out = np.empty(count, dtype=np.float32)
    std64, mean64 = np.float64(std), np.float64(mean)
    for start in range(0, count, 2 * chunk):
        n = min(2 * chunk, count - start)
        z0, z1 = standard_normal_pairs(start // 2, (n + 1) // 2, key)
        both = np.empty(2 * len(z0), dtype=np.float64)
        both[0::2], both[1::2] = z0, z1
        out[start : start + n] = (both[:n] * std64 + mean64).astype(np.float32)
    return out
