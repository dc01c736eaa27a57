"""Normal variates from a counter-based generator, bit for bit the same on the host and on the GPU.

Element i of a tensor keyed (k0, k1) comes from Philox4x32-10 at counter i // 4: the four output
words make two Box-Muller pairs, (w0, w1) for elements 4c and 4c + 1 and (w2, w3) for 4c + 2 and
4c + 3.  Of a pair (a, b): u1 = (a + 1) / 2^32 in (0, 1], the angle is b / 2^32 of a turn;
z_cos = sqrt(-2 ln u1) cos(angle), z_sin = sqrt(-2 ln u1) sin(angle).  The logarithm, sine and
cosine are polynomials evaluated in float64 with separately rounded multiplications and additions
(no fused multiply-add, no library call), square root and division are the IEEE ones: every step
has one correct result, so numpy here and csrc/random_init.cu on the device produce the same bits.
The float64 variate is rounded to float32, scaled (and shifted) in float32, then rounded to the
storage type.

integrallis/models' seeded test model draws from java.util.Random in tensor order
(models-test/.../NanoGgufModel.java:42-49,91); keyed counters make every tensor reproducible on
its own instead, on either side.
"""

from __future__ import annotations

import hashlib
import math
from typing import Tuple

import numpy as np

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_SHIFT = np.uint64(32)

LN2 = math.log(2.0)
QUARTER_PI = math.pi / 4.0
SQRT_HALF = math.sqrt(0.5)
# ln(m) = 2 t (1 + t^2/3 + t^4/5 + ... + t^14/15), t = (m - 1) / (m + 1), |t| <= 0.1716
LOG_TERMS = tuple(1.0 / n for n in (15, 13, 11, 9, 7, 5, 3))
# sin x = x (1 - x^2/3! + ... - x^14/15!), cos x = 1 - x^2/2! + ... + x^16/16!, 0 <= x <= pi/4
SIN_TERMS = tuple((-1.0) ** (n // 2) / math.factorial(n) for n in (15, 13, 11, 9, 7, 5, 3))
COS_TERMS = tuple((-1.0) ** (n // 2) / math.factorial(n) for n in (16, 14, 12, 10, 8, 6, 4, 2))

CHUNK = 1 << 20  # counters per pass: bounds the scratch of a large tensor


def tensor_key(seed: int, name: str) -> Tuple[int, int]:
    """The Philox key of a tensor: 64 bits of SHA-256 over "<seed>:<name>", as two 32-bit words."""
    digest = hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:4], "little"), int.from_bytes(digest[4:8], "little")


def philox_words(counters: np.ndarray, key: Tuple[int, int]):
    """Philox4x32-10 of the 64-bit counters (the upper two counter words are zero): four uint32 arrays."""
    c0, c1 = counters & _MASK, counters >> _SHIFT
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = key[0] & 0xFFFFFFFF, key[1] & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> _SHIFT) ^ c1 ^ np.uint64(k0)) & _MASK, p1 & _MASK, ((p0 >> _SHIFT) ^ c3 ^ np.uint64(k1)) & _MASK, p0 & _MASK
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def _horner(x2: np.ndarray, terms) -> np.ndarray:
    s = np.full_like(x2, terms[0])
    for c in terms[1:]:
        s = s * x2
        s = s + c
    return s


def box_muller(a: np.ndarray, b: np.ndarray):
    """(z_cos, z_sin) in float64 from two arrays of 32-bit words (held in uint64)."""
    n = (a + np.uint64(1)).astype(np.float64)  # 1 ... 2^32, exact
    m, e = np.frexp(n)  # n = m 2^e, m in [0.5, 1)
    low = m < SQRT_HALF
    m = np.where(low, m * 2.0, m)
    e = (e - low.astype(e.dtype) - 32).astype(np.float64)
    t = (m - 1.0) / (m + 1.0)
    t2 = t * t
    series = _horner(t2, LOG_TERMS) * t2 + 1.0
    log_u = e * LN2 + (2.0 * t) * series
    radius = np.sqrt(-2.0 * log_u)
    octant = (b >> np.uint64(29)).astype(np.int64)
    fraction = (b & np.uint64(0x1FFFFFFF)).astype(np.float64) * (1.0 / (1 << 29))
    odd = (octant & 1) == 1
    x = np.where(odd, 1.0 - fraction, fraction) * QUARTER_PI
    x2 = x * x
    sin_x = (_horner(x2, SIN_TERMS) * x2 + 1.0) * x
    cos_x = _horner(x2, COS_TERMS) * x2 + 1.0
    # octants 1, 2, 5, 6 swap the two; the signs follow the quadrant
    swap = ((octant + 1) & 2) != 0
    cos_t = np.where(swap, sin_x, cos_x)
    sin_t = np.where(swap, cos_x, sin_x)
    cos_t = np.where((octant >= 2) & (octant <= 5), -cos_t, cos_t)
    sin_t = np.where(octant >= 4, -sin_t, sin_t)
    return radius * cos_t, radius * sin_t


def normal_float32(count: int, key: Tuple[int, int], mean: float, std: float) -> np.ndarray:
    """`count` values mean + std * z as float32 (z rounded to float32 first, then one multiplication and,
    if mean is not 0, one addition, each rounded to float32)."""
    out = np.empty(-(-count // 4) * 4, dtype=np.float32)
    blocks = out.size // 4
    view = out.reshape(blocks, 4)
    std32, mean32 = np.float32(std), np.float32(mean)
    for first in range(0, blocks, CHUNK):
        counters = np.arange(first, min(blocks, first + CHUNK), dtype=np.uint64)
        w0, w1, w2, w3 = philox_words(counters, key)
        for column, (a, b) in ((0, (w0, w1)), (2, (w2, w3))):
            z_cos, z_sin = box_muller(a, b)
            for offset, z in ((0, z_cos), (1, z_sin)):
                value = z.astype(np.float32) * std32
                if mean != 0.0:
                    value = value + mean32
                view[first:first + counters.size, column + offset] = value
    return out[:count]
