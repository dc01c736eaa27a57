"""Philox4x32-10 on the host, the twin of the device generator in csrc/sampling.cu: the uniform
of draw `counter` of a request seeded `seed` is the top 24 bits of the first output word, scaled by
2^-24 (24 random bits, as java.util.Random.nextFloat() has)."""

from __future__ import annotations

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32(counter: int, seed: int):
    c = [counter & _MASK, (counter >> 32) & _MASK, 0, 0]
    k = [seed & _MASK, (seed >> 32) & _MASK]
    for _ in range(10):
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c[3] ^ k[1]) & _MASK, p0 & _MASK]
        k = [(k[0] + _W0) & _MASK, (k[1] + _W1) & _MASK]
    return c


def uniform(seed: int, counter: int) -> float:
    return (philox4x32(counter, seed)[0] >> 8) / 16777216.0
