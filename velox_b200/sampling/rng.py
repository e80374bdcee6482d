"""A counter-based source of uniform numbers for sampling.

u(seed, stream, counter) is a pure function, so a request's tokens do not depend
on which other requests share its steps or on how its prompt was cut; the kernel
gets u and draws nothing itself.  splitmix64 over the three words, top 24 bits:
every u is a multiple of 2^-24 in [0, 1) and exact in float32.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, stream: int, counter: int) -> float:
    h = _splitmix64(seed & _MASK)
    h = _splitmix64(h ^ (stream & _MASK))
    h = _splitmix64(h ^ (counter & _MASK))
    return (h >> 40) / float(1 << 24)
