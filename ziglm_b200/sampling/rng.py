"""The uniform number behind a draw: a pure function of (seed, counter).

The device kernel computes the same integers (``mix64`` in csrc/sampling.cu), so a
test can state which number a draw used.  The reference seeds one generator per
engine (src/sampler.zig:21); a counter-based number per (request, step) instead
lets a sequence draw the same whatever else is in its batch.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1


def mix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform01(seed: int, counter: int) -> float:
    """24 random bits scaled to [0, 1)."""
    h = mix64((seed & _MASK) ^ mix64(counter & _MASK))
    return (h >> 40) / 16777216.0


def request_seed(seed: int, request: int) -> int:
    """The seed of one request of a ``generate`` call."""
    return mix64((seed & _MASK) ^ mix64(0x5EED0000 + request)) & 0x7FFFFFFFFFFFFFFF
