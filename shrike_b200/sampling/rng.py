"""The counter-based random numbers that sampling uses, on the host.

A draw is a function of (seed, index) only: a 64-bit mix of the two, its top 24
bits turned into a uniform number strictly inside (0, 1), then -log(-log(u)).  The
sampling kernel computes the same function on the device; this copy exists so
tests can predict a sampled token exactly.  Azimml/shrike draws from torch's
global generator instead (shrike/engine/sampler.py:29), which makes a request's
tokens depend on what else is in the batch.
"""

from __future__ import annotations

import numpy as np

_MASK = (1 << 64) - 1


def mix64(x: np.ndarray) -> np.ndarray:
    """The finaliser of MurmurHash3 on 64-bit words."""
    x = x.astype(np.uint64)
    x ^= x >> np.uint64(33)
    x *= np.uint64(0xFF51AFD7ED558CCD)
    x ^= x >> np.uint64(33)
    x *= np.uint64(0xC4CEB9FE1A85EC53)
    x ^= x >> np.uint64(33)
    return x


def uniform_host(seed: int, count: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        index = np.arange(count, dtype=np.uint64)
        word = mix64(np.uint64(seed & _MASK) + index * np.uint64(0x9E3779B97F4A7C15))
    return ((word >> np.uint64(40)).astype(np.float64) + 0.5) * (1.0 / (1 << 24))


def gumbel_noise_host(seed: int, count: int) -> np.ndarray:
    u = uniform_host(seed, count).astype(np.float32)
    return -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)


def _mix64_int(x: int) -> int:
    x &= _MASK
    x ^= x >> 33
    x = (x * 0xFF51AFD7ED558CCD) & _MASK
    x ^= x >> 33
    x = (x * 0xC4CEB9FE1A85EC53) & _MASK
    x ^= x >> 33
    return x


def step_seed(request_seed: int, position: int) -> int:
    """The seed of the draw that picks the token at `position` of a request."""
    return _mix64_int(request_seed * 0xD1342543DE82EF95 + position) & 0x7FFFFFFFFFFFFFFF
