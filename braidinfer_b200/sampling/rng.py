"""Uniform numbers for sampling, from a counter: the draw for (seed, sequence, step)
does not depend on what else is in the batch or on the order of the batch.  (The
reference seeds one generator per call and draws in step order,
crates/braidinfer-runtime/src/sampling.rs:188-191; its generator is not reproduced.)"""
from __future__ import annotations

import os

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, sequence: int, step: int) -> float:
    """A float32-exact number in (0, 1) for this (seed, sequence, step).  It is never 0:
    the inverse CDF takes the first index whose cumulative sum reaches u, and u = 0
    would pick index 0 even when its probability is zero."""
    x = _splitmix64(seed & _MASK)
    x = _splitmix64(x ^ ((sequence + 1) * 0xD6E8FEB86659FD93 & _MASK))
    x = _splitmix64(x ^ ((step + 1) * 0xCA5A826395121157 & _MASK))
    return ((x >> 41) * 2 + 1) / float(1 << 24)


def entropy_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")
