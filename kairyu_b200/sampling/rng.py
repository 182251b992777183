"""Seeds of the stateless sampler (kairyu/engine/core/sampling_types.py:17-31).

A draw depends on (base seed, output position, vocabulary index) only, so it
is the same in any batch and on any replay."""

from __future__ import annotations

import hashlib

MASK64 = (1 << 64) - 1
_SEED_BITS = (1 << 63) - 1


def stable_request_seed(request_id: str) -> int:
    return int.from_bytes(hashlib.sha256(str(request_id).encode()).digest()[:8], "big") & _SEED_BITS


def mix_seed(base: int, position: int) -> int:
    """SplitMix64 of (base, position): the per-position seed, unsigned 64-bit."""
    x = (base ^ ((position + 1) * 0x9E3779B97F4A7C15)) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    return (x ^ (x >> 31)) & MASK64


def as_signed64(value: int) -> int:
    value &= MASK64
    return value if value < (1 << 63) else value - (1 << 64)
