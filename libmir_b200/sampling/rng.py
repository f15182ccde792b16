"""SplitMix64, the generator libmir's sampler draws from (runtime/src/sampling/mod.rs:180-203).

One generator per request, seeded by the request's seed; one uniform draw in [0, 1) per sampled
token, made on the host and passed to the sampling kernel, so a request's tokens do not depend on
what else is in the batch.
"""

from __future__ import annotations

_MASK = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        value = self.state
        value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK
        return value ^ (value >> 31)

    def next_unit(self) -> float:
        """The upper 32 bits as a fraction of 2^32."""
        return (self.next_u64() >> 32) / 4294967296.0
