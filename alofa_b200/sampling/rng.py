"""SplitMix64, the reference's bit source (src/alofa/core/rng.mojo:37-78):
the state advances by an odd constant before every draw, the draw is two
xor-shift-multiply rounds and one xor-shift, and a uniform number in [0, 1) is
the top 53 bits times 2^-53.  Every request owns one, so a request draws the
same sequence whether it runs alone or in a batch
(src/alofa/serve.mojo:176-179, 704-726)."""
from __future__ import annotations

_MASK = (1 << 64) - 1
_GAMMA = 0x9E3779B97F4A7C15
_MIX1 = 0xBF58476D1CE4E5B9
_MIX2 = 0x94D049BB133111EB
_SCALE = 1.1102230246251565e-16  # 2^-53


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + _GAMMA) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * _MIX1) & _MASK
        z = ((z ^ (z >> 27)) * _MIX2) & _MASK
        return z ^ (z >> 31)

    def next_uniform(self) -> float:
        return (self.next_u64() >> 11) * _SCALE
