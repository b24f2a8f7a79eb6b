"""xorshift64*, the reference's generator (`engine/src/sampling.rs:55-76`):
state = seed | 1; one step: s ^= s >> 12; s ^= s << 25; s ^= s >> 27;
u = ((s * 0x2545F4914F6CDD1D) >> 40) / 2^24.  One generator per request, so a
request's sequence does not depend on its neighbours; greedy requests draw
nothing."""
from __future__ import annotations

_MASK = (1 << 64) - 1


class Xorshift64Star:
    def __init__(self, seed: int):
        self.state = (int(seed) | 1) & _MASK

    def next_f32(self) -> float:
        s = self.state
        s ^= s >> 12
        s ^= (s << 25) & _MASK
        s ^= s >> 27
        self.state = s
        return (((s * 0x2545F4914F6CDD1D) & _MASK) >> 40) / 16777216.0
