"""`java.util.Random`'s generator, as far as text generation needs it: the draws behind
`TextGenerator`'s categorical sample (models/TextGenerator.java:77, 143).  48-bit linear
congruential state, `next(bits)` = the top bits after one step, `nextFloat()` = next(24) / 2^24
(Java SE API, general contract of java.util.Random)."""
from __future__ import annotations

_MASK = (1 << 48) - 1
_MULT = 0x5DEECE66D


class JavaRandom:
    def __init__(self, seed: int):
        self.state = (int(seed) ^ _MULT) & _MASK

    def next(self, bits: int) -> int:
        self.state = (self.state * _MULT + 0xB) & _MASK
        r = self.state >> (48 - bits)
        return r - (1 << 32) if r >= (1 << 31) else r

    def next_float(self) -> float:
        return self.next(24) / float(1 << 24)

    def next_int(self, bound: int) -> int:
        if bound <= 0:
            raise ValueError("bound must be positive")
        r = self.next(31)
        m = bound - 1
        if (bound & m) == 0:
            return (bound * r) >> 31
        u = r
        while True:
            r = u % bound
            if u - r + m < (1 << 31):
                return r
            u = self.next(31)
