"""xoshiro256** seeded through splitmix64: one stream per request, one ``next_f64`` per sampled
token, never advanced by greedy decoding (crates/engine/decode/src/rng.rs:14-52)."""
from __future__ import annotations

_M = (1 << 64) - 1


def _rotl(x: int, k: int) -> int:
    return ((x << k) | (x >> (64 - k))) & _M


class Xoshiro256StarStar:
    __slots__ = ("s",)

    def __init__(self, seed: int):
        state = seed & _M
        s = []
        for _ in range(4):
            state = (state + 0x9E3779B97F4A7C15) & _M
            z = state
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
            s.append(z ^ (z >> 31))
        self.s = s

    def next_u64(self) -> int:
        s = self.s
        result = (_rotl((s[1] * 5) & _M, 7) * 9) & _M
        t = (s[1] << 17) & _M
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl(s[3], 45)
        return result

    def next_f64(self) -> float:
        """Uniform in [0, 1) from the top 53 bits."""
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))
