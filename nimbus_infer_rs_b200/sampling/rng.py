"""xoshiro256++ seeded through splitmix64, as the reference's ``Rng`` (src/sampler.rs:41-78).
One generator per sequence, so a sequence's draws do not depend on its batch-mates."""
from __future__ import annotations

_M = (1 << 64) - 1


def _rotl(x: int, k: int) -> int:
    return ((x << k) | (x >> (64 - k))) & _M


class Xoshiro256pp:
    def __init__(self, seed: int):
        sm = (int(seed) + 0x9E3779B97F4A7C15) & _M
        state = []
        for _ in range(4):
            sm = (sm + 0x9E3779B97F4A7C15) & _M
            z = sm
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
            state.append(z ^ (z >> 31))
        self.s = state

    def next_u64(self) -> int:
        s = self.s
        result = (_rotl((s[0] + s[3]) & _M, 23) + s[0]) & _M
        t = (s[1] << 17) & _M
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl(s[3], 45)
        return result

    def next_f64(self) -> float:
        """Uniform in [0, 1): the top 53 bits times 2**-53 (src/sampler.rs:75-77)."""
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))


def sequence_seed(seed: int, seq_index: int) -> int:
    """The seed of sequence ``seq_index`` of a request list.  Sequence 0 uses ``seed`` itself,
    so a single prompt draws exactly as the reference does."""
    return (int(seed) + 0x9E3779B97F4A7C15 * int(seq_index)) & _M
