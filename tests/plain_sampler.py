"""The reference's sampler in plain Python: floats (f64, which is what src/sampler.rs computes
in) and loops, one function for each of its steps, each citing the lines it restates.  It
shares no code with the library (`nimbus_infer_rs_b200/sampling/`), which does the same with
numpy arrays on the host and with kernels on the device; the tests compare the two draw for
draw.  The reference is Rust and cannot be compiled here, so this file rests on its formulas.
"""
import math

import numpy as np

MASK = (1 << 64) - 1
NEG_INF = float("-inf")


def _rotl(x: int, k: int) -> int:
    return ((x << k) | (x >> (64 - k))) & MASK


class PlainRng:
    """xoshiro256++ seeded through splitmix64 (src/sampler.rs:40-78)."""

    def __init__(self, seed: int):
        self.sm = (seed + 0x9E3779B97F4A7C15) & MASK         # src/sampler.rs:47
        self.s = [self._splitmix() for _ in range(4)]

    def _splitmix(self) -> int:                              # src/sampler.rs:48-54
        self.sm = (self.sm + 0x9E3779B97F4A7C15) & MASK
        z = self.sm
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
        return z ^ (z >> 31)

    def next_u64(self) -> int:                               # src/sampler.rs:58-72
        s = self.s
        result = (_rotl((s[0] + s[3]) & MASK, 23) + s[0]) & MASK
        t = (s[1] << 17) & MASK
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = _rotl(s[3], 45)
        return result

    def next_f64(self) -> float:                             # src/sampler.rs:75-77
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))


def widen(x) -> float:
    """A 32-bit option or logit as the f64 the reference computes with (`as f64`)."""
    return float(np.float32(x))


def repetition_penalty(work: list, generated, penalty: float) -> None:
    """src/sampler.rs:83-101: every distinct generated token once; a positive logit is divided
    by the penalty, any other multiplied."""
    if penalty == 1.0 or len(generated) == 0:
        return
    for tok in sorted(set(int(t) for t in generated)):
        if tok >= len(work):
            continue
        if work[tok] > 0.0:
            work[tok] = work[tok] / penalty
        else:
            work[tok] = work[tok] * penalty


def top_k(work: list, k: int) -> None:
    """src/sampler.rs:103-116: everything below the k-th largest value goes to -inf (values
    equal to it stay, so more than k may be kept)."""
    if k == 0 or k >= len(work):
        return
    kth = sorted(work, reverse=True)[k - 1]
    for i in range(len(work)):
        if work[i] < kth:
            work[i] = NEG_INF


def top_p(work: list, p: float) -> None:
    """src/sampler.rs:118-160.  p <= 0 keeps one maximum, the last of equal ones (Rust's
    `max_by`).  Otherwise, in descending order (equal values in index order: a stable sort)
    with softmax probabilities, a token is dropped once the mass of the tokens before it,
    less its own probability, exceeds p."""
    if p >= 1.0:
        return
    n = len(work)
    if p <= 0.0:
        best = 0
        for i in range(1, n):
            if work[i] >= work[best]:
                best = i
        keep = work[best]
        for i in range(n):
            work[i] = NEG_INF
        work[best] = keep
        return
    order = sorted(range(n), key=lambda i: -work[i])          # sorted() is stable
    top = work[order[0]]
    probs = [math.exp(work[i] - top) for i in order]
    total = 0.0
    for v in probs:
        total += v
    probs = [v / total for v in probs]
    cum = 0.0
    remove = []
    for pos, i in enumerate(order):
        if cum - probs[pos] > p:
            remove.append(i)
        cum += probs[pos]
    for i in remove:
        work[i] = NEG_INF


def first_max(work: list) -> int:
    """src/sampler.rs:173-179: the first index of the maximum."""
    best = 0
    for i in range(len(work)):
        if work[i] > work[best]:
            best = i
    return best


def sample(logits, temperature, top_k_n, top_p_mass, penalty, generated, rng: PlainRng,
           report: dict | None = None) -> int:
    """src/sampler.rs:163-217.  `report`, if given, receives `margin`: how far the number drawn
    lay from the nearest edge between two tokens, as a fraction of the whole (a comparison
    with another implementation means nothing closer than rounding to such an edge)."""
    work = [widen(v) for v in logits]
    repetition_penalty(work, generated, widen(penalty))
    if widen(temperature) <= 0.0:                             # src/sampler.rs:31-35
        return first_max(work)
    temp = max(widen(temperature), 1e-6)
    work = [v / temp for v in work]
    top_k(work, top_k_n)
    top_p(work, widen(top_p_mass))
    mx = NEG_INF
    for v in work:                                            # f64::max skips a NaN
        if v > mx:
            mx = v
    if not math.isfinite(mx):
        return first_max(work)                                # nothing is drawn
    total = 0.0
    for i in range(len(work)):
        work[i] = math.exp(work[i] - mx) if work[i] == work[i] else float("nan")
        total += work[i]
    if not math.isfinite(total) or total <= 0.0:
        return 0
    r = rng.next_f64() * total
    if report is not None:
        edge, margin = 0.0, 1.0
        for v in work:
            edge += v
            margin = min(margin, abs(r - edge) / total)
        report["margin"] = margin
    for i, v in enumerate(work):
        r -= v
        if r <= 0.0:
            return i
    return len(work) - 1
