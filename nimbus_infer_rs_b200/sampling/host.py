"""The reference's sampler restated on the host in float64 (src/sampler.rs:163-217): the
path taken when top-k or top-p filtering is on, and the yardstick of the device kernels."""
from __future__ import annotations

import numpy as np

from .params import SamplingParams
from .rng import Xoshiro256pp


def apply_repetition_penalty(logits: np.ndarray, generated, penalty: float) -> None:
    """src/sampler.rs:83-101: each distinct generated token once; positive logits are divided,
    others multiplied."""
    if penalty == 1.0 or len(generated) == 0:
        return
    for tok in sorted(set(int(t) for t in generated)):
        if tok >= logits.shape[0]:
            continue
        if logits[tok] > 0.0:
            logits[tok] /= penalty
        else:
            logits[tok] *= penalty


def top_k_filter(logits: np.ndarray, k: int) -> None:
    """src/sampler.rs:103-116: keep everything >= the k-th largest value."""
    if k == 0 or k >= logits.shape[0]:
        return
    kth = np.sort(logits)[::-1][k - 1]
    logits[logits < kth] = -np.inf


def top_p_filter(logits: np.ndarray, p: float) -> None:
    """src/sampler.rs:118-160.  In descending order, with softmax probabilities, a token is
    dropped when ``cum - prob > p`` where ``cum`` is the mass of the tokens before it."""
    if p >= 1.0:
        return
    if p <= 0.0:
        best = _first_argmax(logits)
        keep = logits[best]
        logits[:] = -np.inf
        logits[best] = keep
        return
    order = np.argsort(-logits, kind="stable")
    srt = logits[order]
    probs = np.exp(srt - srt[0])
    probs /= probs.sum()
    cum_before = np.concatenate([[0.0], np.cumsum(probs)[:-1]])
    remove = (cum_before - probs) > p
    logits[order[remove]] = -np.inf


def _first_argmax(work: np.ndarray) -> int:
    """First index of the maximum; NaN never wins (src/sampler.rs:173-179)."""
    best = 0
    bv = work[0]
    for i in range(1, work.shape[0]):
        if work[i] > bv:
            best, bv = i, work[i]
    return best


def first_argmax(work: np.ndarray) -> int:
    if not np.isnan(work).any():
        return int(np.argmax(work))
    return _first_argmax(work)


def sample(logits, params: SamplingParams, generated, rng: Xoshiro256pp) -> int:
    work = np.asarray(logits, dtype=np.float64).copy()
    apply_repetition_penalty(work, generated, float(np.float32(params.repetition_penalty)))
    if params.greedy:
        return first_argmax(work)
    temp = max(float(np.float32(params.temperature)), 1e-6)
    work /= temp
    top_k_filter(work, params.top_k)
    top_p_filter(work, float(np.float32(params.top_p)))
    mx = np.max(work) if not np.isnan(work).all() else np.nan
    if not np.isfinite(mx):
        return first_argmax(work)
    e = np.exp(work - mx)
    total = float(np.sum(e))
    if not np.isfinite(total) or total <= 0.0:
        return 0
    r = rng.next_f64() * total
    # walk the cumulative sum in index order (src/sampler.rs:208-215)
    c = np.cumsum(e)
    idx = int(np.searchsorted(c, r, side="left"))
    # cumsum rounding may differ from the sequential subtraction by an ulp; settle locally
    idx = min(idx, work.shape[0] - 1)
    return idx
