"""The reference's sampler restated on the host in float64 (src/sampler.rs:163-217): the
path taken when top-k or top-p filtering is on, and the yardstick of the device kernels.

Where it parts from the reference, all in degenerate rows: a row with a NaN gives the first
index of the maximum as numpy sees it (the reference's ``fold(f64::max)`` ignores the NaN and
returns token 0 once the total is not finite); with ``top_p <= 0`` the first of tied maxima is
kept (Rust's ``max_by`` keeps the last); and the callers draw a number for every row and
step, while the reference draws none when it falls back to the argmax of a row without a
finite maximum, so after such a row the two random streams differ."""
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


def sample_from_candidates(vals, idx, count: int, row_max: float, row_sum: float,
                           params: SamplingParams, rng: Xoshiro256pp, n_keep: int,
                           vocab: int | None = None, gen_idx=None, gen_vals=None) -> int | None:
    """The same decision as :func:`sample` from the largest logits of a row only: ``vals`` /
    ``idx`` hold every logit that is not smaller than the ``n_keep``-th largest, ``row_sum`` is
    the f64 sum of ``exp((x - max) / temp)`` over the whole row.  With a repetition penalty,
    ``gen_idx`` / ``gen_vals`` are the distinct generated tokens and their logits (wherever
    they rank).  Both filters only ever keep the largest values, and every token that is not
    known here has a value below the smallest candidate's, so the known ones decide as long as
    the cut falls above that bound; returns ``None`` (the caller then takes the whole row)
    when it does not, or when the row is not plain numbers.  Nothing is drawn from ``rng`` in
    that case."""
    if count <= 0 or count > len(vals) or not np.isfinite(row_max) or not np.isfinite(row_sum):
        return None
    temp = max(float(np.float32(params.temperature)), 1e-6)
    k, p = params.top_k, float(np.float32(params.top_p))
    penalty = float(np.float32(params.repetition_penalty))
    if (k == 0 and p >= 1.0) or k > n_keep:
        return None
    raw = np.asarray(vals[:count], dtype=np.float64)
    idx = np.asarray(idx[:count], dtype=np.int64)
    # every token not listed has a logit below `bound` (none, if the whole row is listed)
    whole_listed = vocab is not None and count >= vocab
    bound = -np.inf if (count < n_keep or whole_listed) else float(raw.min())
    correction = 0.0                                   # what the penalty changes in row_sum
    if penalty != 1.0 and gen_idx is not None and len(gen_idx) > 0:
        g_idx = np.asarray(gen_idx, dtype=np.int64)
        g_raw = np.asarray(gen_vals, dtype=np.float64)
        if not np.isfinite(g_raw).all():
            return None
        extra = ~np.isin(g_idx, idx)                   # generated tokens outside the candidates
        raw = np.concatenate([raw, g_raw[extra]])
        idx = np.concatenate([idx, g_idx[extra]])
        work = raw.copy()
        hit = np.isin(idx, g_idx)                      # src/sampler.rs:83-101
        work[hit] = np.where(work[hit] > 0.0, work[hit] / penalty, work[hit] * penalty)
    else:
        work = raw.copy()
        hit = np.zeros(raw.shape[0], dtype=bool)
    work /= temp
    bound_t = bound / temp
    order = np.lexsort((idx, -work))                   # descending value, ties by index: stable argsort
    work, idx, raw, hit = work[order], idx[order], raw[order], hit[order]
    if not work[0] >= bound_t:
        return None                                    # an unknown token could be the largest
    # only the tokens at or above the bound are surely the row's largest, in this order
    sure = int(np.searchsorted(-work, -bound_t, side="right"))
    keep = np.zeros(work.shape[0], dtype=bool)
    keep[:sure] = True
    whole_row = True                                   # the survivors are still the whole row
    if k > 0:
        if k > sure:
            return None
        keep &= work >= work[k - 1]                    # src/sampler.rs:103-116
        whole_row = False
    if p < 1.0:
        if p <= 0.0:
            keep[:] = False
            keep[0] = True
            whole_row = False
        else:
            probs = np.where(keep, np.exp(work - work[0]), 0.0)
            if whole_row:
                # the whole row's denominator, from the unpenalised one
                total = row_sum * np.exp(row_max / temp - work[0])
                if hit.any():
                    total += float(np.sum(np.exp(work[hit] - work[0]) - np.exp(raw[hit] / temp - work[0])))
            else:
                total = probs.sum()
            probs = probs / total
            cum_before = np.concatenate([[0.0], np.cumsum(probs)[:-1]])
            remove = (cum_before - probs) > p          # src/sampler.rs:118-160
            if whole_row and not remove[:sure].any():
                return None                            # the cut lies beyond the known tokens
            keep &= ~remove
            whole_row = False
    if whole_row:
        return None
    work, idx = work[keep], idx[keep]
    by_index = np.argsort(idx, kind="stable")          # the draw walks the tokens in index order
    work, idx = work[by_index], idx[by_index]
    e = np.exp(work - np.max(work))
    total = float(np.sum(e))
    if not np.isfinite(total) or total <= 0.0:
        return None
    r = rng.next_f64() * total
    pos = int(np.searchsorted(np.cumsum(e), r, side="left"))
    return int(idx[min(pos, idx.shape[0] - 1)])


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
