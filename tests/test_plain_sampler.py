"""The library's sampler on the host (numpy, `sampling/host.py`: the yardstick of the sampling
kernels and the one that settles the rows they hand back) against the plain restatement of
src/sampler.rs in `tests/plain_sampler.py`: the same random numbers, the same filters, the same
token for the same draw.  Where the library parts from the reference on purpose (rows with a
NaN, tied maxima with top_p <= 0) the test says what each of the two does."""
import itertools

import numpy as np
import pytest

import plain_sampler as P
from nimbus_infer_rs_b200.sampling import SamplingParams
from nimbus_infer_rs_b200.sampling import host as H
from nimbus_infer_rs_b200.sampling.rng import Xoshiro256pp

EDGE = 1e-12          # a draw closer than this to the edge between two tokens decides nothing


@pytest.mark.parametrize("seed", [0, 1, 42, 2 ** 63, 2 ** 64 - 1])
def test_random_numbers(seed):
    a, b = P.PlainRng(seed), Xoshiro256pp(seed)
    for _ in range(300):
        assert a.next_f64() == b.next_f64()


def _rows(rng, vocab, n):
    """Rows of three kinds: smooth, with many equal values, with tokens that cannot be drawn."""
    for i in range(n):
        x = rng.standard_normal(vocab).astype(np.float32) * np.float32(3.0)
        if i % 3 == 1:
            x = np.round(x)                                   # ties, also at the cuts
        if i % 3 == 2:
            x[rng.integers(0, vocab, size=max(1, vocab // 4))] = -np.inf
        yield x


@pytest.mark.parametrize("vocab", [7, 50, 513])
def test_filters_one_by_one(vocab):
    rng = np.random.default_rng(vocab)
    for x in _rows(rng, vocab, 12):
        for k in (0, 1, 3, vocab - 1, vocab, vocab + 5):
            a, b = [float(v) for v in x], x.astype(np.float64)
            P.top_k(a, k)
            H.top_k_filter(b, k)
            assert a == b.tolist()
        for p in (1.0, 0.95, 0.5, 0.1, 1e-4):
            a, b = [float(v) for v in x], x.astype(np.float64)
            P.top_p(a, p)
            H.top_p_filter(b, p)
            assert a == b.tolist(), (p, x)
        gen = [int(t) for t in rng.integers(0, vocab + 3, size=9)] + [0, 0]   # repeats, ids beyond the row
        for pen in (1.0, 1.3, 0.7):
            a, b = [float(v) for v in x], x.astype(np.float64)
            P.repetition_penalty(a, gen, P.widen(pen))
            H.apply_repetition_penalty(b, gen, float(np.float32(pen)))
            assert a == b.tolist()


@pytest.mark.parametrize("vocab", [7, 50, 513])
def test_the_same_token_for_the_same_draw(vocab):
    rng = np.random.default_rng(100 + vocab)
    compared = skipped = 0
    grid = itertools.product((0.0, 0.7, 1.0, 1.6), (0, 1, 5, 40), (1.0, 0.9, 0.4, 0.0), (1.0, 1.3))
    for n, (temp, k, p, pen) in enumerate(grid):
        params = SamplingParams(temperature=temp, top_k=k, top_p=p, repetition_penalty=pen, seed=n)
        a, b = P.PlainRng(n), Xoshiro256pp(n)
        generated = []
        for x in _rows(rng, vocab, 6):
            if p <= 0.0 and temp > 0.0 and np.sum(x == x.max()) > 1:
                continue                                      # tied maxima: see the test below
            report = {}
            want = P.sample(x, temp, k, p, pen, generated, a, report)
            got = H.sample(x, params, generated, b)
            if report.get("margin", 1.0) < EDGE:
                skipped += 1
            else:
                assert got == want, (temp, k, p, pen, x)
                compared += 1
            generated.append(want)
        assert a.next_u64() == b.next_u64()                   # as many numbers drawn by both
    assert compared > 500 and skipped < 5


def test_rows_without_a_finite_maximum():
    """src/sampler.rs:191-200: the first maximum, and no number is drawn."""
    for row in ([-np.inf] * 5, [-np.inf, -np.inf, np.inf, 1.0, np.inf]):
        x = np.array(row, dtype=np.float32)
        a, b = P.PlainRng(3), Xoshiro256pp(3)
        params = SamplingParams(temperature=0.8, seed=3)
        assert P.sample(x, 0.8, 0, 1.0, 1.0, [], a) == H.sample(x, params, [], b) == (0 if row[2] < 0 else 2)
        assert a.next_u64() == b.next_u64()


def test_where_the_library_parts_from_the_reference():
    # tied maxima with top_p <= 0: the reference keeps the last of them (Rust's max_by), the
    # library the first
    x = np.array([1.0, 5.0, 5.0, 0.0], dtype=np.float32)
    params = SamplingParams(temperature=1.0, top_p=0.0, seed=0)
    assert P.sample(x, 1.0, 0, 0.0, 1.0, [], P.PlainRng(0)) == 2
    assert H.sample(x, params, [], Xoshiro256pp(0)) == 1
    # a NaN in the row: the reference's maximum skips it, its sum does not, and it returns
    # token 0; the library returns the first maximum of the numbers
    x = np.array([0.5, np.nan, 3.0, 1.0], dtype=np.float32)
    params = SamplingParams(temperature=1.0, seed=0)
    assert P.sample(x, 1.0, 0, 1.0, 1.0, [], P.PlainRng(0)) == 0
    assert H.sample(x, params, [], Xoshiro256pp(0)) == 2
    # greedy agrees in both cases
    greedy = SamplingParams(temperature=0.0)
    for row in ([1.0, 5.0, 5.0, 0.0], [0.5, np.nan, 3.0, 1.0]):
        x = np.array(row, dtype=np.float32)
        assert P.sample(x, 0.0, 0, 1.0, 1.0, [], P.PlainRng(0)) == H.sample(x, greedy, [], Xoshiro256pp(0))
