import numpy as np
import pytest

from nimbus_infer_rs_b200.sampling import SamplingParams, Xoshiro256pp, sequence_seed
from nimbus_infer_rs_b200.sampling import host as H


def test_greedy_takes_first_max():            # src/sampler.rs:223-228
    p = SamplingParams(temperature=0.0)
    assert H.sample(np.array([0.1, 5.0, 5.0, -1.0], dtype=np.float32), p, [], Xoshiro256pp(0)) == 1
    assert H.sample(np.array([np.nan, 1.0, 2.0], dtype=np.float32), p, [], Xoshiro256pp(0)) == 0


def test_rng_is_deterministic_and_seeded():   # src/sampler.rs:230-239
    a, b, c = Xoshiro256pp(42), Xoshiro256pp(42), Xoshiro256pp(43)
    xs = [a.next_u64() for _ in range(100)]
    assert xs == [b.next_u64() for _ in range(100)]
    assert xs[0] != c.next_u64()
    assert all(0 <= x < 2 ** 64 for x in xs)
    u = [Xoshiro256pp(7).next_f64() for _ in range(3)]
    assert all(0.0 <= v < 1.0 for v in u)
    assert sequence_seed(5, 0) == 5 and sequence_seed(5, 1) != 5


def test_splitmix_seeding_known_value():
    # splitmix64 from state 0 gives 0xE220A8397B1DCDAF as its first output; the reference
    # advances the state once before the first draw (src/sampler.rs:47-48), so seeding with
    # -golden lands exactly there.
    r = Xoshiro256pp(-0x9E3779B97F4A7C15)
    assert r.s[0] == 0xE220A8397B1DCDAF


def test_top_k_keeps_only_best_k():           # src/sampler.rs:241-249
    x = np.array([1.0, 5.0, 3.0, 4.0])
    H.top_k_filter(x, 2)
    assert x.tolist() == [-np.inf, 5.0, -np.inf, 4.0]
    y = np.array([1.0, 2.0])
    H.top_k_filter(y, 0)
    H.top_k_filter(y, 5)
    assert y.tolist() == [1.0, 2.0]


def test_repetition_penalty_signs():          # src/sampler.rs:251-257
    x = np.array([2.0, -2.0, 1.0])
    H.apply_repetition_penalty(x, [0, 1, 1, 0, 99], 2.0)
    assert x.tolist() == [1.0, -4.0, 1.0]     # each distinct token once; out of range skipped


def test_top_p():                              # src/sampler.rs:118-160, :259-266
    x = np.array([1.0, 5.0, 3.0])
    H.top_p_filter(x, 0.0)
    assert x.tolist() == [-np.inf, 5.0, -np.inf]
    # probs (desc): .6439 .2369 .0871 .0321 ; cum_before - prob: -.64 .41 .79 .94
    x = np.log(np.array([0.0871, 0.6439, 0.0321, 0.2369]))
    H.top_p_filter(x, 0.5)
    assert np.isinf(x).tolist() == [True, False, True, False]
    x = np.array([1.0, 2.0])
    H.top_p_filter(x, 1.0)
    assert x.tolist() == [1.0, 2.0]


def test_temperature_sampling_follows_the_cdf():
    logits = np.log(np.array([0.1, 0.2, 0.3, 0.4], dtype=np.float64)).astype(np.float32)
    p = SamplingParams(temperature=1.0)
    rng = Xoshiro256pp(9)
    counts = np.zeros(4)
    for _ in range(4000):
        counts[H.sample(logits, p, [], rng)] += 1
    assert np.allclose(counts / 4000, [0.1, 0.2, 0.3, 0.4], atol=0.03)
    # degenerate cases (src/sampler.rs:191-216)
    assert H.sample(np.full(5, -np.inf, dtype=np.float32), p, [], rng) == 0
    low = SamplingParams(temperature=1e-9)     # clamped to 1e-6: effectively greedy
    assert H.sample(np.array([0.0, 1.0, 0.5], dtype=np.float32), low, [], rng) == 1


def test_params_defaults_and_validation():     # src/sampler.rs:17-29
    p = SamplingParams()
    assert (p.max_new_tokens, p.temperature, p.top_k, p.top_p, p.repetition_penalty, p.seed,
            p.stop_tokens) == (64, 1.0, 0, 1.0, 1.0, None, [])
    assert not p.greedy and SamplingParams(temperature=0.0).greedy
    with pytest.raises(ValueError):
        SamplingParams(top_k=-1).validate()


def test_the_largest_logits_decide_as_the_whole_row_does():
    """top-k / top-p from a row's largest logits only (what the device hands over) must pick
    the token the whole row picks, or say that it cannot (None), never something else."""
    from nimbus_infer_rs_b200.sampling import host
    rng = np.random.default_rng(0)
    decided = 0
    for trial in range(300):
        V = int(rng.integers(40, 3000))
        logits = (rng.standard_normal(V) * float(rng.choice([0.5, 2.0, 8.0]))).astype(np.float32)
        if trial % 5 == 0:
            logits[rng.integers(0, V, 4)] = logits.max()              # ties at the top
        k = int(rng.choice([0, 1, 5, 50, 300]))
        p = float(rng.choice([1.0, 0.9, 0.5, 0.1, 0.0]))
        T = float(rng.choice([0.7, 1.0, 1.5]))
        if k == 0 and p >= 1.0:
            continue
        pen = float(rng.choice([1.0, 1.3, 0.7, 2.5]))                 # a penalty moves generated tokens
        gen = [int(t) for t in rng.integers(0, V, int(rng.integers(0, 30)))]
        if trial % 3 == 0:
            gen.append(int(np.argmax(logits)))
        params = SamplingParams(temperature=T, top_k=k, top_p=p, repetition_penalty=pen)
        n_keep = min(128, V)
        temp = max(float(np.float32(T)), 1e-6)
        thr = np.sort(logits)[::-1][n_keep - 1]
        sel = rng.permutation(np.nonzero(logits >= thr)[0])           # in any order
        cap = n_keep + 32
        vals, idx = np.zeros(cap, np.float32), np.zeros(cap, np.int32)
        vals[:min(len(sel), cap)], idx[:min(len(sel), cap)] = logits[sel][:cap], sel[:cap]
        mx = float(logits.max())
        total = float(np.sum(np.exp(logits.astype(np.float64) / temp - mx / temp)))
        whole = host.sample(logits, params, gen, Xoshiro256pp(trial))
        r = Xoshiro256pp(trial)
        g = np.array(sorted(set(gen)), dtype=np.int64)
        few = host.sample_from_candidates(vals, idx, len(sel), mx, total, params, r, n_keep, V,
                                          g if pen != 1.0 else None, logits[g] if pen != 1.0 else None)
        if few is None:
            assert r.next_f64() == Xoshiro256pp(trial).next_f64()     # nothing was drawn
        else:
            assert few == whole, (trial, V, k, p, T)
            decided += 1
    assert decided > 120
    # not plain numbers, too many ties, k beyond the candidates: the whole row has to decide
    assert host.sample_from_candidates(np.zeros(4, np.float32), np.zeros(4, np.int32), -1, 0.0, 1.0,
                                       SamplingParams(top_k=2), Xoshiro256pp(1), 4) is None
    assert host.sample_from_candidates(np.zeros(4, np.float32), np.zeros(4, np.int32), 9, 0.0, 1.0,
                                       SamplingParams(top_k=2), Xoshiro256pp(1), 4) is None
    assert host.sample_from_candidates(np.zeros(4, np.float32), np.arange(4, dtype=np.int32), 4, 0.0,
                                       4.0, SamplingParams(top_k=9), Xoshiro256pp(1), 4) is None


def test_whole_rows_sampled_side_by_side_equal_one_after_the_other():
    """Rows that the host's sampler takes whole are handed to threads; every sequence has its
    own generator and history, so the tokens must be the ones a plain loop picks, draw for
    draw and step after step."""
    import torch
    from nimbus_infer_rs_b200.sampling import BatchSampler, SequenceSampler
    params = SamplingParams(temperature=0.9, top_p=0.8, top_k=7, repetition_penalty=1.3, seed=5)
    n, vocab = 6, 301
    g = np.random.default_rng(3)
    sampler = BatchSampler(params, ops=None, device="cpu")
    seqs = [SequenceSampler(params, i) for i in range(n)]
    plain = [SequenceSampler(params, i) for i in range(n)]
    for step in range(5):
        logits = g.normal(size=(n, vocab)).astype(np.float32) * 3
        got = sampler.sample(torch.from_numpy(logits.copy()), seqs)
        want = []
        for i in range(n):
            t = H.sample(logits[i], params, plain[i].generated, plain[i].rng)
            plain[i].generated.append(int(t))
            want.append(int(t))
        assert got == want, step


def test_which_options_the_sampling_kernels_take():
    """The batch sampler asks the host only where the backend has no kernel for the options:
    top-p with a top-k beyond the kernel's room, or a backend without the sampling kernels."""
    from nimbus_infer_rs_b200.sampling import BatchSampler

    class WithKernels:
        def sample_top_k(self, *a): pass
        def sample_top_p(self, *a): pass
        def top_p_max_k(self): return 1024

    class Without:
        pass

    def needs(ops, **kw):
        return BatchSampler(SamplingParams(**kw), ops, "cpu").needs_host()
    full, bare = WithKernels(), Without()
    assert not needs(full, temperature=0.0, top_k=5, top_p=0.5)          # greedy: argmax
    assert not needs(full, temperature=0.7)
    assert not needs(full, temperature=0.7, top_k=40)
    assert not needs(full, temperature=0.7, top_p=0.9)
    assert not needs(full, temperature=0.7, top_k=1024, top_p=0.9, repetition_penalty=1.2)
    assert needs(full, temperature=0.7, top_k=1025, top_p=0.9)
    assert not needs(full, temperature=0.7, top_k=5000)                  # top-k alone: any k
    assert not needs(bare, temperature=0.7)
    assert needs(bare, temperature=0.7, top_k=40)
    assert needs(bare, temperature=0.7, top_p=0.9)
