"""Generation through the entry points (Python API, command line) against the plain
implementation's greedy loop."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_gpt2 as P
from gpu_helpers import DTYPES, assert_greedy_matches
from make_golden_lib import WORKLOADS, prompts_for
from nimbus_infer_rs_b200 import Engine, SamplingParams

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_python_entry_point(model_dirs, name, dtype):
    W = P.PlainWeights(model_dirs[name])
    e = Engine.load(model_dirs[name], dtype=dtype, cache_tokens=1024)
    key = name if name in WORKLOADS else "A"
    prompts = prompts_for(key, e.spec.vocab_size)
    n_new = WORKLOADS[key][1]
    out = e.generate(prompts, SamplingParams(max_new_tokens=n_new, temperature=0.0))
    assert [len(o) for o in out] == [n_new] * len(prompts)
    for p, o in zip(prompts, out):
        assert_greedy_matches(o, W, p, dtype)
    again = e.generate(prompts, SamplingParams(max_new_tokens=n_new, temperature=0.0))
    assert again == out                                     # tests/engine.rs:14-23
    assert e.cache.slots.n_free == e.cache.n_slots


def test_golden_greedy_ids_in_32bit(model_dirs):
    golden = json.loads((ROOT / "tests" / "golden" / "tiny_A.json").read_text())
    e = Engine.load(model_dirs["A"], dtype="float32", cache_tokens=1024)
    out = e.generate(golden["prompts"], SamplingParams(max_new_tokens=8, temperature=0.0))
    assert out == golden["greedy"]


def test_more_requests_than_slots_run_as_batches_one_after_another(model_dirs):
    W = P.PlainWeights(model_dirs["B"])
    e = Engine.load(model_dirs["B"], dtype="float32", cache_tokens=3 * 64, n_slots=3)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (1, 17, 5, 9, 13, 30, 2)]
    stop = P.greedy_generate(W, prompts[2], 10)[3]
    out = e.generate(prompts, SamplingParams(max_new_tokens=10, temperature=0.0, stop_tokens=[stop]))
    for p, o in zip(prompts, out):
        assert o == P.greedy_generate(W, p, 10, stop_tokens=(stop,))
    assert out[2][-1] == stop and len(out[2]) <= 4


def test_temperature_top_k_top_p_and_penalty_run_and_are_seeded(model_dirs):
    e = Engine.load(model_dirs["B"], dtype="float32", cache_tokens=1024)
    prompts = [[1], list(range(2, 19))]
    for kw in (dict(temperature=0.7), dict(temperature=0.7, repetition_penalty=1.3),
               dict(temperature=0.9, top_k=5), dict(temperature=0.9, top_p=0.5),
               dict(temperature=0.0, repetition_penalty=2.0)):
        p = SamplingParams(max_new_tokens=12, seed=7, **kw)
        a = e.generate(prompts, p)
        assert a == e.generate(prompts, p) and [len(x) for x in a] == [12, 12]
        assert e.generate(prompts[:1], p)[0] == a[0]       # independent of batch-mates
    k1 = e.generate(prompts, SamplingParams(max_new_tokens=12, temperature=5.0, top_k=1, seed=3))
    assert k1 == e.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0))


def _cli(*args):
    return subprocess.run([sys.executable, "-m", "nimbus_infer_rs_b200", *args], cwd=ROOT,
                          capture_output=True, text=True, timeout=600)


def test_command_line(model_dirs):
    W = P.PlainWeights(model_dirs["A"])
    r = _cli("generate", "--model", str(model_dirs["A"]), "--ids", "5,17,3", "--max-new-tokens", "6",
             "--dtype", "float32", "--json")
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout)
    assert out["prompt_tokens"] == 3 and out["generated_ids"] == P.greedy_generate(W, [5, 17, 3], 6)
    assert "tok/s]" in r.stderr
    r = _cli("generate", "--model", str(model_dirs["A"]), "--ids", "5,17,3", "--max-new-tokens", "6",
             "--dtype", "float32", "--stream")
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()     # the ids as they came, then the whole list
    assert [int(t) for t in lines[0].split()] == out["generated_ids"]
    assert json.loads(lines[1]) == out["generated_ids"]
    r = _cli("logits", "--model", str(model_dirs["A"]), "--ids", "5,17,3", "--dtype", "float32")
    probe = json.loads(r.stdout)
    ref = P.forward_logits(W, [5, 17, 3])[-1]
    assert probe["argmax"] == int(torch.argmax(ref))
    assert abs(probe["sum"] - float(ref.sum())) < 1e-3
    r = _cli("inspect", "--model", str(model_dirs["A"]))
    info = json.loads(r.stdout)
    assert info["layers"] == 2 and info["d_model"] == 64 and info["vocab"] == 512
    r = _cli("generate", "--model", str(model_dirs["A"]), "--prompt", "hello")
    assert r.returncode != 0 and "no tokenizer" in r.stderr
    r = _cli("bench", "--model", str(model_dirs["A"]), "--prefill", "16", "--decode", "4", "--runs", "1")
    assert r.returncode == 0, r.stderr
    assert json.loads(r.stdout)["decode_tokens"] == 4


def test_top_k_and_top_p_from_the_largest_logits_equal_the_whole_row(model_dirs):
    """With top-k / top-p on, the device hands the host each row's largest logits; the tokens
    must be the ones the host's sampler picks from whole rows, draw for draw."""
    from nimbus_infer_rs_b200.csrc import ops as ops_mod
    from nimbus_infer_rs_b200.sampling import BatchSampler, SequenceSampler
    from nimbus_infer_rs_b200.sampling import host as host_sampler
    ops = ops_mod.backend()
    torch.manual_seed(11)
    fast_rows = 0
    for kw in (dict(temperature=0.8, top_k=40), dict(temperature=1.0, top_p=0.9),
               dict(temperature=1.3, top_k=200, top_p=0.6), dict(temperature=0.5, top_p=0.0),
               dict(temperature=1.0, top_p=0.999), dict(temperature=0.9, top_k=5000),
               dict(temperature=0.8, top_k=40, repetition_penalty=1.3),
               dict(temperature=1.1, top_p=0.5, repetition_penalty=0.8)):
        p = SamplingParams(seed=3, **kw)
        logits = torch.randn(6, 50257, device="cuda:0") * 4.0
        logits[0, 100:140] = logits[0].max()                 # ties
        a = [SequenceSampler(p, i) for i in range(6)]
        b = [SequenceSampler(p, i) for i in range(6)]
        for i in range(6):                                   # a history: the row's best tokens and others
            hist = logits[i].topk(3 + i).indices.tolist() + [7, 7, 50000 - i]
            a[i].generated, b[i].generated = list(hist), list(hist)
        got = BatchSampler(p, ops, logits.device).sample(logits.clone(), a)
        rows = logits.cpu().numpy()
        want = [host_sampler.sample(rows[i], p, b[i].generated, b[i].rng) for i in range(6)]
        assert got == want, kw
        assert [s.rng.next_f64() for s in a] == [s.rng.next_f64() for s in b]   # same draws used
        vals, idx, counts, stats = ops.top_candidates(logits, 1024, max(p.temperature, 1e-6))
        for i in range(6):
            r = host_sampler.sample_from_candidates(
                vals[i].cpu().numpy(), idx[i].cpu().numpy(), int(counts[i]), float(stats[i, 0]),
                float(stats[i, 1]), p, SequenceSampler(p, i).rng, 1024)
            fast_rows += r is not None
    assert fast_rows >= 18                                   # most rows never leave the device whole


@pytest.mark.parametrize("vocab", [512, 2500])
def test_top_p_inside_the_decode_session_equals_the_host_sampler(vocab):
    """Generation with top-p runs in the decode session (the sampling kernel inside the recorded
    step).  With a vocabulary of 512 the kernel lists every token and settles each row; with
    2,500 tokens and random weights the distribution is flat, the cut lies beyond the 1024
    largest logits and the rows are handed back to the host each step.  Both ways the tokens are
    the ones the host's sampler draws from the same logits."""
    from nimbus_infer_rs_b200 import GPT2Config
    from nimbus_infer_rs_b200.sampling import BatchSampler
    # (one page of context, so that the session's step and a plain step run the same kernels on
    # the same shapes and give the same bits)
    cfg = GPT2Config.from_json(dict(model_type="gpt2", vocab_size=vocab, n_positions=64, n_embd=64,
                                    n_layer=2, n_head=4, n_inner=128, layer_norm_epsilon=1e-5,
                                    activation_function="gelu_new"))
    e = Engine.random(cfg, seed=4, dtype="bfloat16", cache_tokens=1024)
    prompts = [[5, 17, 3, 9], [11, 2], [7] * 9]
    from nimbus_infer_rs_b200.sampling import SequenceSampler

    def step_by_step(p):
        """Plain steps and the batch sampler: what generation did before there was a session."""
        sampler = BatchSampler(p, e.ops, e.rt.device)
        seqs = [SequenceSampler(p, i) for i in range(len(prompts))]
        slots = [e.alloc_slot() for _ in prompts]
        toks = sampler.sample(e.step([(s, pr, [len(pr) - 1]) for s, pr in zip(slots, prompts)]), seqs)
        out = [[t] for t in toks]
        for _ in range(p.max_new_tokens - 1):
            toks = sampler.sample(e.step([(s, [t], [0]) for s, t in zip(slots, toks)]), seqs)
            for o, t in zip(out, toks):
                o.append(t)
        for s in slots:
            e.free_slot(s)
        return out

    # with a repetition penalty the session keeps each sequence's tokens on the device
    for kw in (dict(temperature=0.0, repetition_penalty=1.7), dict(temperature=0.8, repetition_penalty=1.3),
               dict(temperature=1.1, top_k=30, top_p=0.9, repetition_penalty=0.7)):
        p = SamplingParams(max_new_tokens=20, seed=5, **kw)
        assert e.generate(prompts, p) == step_by_step(p), kw
    for kw in (dict(temperature=0.9, top_p=0.8), dict(temperature=1.2, top_k=50, top_p=0.95)):
        p = SamplingParams(max_new_tokens=20, seed=5, **kw)
        assert not BatchSampler(p, e.ops, e.rt.device).needs_host()
        in_session = e.generate(prompts, p)
        assert in_session == step_by_step(p), kw
        orig = BatchSampler.needs_host
        BatchSampler.needs_host = lambda self: True          # the host decides every token
        try:
            on_host = e.generate(prompts, p)
        finally:
            BatchSampler.needs_host = orig
        assert in_session == on_host, kw
        assert [len(x) for x in in_session] == [20, 20, 20]


# ---------------------------------------------------------------------------------------------
# The decode session: generation decodes through `DecodeSession` (fixed device buffers, the
# step recorded in a CUDA graph, pages reserved between replays), not through `Engine.step`.
# ---------------------------------------------------------------------------------------------
def _session_prompts(e, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    V = e.spec.vocab_size
    return [torch.randint(0, V, (n,), generator=g).tolist() for n in lengths]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_generation_crosses_pages_and_reaches_the_context_end_inside_the_decode_session(
        model_dirs, name, dtype):
    """Unequal prompts (3, 61, 64 and 70 tokens) generate until the longest allowed: every
    sequence crosses a page end (64 tokens) *inside* the session, the prompt of 64 needs its
    new page for the session's very first token, and the prompts of 61 and 70 run into the end
    of the context, where their budget is clipped.  Guards `DecodeSession.step`'s
    `cache.reserve(grow)` between replays (a page that was not reserved, or a block table that
    was not brought up to date before the replay, would make the step read or write a wrong
    page, and the ids would part from the plain implementation's at that token) and the
    session's layout (`max_kv_len` pinned to the context, positions advanced on the device).
    A second call with other lengths and the same batch size finds the buffers and the recorded
    step that `close()` kept (`engine.decode_states`) and must be as right as the first."""
    W = P.PlainWeights(model_dirs[name])
    e = Engine.load(model_dirs[name], dtype=dtype, cache_tokens=4096)
    m = e.spec.max_seq_len
    n_new = min(m - 61, 75)
    for call, lengths in enumerate(((3, 61, 64, 70), (66, 2, 63, 17))):
        prompts = _session_prompts(e, lengths, seed=31 + call)
        out = e.generate(prompts, SamplingParams(max_new_tokens=n_new, temperature=0.0))
        crossed = 0
        for p, o in zip(prompts, out):
            assert len(o) == min(n_new, m - len(p))                  # clipped at the context end
            crossed += (len(p) + len(o) - 2) // 64 > (len(p) - 1) // 64   # cached tokens: a new page
            assert_greedy_matches(o, W, p, dtype)
        assert crossed >= 3                     # (a prompt of 70 in a context of 128 cannot)
        if call == 0:
            assert len(e.decode_states) == 1                          # kept for the next batch
            kept = next(iter(e.decode_states.values()))["graph"]
        else:
            assert next(iter(e.decode_states.values()))["graph"] is kept   # and used again
    assert e.cache.slots.n_free == e.cache.n_slots
    assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)
    e.ops.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_row_that_stops_becomes_padding_while_the_others_cross_a_page(model_dirs, dtype):
    """One sequence samples a stop token early; `DecodeSession.retire` turns its row into
    padding (slot -1) and its slot and pages go back at once, while the other rows go on past
    a page end.  A row that was not retired (or whose freed pages the step still wrote) would
    change the others' ids, and the plain implementation's stop rule would not be met."""
    W = P.PlainWeights(model_dirs["A"])
    e = Engine.load(model_dirs["A"], dtype=dtype, cache_tokens=4096)
    prompts = _session_prompts(e, (50, 60, 7), seed=77)
    free_run = P.greedy_generate(W, prompts[2], 30)
    stop = free_run[5]                                  # request 2 ends after at most 6 tokens
    out = e.generate(prompts, SamplingParams(max_new_tokens=30, temperature=0.0, stop_tokens=[stop]))
    for p, o in zip(prompts, out):
        assert_greedy_matches(o, W, p, dtype, stop_tokens=(stop,))
    assert out[2][-1] == stop and len(out[2]) <= 6
    assert any(len(o) == 30 for o in out[:2]) or all(o[-1] == stop for o in out[:2])
    assert e.cache.slots.n_free == e.cache.n_slots


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "D"])
@pytest.mark.parametrize("clusters", [1, 0])
def test_the_sessions_logits_equal_the_plain_implementations(model_dirs, name, dtype, clusters):
    """Not only ids: after N replayed steps of a session (N chosen so that a page end lies
    behind every row) the logits the session holds are the plain implementation's last-row
    logits of each sequence, at the tolerance of every other logits test.  In bfloat16 the
    splits of a sequence's pages (2 for A, 5 for D) merge inside thread-block clusters, or
    with `clusters` off through scratch memory: both inside the replayed graph."""
    from gpu_helpers import assert_close
    from nimbus_infer_rs_b200.engine.decode import DecodeSession
    if dtype == "float32" and not clusters:
        pytest.skip("the 32-bit kernel has one way to merge")
    W = P.PlainWeights(model_dirs[name])
    e = Engine.load(model_dirs[name], dtype=dtype, cache_tokens=4096)
    was = e.ops.decode_clusters
    e.ops.set_decode_clusters(clusters)
    try:
        _session_logits(e, W, name, dtype)
    finally:
        e.ops.set_decode_clusters(was)


def _session_logits(e, W, name, dtype):
    from gpu_helpers import assert_close
    from nimbus_infer_rs_b200.engine.decode import DecodeSession
    seqs = _session_prompts(e, (40, 62, 64), seed=5)
    extra = _session_prompts(e, (30, 30, 30), seed=6)
    slots = [e.alloc_slot() for _ in seqs]
    e.step([(s, p[:-1], []) for s, p in zip(slots, seqs)])
    session = DecodeSession(e, slots, [p[-1] for p in seqs])
    n_steps = 27
    for t in range(n_steps):
        session.step([(seqs[i] + extra[i])[len(seqs[i]) - 1 + t] for i in range(3)])
        session.read_tokens()
        if t in (0, 1, 2, 5, n_steps - 1):
            got = session.logits.clone()
            want = torch.stack([P.forward_logits(W, (seqs[i] + extra[i])[:len(seqs[i]) + t])[-1]
                                for i in range(3)])
            assert_close(got, want, dtype, f"{name} session step {t}")
    assert session._graph is not None                   # the steps after the first were replays
    session.close()
    for s in slots:
        e.free_slot(s)


def test_tiny_b_samples_at_temperature_as_the_host_sampler_does_on_plain_logits(model_dirs):
    """Tiny B's own workload: prompts of 1 and 17 tokens, 12 steps at temperature 0.7 from a
    fixed seed.  In 32-bit the ids must be the ones `sampling.host.sample` draws, with the same
    per-sequence xoshiro256++ stream, from the plain implementation's logits; the comparison of
    a sequence ends where a draw falls so close to an edge of the cumulative distribution that
    rounding may decide it (as `assert_greedy_matches` ends at a near tie)."""
    import copy

    import numpy as np
    from nimbus_infer_rs_b200.sampling import SequenceSampler
    from nimbus_infer_rs_b200.sampling import host as host_sampler
    W = P.PlainWeights(model_dirs["B"])
    e = Engine.load(model_dirs["B"], dtype="float32", cache_tokens=1024)
    prompts = prompts_for("B", e.spec.vocab_size)
    assert [len(p) for p in prompts] == [1, 17]
    params = SamplingParams(max_new_tokens=12, temperature=0.7, seed=1234)
    out = e.generate(prompts, params)
    assert [len(o) for o in out] == [12, 12]
    compared = 0
    for i, (p, o) in enumerate(zip(prompts, out)):
        seq = SequenceSampler(params, i)
        ctx = list(p)
        for step, tok in enumerate(o):
            row = P.forward_logits(W, ctx)[-1].numpy()
            # where the draw lands in the cumulative distribution, and how near an edge
            z = (row - row.max()) / 0.7
            pr = np.exp(z) / np.exp(z).sum()
            cdf = np.cumsum(pr)
            u = copy.deepcopy(seq.rng).next_f64()          # the number this step will draw
            want = host_sampler.sample(row.astype(np.float32), params, [], seq.rng)
            near_edge = np.abs(cdf - u).min() < 1e-4
            if tok != want:
                assert near_edge, f"request {i} step {step}: got {tok}, host sampler says {want}"
                break
            compared += 1
            ctx.append(tok)
    assert compared >= 12
