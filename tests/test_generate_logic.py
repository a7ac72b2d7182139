"""The generation loop's decisions, and the loop itself over the engine's host logic with the
torch-CPU stand-in for the kernels."""
import pytest
import torch

import plain_gpt2 as P
from nimbus_infer_rs_b200 import Engine, SamplingParams
from nimbus_infer_rs_b200.cache import CacheError
from nimbus_infer_rs_b200.engine.generate import SequenceProgress, plan_batches, token_budget


def test_token_budget():          # src/engine.rs:265-266
    assert token_budget(10, 64, 1024) == 64
    assert token_budget(1000, 64, 1024) == 24
    assert token_budget(1024, 64, 1024) == 0
    assert token_budget(2000, 64, 1024) == 0


def test_sequence_progress_stop_rules():     # src/engine.rs:279-291
    s = SequenceProgress(0, 5, 3, frozenset({9}))
    assert s.record(4) and s.record(4) and not s.record(4)      # ends at its last step
    assert s.generated == [4, 4, 4] and s.finished
    s = SequenceProgress(0, 5, 8, frozenset({9}))
    assert s.record(1) and not s.record(9)                        # the stop token is kept
    assert s.generated == [1, 9]
    assert SequenceProgress(0, 5, 0, frozenset()).finished        # nothing to generate


def test_plan_batches():
    # by count
    assert plan_batches([5] * 5, [4] * 5, max_batch=2, cache_pages=100) == [[0, 1], [2, 3], [4]]
    # by pages: 60+5-1 = 64 tokens -> one page each; 70 -> two pages
    assert plan_batches([60, 60, 70, 10], [5, 5, 5, 5], max_batch=8, cache_pages=3) == \
        [[0, 1], [2, 3]]
    with pytest.raises(ValueError, match="needs"):
        plan_batches([200], [10], max_batch=1, cache_pages=2)
    assert plan_batches([], [], max_batch=3, cache_pages=3) == []


@pytest.fixture()
def engine_b(model_dirs, cpu_backend):
    return Engine.load(model_dirs["B"], dtype="float32", device="cpu", cache_tokens=4 * 64,
                       n_slots=3)


def test_generate_matches_plain_greedy_over_several_batches(engine_b, model_dirs):
    W = P.PlainWeights(model_dirs["B"])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (1, 17, 5, 9, 13, 30, 2)]
    seen = []
    out = engine_b.generate(prompts, SamplingParams(max_new_tokens=6, temperature=0.0),
                            on_token=lambda i, t, s: seen.append((i, t, s)), max_batch=3)
    want = [P.greedy_generate(W, p, 6) for p in prompts]
    assert out == want
    assert engine_b.cache.slots.n_free == 3                      # every slot came back
    assert all(g_.pool.n_free == g_.pool.n_pages for g_ in engine_b.cache.groups)
    for i, ids in enumerate(out):                                # callback: (request, token, step)
        assert [(t, s) for j, t, s in seen if j == i] == [(t, s) for s, t in enumerate(ids)]


def test_stop_tokens_end_a_sequence_early_and_the_rest_go_on(engine_b, model_dirs):
    W = P.PlainWeights(model_dirs["B"])
    prompts = [[3, 4, 5], [100, 200], [7]]
    free_run = [P.greedy_generate(W, p, 8) for p in prompts]
    stop = free_run[1][2]                                        # third token of request 1
    out = engine_b.generate(prompts, SamplingParams(max_new_tokens=8, temperature=0.0,
                                                    stop_tokens=[stop]))
    want = [P.greedy_generate(W, p, 8, stop_tokens=(stop,)) for p in prompts]
    assert out == want
    assert len(out[1]) <= 3 and out[1][-1] == stop


def test_budget_is_clipped_at_the_context_end(engine_b, model_dirs):
    W = P.PlainWeights(model_dirs["B"])      # max_seq_len 64
    prompt = list(range(1, 61))
    out = engine_b.generate([prompt], SamplingParams(max_new_tokens=50, temperature=0.0))
    assert len(out[0]) == 4 and out[0] == P.greedy_generate(W, prompt, 50)
    assert engine_b.generate([list(range(64))], SamplingParams(max_new_tokens=5)) == [[]]


def test_empty_prompt_and_bad_tokens_are_errors_before_any_launch(engine_b):
    with pytest.raises(ValueError, match="empty token sequence"):    # src/engine.rs:261-263
        engine_b.generate([[1], []])
    s = engine_b.alloc_slot()
    launches = engine_b.ops.launches
    with pytest.raises(ValueError, match="token id outside"):
        engine_b.step([(s, [1, 1000], None)])
    with pytest.raises(ValueError, match="wanted place"):
        engine_b.step([(s, [1, 2], [2])])
    with pytest.raises(CacheError, match="exceeds the longest"):
        engine_b.step([(s, list(range(65)), None)])
    with pytest.raises(CacheError, match="not held"):
        engine_b.step([(2, [1], None)])
    assert engine_b.ops.launches == launches and engine_b.cache.lens[s] == 0


def test_temperature_sampling_is_seeded_and_independent_of_batch_mates(engine_b):
    p = SamplingParams(max_new_tokens=5, temperature=0.7, seed=123)
    a = engine_b.generate([[5, 6, 7], [9]], p)
    b = engine_b.generate([[5, 6, 7], [9]], p)
    assert a == b
    alone = engine_b.generate([[5, 6, 7]], p)
    assert alone[0] == a[0]                                       # same stream when run alone
    c = engine_b.generate([[5, 6, 7]], SamplingParams(max_new_tokens=5, temperature=0.7, seed=124))
    assert c != alone


def test_rows_the_sampling_kernel_hands_back_are_settled_from_the_steps_logits(engine_b, cpu_backend):
    """Top-p and a repetition penalty inside the decode session: the session keeps each
    sequence's tokens for the penalty, and a row that the top-p kernel marks instead of
    settling is decided by the host from the step's logits with the number drawn for it.
    Marked or not, in the session or step by step, the tokens are the same."""
    from nimbus_infer_rs_b200.sampling import BatchSampler, SequenceSampler
    prompts = [[5, 17, 3], [9], [1, 2, 3, 4, 5, 6, 7]]
    p = SamplingParams(max_new_tokens=9, temperature=0.9, top_k=50, top_p=0.8,
                       repetition_penalty=1.4, seed=11, stop_tokens=[])
    settled = engine_b.generate(prompts, p)
    cpu_backend.hand_back = True
    try:
        handed_back = engine_b.generate(prompts, p)
    finally:
        cpu_backend.hand_back = False
    assert handed_back == settled and [len(x) for x in settled] == [9, 9, 9]
    # step by step, with the batch sampler (what generation does without a session)
    sampler = BatchSampler(p, engine_b.ops, engine_b.rt.device)
    seqs = [SequenceSampler(p, i) for i in range(3)]
    slots = [engine_b.alloc_slot() for _ in prompts]
    toks = sampler.sample(engine_b.step([(s, pr, [len(pr) - 1]) for s, pr in zip(slots, prompts)]), seqs)
    out = [[t] for t in toks]
    for _ in range(8):
        toks = sampler.sample(engine_b.step([(s, [t], [0]) for s, t in zip(slots, toks)]), seqs)
        for o, t in zip(out, toks):
            o.append(t)
    for s in slots:
        engine_b.free_slot(s)
    assert out == settled


def test_step_shapes_that_share_a_recording():
    """The key under which a step's launches are recorded: its numbers of rows, sequences and
    wanted places, its longest chunk, whether it is one token each, and the power-of-two range
    of its longest sequence (not its tokens, slots or exact lengths)."""
    from types import SimpleNamespace

    from nimbus_infer_rs_b200.engine.batch import pack_step
    from nimbus_infer_rs_b200.engine.step_graphs import StepGraphs, _kv_range

    assert [_kv_range(n, 1024) for n in (1, 64, 65, 128, 129, 1000, 5000)] == \
        [64, 64, 128, 128, 256, 1024, 1024]
    class Owner:                              # stands for the engine; held weakly
        spec = SimpleNamespace(max_seq_len=1024, vocab_size=100)
    owner = Owner()
    g = StepGraphs(owner)
    a = pack_step([(0, [1, 2, 3], [2]), (1, [4], [0])], [0, 10])
    b = pack_step([(5, [9, 9, 9], [0]), (2, [7], [0])], [30, 3])          # other slots, tokens, places
    c = pack_step([(0, [1, 2, 3], [2]), (1, [4], [0])], [100, 10])        # a longer sequence
    d = pack_step([(0, [1, 2], [1]), (1, [4, 5], [0])], [0, 10])          # other chunks, same total
    assert g.key(a) == g.key(b) == g.key(d) and g.key(a) != g.key(c)
    # chunks count in units of 128 rows, rows beyond 64 in units of 64
    from nimbus_infer_rs_b200.engine.step_graphs import q_bound, row_padding
    assert [q_bound(n) for n in (1, 2, 128, 129, 1000)] == [1, 128, 128, 256, 1024]
    assert [row_padding(n) for n in (1, 64, 65, 2000)] == [1, 1, 64, 64]
    long_a = pack_step([(0, [1] * 1000, [999]), (1, [2] * 990, [989])], [0, 0], pad_rows_to=64)
    long_b = pack_step([(3, [1] * 1021, [1020]), (4, [2] * 985, [0])], [0, 0], pad_rows_to=64)
    long_c = pack_step([(3, [1] * 1021, [1020]), (4, [2] * 985, [0])], [0, 10], pad_rows_to=64)
    assert long_a.n_rows == long_b.n_rows == 2048 and g.key(long_a) == g.key(long_b)
    assert g.key(long_c) != g.key(long_b)      # a chunk that starts inside the cache: other kernels
    assert g.kv_bound(c) == 128 and not a.is_decode
    e = pack_step([(0, [1], [0]), (1, [4], [0])], [70, 10])
    assert e.is_decode and e.want_all_rows and g.kv_bound(e) == 128
    # padding rows change the row count, and with it the key, but no sequence's rows
    p = pack_step([(0, [1, 2, 3], [2]), (1, [4], [0])], [0, 10], pad_rows_to=8)
    assert p.n_rows == 8 and p.n_tokens == 4 and g.key(p) != g.key(a)
    assert list(p.buf[p.offs[0]:p.offs[1]]) == [1, 2, 3, 4, -1, -1, -1, -1]


def test_a_preset_name_builds_a_model_with_no_file_on_disk(cpu_backend):
    """``Engine.random("tiny-a")``: the preset's sizes and its spread of random values; the
    report reads the kinds of the parts and the head counts off the model's description."""
    e = Engine.random("tiny-a", seed=3, dtype="float32", device="cpu", cache_tokens=128)
    again = Engine.random("tiny-a", seed=3, dtype="float32", device="cpu", cache_tokens=128)
    other = Engine.random("tiny-a", seed=4, dtype="float32", device="cpu", cache_tokens=128)
    w = "layers.1.ffn.fc.weight"
    assert torch.equal(e.model.params[w], again.model.params[w])
    assert not torch.equal(e.model.params[w], other.model.params[w])
    assert e.model.params["layers.0.mixer.out.bias"].abs().max() > 0     # the preset's bias spread
    info = e.inspect()
    assert info["n_params"] == e.config.n_params() == 141_056
    assert (info["layers"], info["heads"], info["kv_heads"], info["head_dim"]) == (2, 4, 4, 16)
    assert (info["norm"], info["mixer"], info["ffn"], info["pos"]) == \
        ("layernorm", "causal_attention", "dense_mlp", "learned_absolute")
    assert info["activation"] == "gelu_tanh" and info["tie_head"]
    assert set(info["weight_mb_by_dtype"]) == {"float32"}
    out = e.generate([[1, 2, 3]], SamplingParams(max_new_tokens=4, temperature=0.0))
    assert len(out[0]) == 4


def test_splits_of_the_decode_attention():
    """How many CTAs share a sequence's pages (GPT-2 small's 12 heads of 64, a B200's 148 SMs,
    pages of 64 tokens): the rule's answers where a sweep on the GPU gave the best or nearly
    the best count."""
    from nimbus_infer_rs_b200.csrc.ops import decode_splits

    def s(batch, pages, heads=12, most=8):
        return decode_splits(batch * heads, pages, 64, 64, 148, most)
    # context 1,024 (16 pages): four pages a split while the launch fits, more for one row
    assert [s(b, 16) for b in (1, 2, 4, 8, 12, 16, 24, 32, 64)] == [8, 4, 4, 4, 4, 2, 2, 1, 1]
    # context 256 (4 pages): no split, but a launch far smaller than the GPU is cut anyway
    assert [s(b, 4) for b in (1, 2, 4, 8, 32)] == [4, 4, 2, 1, 1]
    # pages that no count deals out evenly stay whole; one page cannot be cut
    assert s(3, 5, heads=2) == 1 and s(1, 1) == 1
    # 16 heads (GPT-2 medium) at batch 8: 512 CTAs are still taken, 768 would not be
    assert s(8, 16, heads=16) == 4 and s(12, 16, heads=16) == 2
    # without clusters up to 16 splits
    assert s(1, 64, most=16) == 16 and s(1, 64) == 8


def test_every_row_of_a_packed_step_says_where_it_belongs():
    """Any batch, any padding: row r of sequence i carries its token, the position
    ``pos0[i] + offset`` and the sequence's slot; ``cu_rows`` cuts the rows into the sequences;
    the wanted places point at rows of their own sequence; padding rows carry -1 / -1."""
    from hypothesis import given, settings, strategies as st

    from nimbus_infer_rs_b200.engine.batch import pack_step

    seq = st.tuples(st.integers(0, 500), st.lists(st.integers(0, 50_000), min_size=1, max_size=40),
                    st.integers(0, 900), st.data())

    @settings(max_examples=60, deadline=None)
    @given(st.lists(seq, min_size=1, max_size=9), st.sampled_from([1, 8, 64]))
    def check(seqs, pad):
        entries, pos0 = [], []
        for slot, toks, p0, data in seqs:
            wants = data.draw(st.lists(st.integers(0, len(toks) - 1), max_size=4))
            entries.append((slot, toks, wants))
            pos0.append(p0)
        p = pack_step(entries, pos0, pad_rows_to=pad)
        tokens, row_pos, row_slot, cu_rows, seq_slot, seq_pos0, want = (
            p.buf[p.offs[i]:p.offs[i + 1]] for i in range(7))
        n = sum(len(e[1]) for e in entries)
        assert p.n_tokens == n and p.n_rows % pad == 0 and 0 <= p.n_rows - n < pad
        assert list(tokens[n:]) == [-1] * (p.n_rows - n) == list(row_slot[n:])
        assert cu_rows[0] == 0 and cu_rows[-1] == n and len(cu_rows) == len(entries) + 1
        w = 0
        for i, (slot, toks, wants) in enumerate(entries):
            lo, hi = cu_rows[i], cu_rows[i + 1]
            assert hi - lo == len(toks) and list(tokens[lo:hi]) == toks
            assert list(row_pos[lo:hi]) == list(range(pos0[i], pos0[i] + len(toks)))
            assert set(row_slot[lo:hi]) == {slot} and seq_slot[i] == slot and seq_pos0[i] == pos0[i]
            for x in wants:
                assert want[w] == lo + x
                w += 1
        assert w == p.n_want == len(want)
        assert p.max_q_len == max(len(e[1]) for e in entries)
        assert p.max_kv_len == max(a + len(e[1]) for a, e in zip(pos0, entries))
        assert p.is_decode == all(len(e[1]) == 1 for e in entries)
        assert p.want_all_rows == (list(want) == list(range(p.n_rows)))

    check()


def test_when_a_step_is_recorded_replayed_and_forgotten():
    """engine/step_graphs.py: a shape runs plainly at first sight, is recorded at the second
    and replayed from then on; the least recently used recording goes when there are more than
    `capacity`; steps whose logits would be large, and everything with capacity 0, run plainly.
    (The recording itself is stubbed: this is about the decisions around it.)"""
    from types import SimpleNamespace

    from nimbus_infer_rs_b200.engine.batch import pack_step
    from nimbus_infer_rs_b200.engine.step_graphs import StepGraphs

    class Owner:
        spec = SimpleNamespace(max_seq_len=1024, vocab_size=100)
        rt = SimpleNamespace(device=torch.device("cpu"))
        ops = SimpleNamespace(launches=0)
    owner = Owner()

    class Recorder(StepGraphs):
        def _record(self, p, key):
            entry = {"graph": SimpleNamespace(replay=lambda: replayed.append(key)),
                     "buf": torch.empty(p.buf.size, dtype=torch.int32),
                     "logits": torch.zeros(p.n_want, 100), "launches": 7}
            self._graphs[key] = entry
            self.captures += 1
            while len(self._graphs) > self.capacity:
                self._graphs.popitem(last=False)
            return entry

    replayed = []
    g = Recorder(owner, capacity=2)
    def step(n_seqs, tokens=5):
        return pack_step([(i, [tokens], [0]) for i in range(n_seqs)], [3] * n_seqs)
    assert g.run(step(1)) == (False, None) and g.captures == 0          # first sight
    ok, logits = g.run(step(1, tokens=9))                                 # second: recorded, replayed
    assert ok and logits.shape == (1, 100) and g.captures == 1 and len(replayed) == 1
    assert owner.ops.launches == 7                                        # the recording's launches count
    ok, _ = g.run(step(1))
    assert ok and g.captures == 1 and g.replays == 2 and owner.ops.launches == 14
    # the replayed step read this step's batch: the buffer holds its tokens
    entry = next(iter(g._graphs.values()))
    assert entry["buf"][0] == 5
    for n in (2, 3):                                                      # two more shapes
        assert g.run(step(n)) == (False, None)
        assert g.run(step(n))[0]
    assert g.captures == 3 and len(g._graphs) == 2                        # the first one is gone
    assert g.key(step(1)) not in g._graphs and g.key(step(3)) in g._graphs
    assert g.run(step(2))[0] and g.captures == 3                          # still there: replayed
    assert g.run(step(1))[0] and g.captures == 4                          # seen before: recorded anew
    assert g.key(step(3)) not in g._graphs                                # 2 was used after 3
    # large logits stay out of graphs; capacity 0 switches recording off
    big = Recorder(owner, capacity=2, max_logit_bytes=100 * 4)
    two = pack_step([(0, [1, 2], [0, 1])], [0])
    assert big.run(two) == (False, None) and big.run(two) == (False, None) and big.captures == 0
    off = Recorder(owner, capacity=0)
    assert off.run(step(1)) == (False, None) and off.run(step(1)) == (False, None)


def test_generation_across_page_ends_with_a_row_that_stops_on_the_way(model_dirs, cpu_backend):
    """The decode session's bookkeeping on the host: prompts of 40 and 61 tokens cross a page
    end (64 tokens) while they decode, one of 64 starts its second page with its first new
    token, one of 70 stays inside it; one stops early and its row is retired while the others
    go on; a second batch of the same size finds the first one's kept buffers; grouped heads
    (tiny C).  All pages and slots come back."""
    W = P.PlainWeights(model_dirs["C"])
    eng = Engine.load(model_dirs["C"], dtype="float32", device="cpu", cache_tokens=12 * 64, n_slots=4)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 777, (n,), generator=g).tolist() for n in (40, 61, 64, 70)]
    free_run = [P.greedy_generate(W, p, 30) for p in prompts]
    stop = free_run[1][5]                                   # request 1 ends inside its second page
    params = SamplingParams(max_new_tokens=30, temperature=0.0, stop_tokens=[stop])
    # greedy tokens depend on nothing but what came before: a run with a stop token is the
    # free run up to and with the first stop
    want = [r[:r.index(stop) + 1] if stop in r else r for r in free_run]
    assert len(want[1]) <= 6 and max(len(w) for w in want) == 30
    assert eng.generate(prompts, params) == want
    assert eng.cache.slots.n_free == 4
    assert all(gr.pool.n_free == gr.pool.n_pages for gr in eng.cache.groups)
    # the same batch size again, other lengths: the kept session state is found and reset
    prompts2 = [p[:n] for p, n in zip(prompts[::-1], (66, 2, 63, 1))]
    want2 = [P.greedy_generate(W, p, 9) for p in prompts2]
    assert eng.generate(prompts2, SamplingParams(max_new_tokens=9, temperature=0.0)) == want2
    assert eng.cache.slots.n_free == 4
    assert all(gr.pool.n_free == gr.pool.n_pages for gr in eng.cache.groups)
