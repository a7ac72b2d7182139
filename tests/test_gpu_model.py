"""The engine against the plain implementation, in 32-bit and in bfloat16, cut in every way:
each request alone and whole; its last 32 tokens one by one; batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots and pages are used again;
long decoding from the first token on; inputs made so that a far key or a stale slot shows."""
import json

import pytest
import torch

import plain_gpt2 as P
from gpu_helpers import DTYPES, assert_close, plain_logits, random_tokens
from nimbus_infer_rs_b200 import Engine
from nimbus_infer_rs_b200.cache import PAGE

pytestmark = pytest.mark.gpu
CONFIGS = ["A", "B", "C", "D"]


def _engine(model_dirs, name, dtype, cache_tokens=2048, **kw):
    return Engine.load(model_dirs[name], dtype=dtype, cache_tokens=cache_tokens, **kw)


def _lengths(engine):
    m = engine.spec.max_seq_len
    return [n for n in (1, 2, 33, 40, 64, 65, m) if n <= m]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_each_request_alone_and_whole(model_dirs, name, dtype):
    e = _engine(model_dirs, name, dtype)
    for i, n in enumerate(_lengths(e)):
        toks = random_tokens(e.spec.vocab_size, n, seed=10 + i)
        ref = plain_logits(model_dirs[name], toks)
        s = e.alloc_slot()
        out = e.step([(s, toks, list(range(n)))])
        e.free_slot(s)
        assert_close(out, ref, dtype, f"{name} whole, {n} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_last_32_tokens_one_by_one(model_dirs, name, dtype):
    e = _engine(model_dirs, name, dtype)
    for n in (33, min(100, e.spec.max_seq_len)):
        toks = random_tokens(e.spec.vocab_size, n, seed=n)
        ref = plain_logits(model_dirs[name], toks)
        s = e.alloc_slot()
        head = n - 32
        outs = [e.step([(s, toks[:head], [head - 1])])]
        for t in range(head, n):
            outs.append(e.step([(s, [toks[t]], [0])]))
        e.free_slot(s)
        assert_close(torch.cat(outs), ref[head - 1:], dtype, f"{name} last 32 of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", CONFIGS)
def test_unequal_batches_one_after_another(model_dirs, name, dtype):
    """Three batches over a cache that holds one batch at a time, with 4 slots: prompts of
    unequal lengths in one step, then one token each; a request that is out of tokens ends
    and frees its slot while the others go on; the next batch gets the same slots and pages,
    still holding the previous batch's keys and values."""
    e = _engine(model_dirs, name, dtype, cache_tokens=6 * PAGE, n_slots=4)
    m = e.spec.max_seq_len
    V = e.spec.vocab_size
    batches = [
        [(5, 12), (9, 3), (13, 20), (1, 7)],          # (prompt length, decoded tokens)
        [(min(60, m - 6), 6), (2, 30), (17, 1)],
        [(1, 40), (33, 0), (7, 33), (20, 9)],
    ]
    seed = 0
    for bi, batch in enumerate(batches):
        reqs = []
        for plen, ndec in batch:
            seed += 1
            toks = random_tokens(V, min(plen + ndec, m), seed=1000 + seed)
            reqs.append({"toks": toks, "plen": min(plen, len(toks)), "got": [],
                         "slot": e.alloc_slot()})
        outs = e.step([(r["slot"], r["toks"][:r["plen"]], list(range(r["plen"]))) for r in reqs])
        o = 0
        for r in reqs:
            r["got"].append(outs[o:o + r["plen"]])
            o += r["plen"]
            r["pos"] = r["plen"]
        live = list(reqs)
        while True:
            for r in [r for r in live if r["pos"] >= len(r["toks"])]:
                e.free_slot(r["slot"])                                  # ends earlier
                live.remove(r)
            if not live:
                break
            outs = e.step([(r["slot"], [r["toks"][r["pos"]]], [0]) for r in live])
            for i, r in enumerate(live):
                r["got"].append(outs[i:i + 1])
                r["pos"] += 1
        assert e.cache.slots.n_free == 4
        for ri, r in enumerate(reqs):
            ref = plain_logits(model_dirs[name], r["toks"])
            assert_close(torch.cat(r["got"]), ref, dtype, f"{name} batch {bi} request {ri}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_from_the_first_token(model_dirs, name, dtype):
    """A one-token prompt, then token by token to the end of the context: the first tokens of
    a sequence, every page boundary and the last position are all single-token steps."""
    e = _engine(model_dirs, name, dtype)
    n = min(e.spec.max_seq_len, 200)
    toks = random_tokens(e.spec.vocab_size, n, seed=77)
    ref = plain_logits(model_dirs[name], toks)
    s = e.alloc_slot()
    outs = [e.step([(s, [t], [0])]) for t in toks]
    e.free_slot(s)
    assert_close(torch.cat(outs), ref, dtype, f"{name} token by token")
    assert_close(torch.cat(outs[:3]), ref[:3], dtype, f"{name} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunks_of_any_size_continue_a_sequence(model_dirs, dtype):
    e = _engine(model_dirs, "C", dtype)
    toks = random_tokens(e.spec.vocab_size, 150, seed=5)
    ref = plain_logits(model_dirs["C"], toks)
    s = e.alloc_slot()
    outs, p = [], 0
    for n in (1, 62, 2, 1, 70, 14):                   # crosses page boundaries inside chunks
        outs.append(e.step([(s, toks[p:p + n], list(range(n)))]))
        p += n
    e.free_slot(s)
    assert_close(torch.cat(outs), ref, dtype, "chunked continuation")


def _spiky_model(tmp_path, dtype_store):
    """Tiny C with weights made so that, in layer 0, a query of token `b` scores one key of
    token `a` far above all others: the answer then hangs on that single far key."""
    from nimbus_infer_rs_b200.config import GPT2Config
    from nimbus_infer_rs_b200.models.gpt2 import random_tensors as gpt2_tensors
    from nimbus_infer_rs_b200.weights import write_safetensors
    from tiny_configs import TINY_C
    cfg = GPT2Config.from_json(TINY_C)
    t = gpt2_tensors(cfg, 99, std=0.05, bias_std=0.01, dtype=torch.float32)
    d, hd = cfg.d_model, cfg.head_dim
    a, b = 700, 701
    e1 = torch.zeros(d); e1[::2] = 1.0; e1[1::2] = -1.0
    e2 = torch.zeros(d); e2[: d // 2] = 1.0; e2[d // 2:] = -1.0
    t["wte"][a] = e1 * 0.1
    t["wte"][b] = e2 * 0.1
    f = torch.zeros(hd); f[:8] = 1.0
    for head in range(cfg.n_heads):                    # queries of every head look for e1's key
        t["h.0.attn.q.weight"][:, head * hd:(head + 1) * hd] += torch.outer(e2, f) * 0.03
    for kvh in range(cfg.n_kv_heads):
        t["h.0.attn.k.weight"][:, kvh * hd:(kvh + 1) * hd] += torch.outer(e1, f) * 0.03
        t["h.0.attn.v.weight"][:, kvh * hd:(kvh + 1) * hd] += torch.outer(e1, torch.ones(hd)) * 0.03
    t = {k: (v.to(dtype_store) if v.dim() == 2 else v) for k, v in t.items()}
    dd = tmp_path / "spiky"
    dd.mkdir()
    (dd / "config.json").write_text(json.dumps(TINY_C))
    write_safetensors(dd / "model.safetensors", t)
    return dd, a, b


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_and_a_reused_slot_show(tmp_path, dtype):
    d, a, b = _spiky_model(tmp_path, torch.bfloat16)
    W = P.PlainWeights(d)
    e = Engine.load(d, dtype=dtype, cache_tokens=8 * PAGE, n_slots=1)
    V = e.spec.vocab_size
    n = 430
    toks = [t % 699 for t in random_tokens(V, n, seed=3)]      # neither special token
    toks[5] = a                                                 # the far key, on the first page
    toks[-1] = b                                                # the query, seven pages later
    ref = P.forward_logits(W, toks)
    # the construction works: without the far key the last logits are clearly different
    without = list(toks); without[5] = 1
    diff = (P.forward_logits(W, without)[-1] - ref[-1]).abs().max()
    assert diff > 10 * 2e-2 * ref[-1].abs().max()
    s = e.alloc_slot()
    out = e.step([(s, toks[:-1], [n - 2])])
    out2 = e.step([(s, [toks[-1]], [0])])                       # decode step reads the far key
    e.free_slot(s)
    assert_close(torch.cat([out, out2]), ref[-2:], dtype, "far key, decode")
    # the same slot and pages again, now for a short sequence that ends with the query token:
    # the previous sequence's key of `a` is still in the first page, at a position this
    # sequence has not reached
    s2 = e.alloc_slot()
    assert s2 == s
    short = [3, 4, b]
    ref_short = P.forward_logits(W, short)
    out = e.step([(s2, short, [0, 1, 2])])
    assert_close(out, ref_short, dtype, "reused slot, whole")
    out = e.step([(s2, [b], [0])])
    assert_close(out, P.forward_logits(W, short + [b])[-1:], dtype, "reused slot, decode")
    e.free_slot(s2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_changes_no_result(model_dirs, dtype):
    """The same step with padding rows appended gives the same logits bit for bit."""
    from nimbus_infer_rs_b200.engine.batch import build_layout
    from nimbus_infer_rs_b200.engine.context import StepContext
    e = _engine(model_dirs, "B", dtype)
    toks = [random_tokens(1000, n, seed=n) for n in (7, 3)]
    got = []
    for pad in (1, 16):
        slots = [e.alloc_slot() for _ in toks]
        entries = e._check_entries([(s, t, list(range(len(t)))) for s, t in zip(slots, toks)])
        e.cache.reserve([(s, len(t)) for s, t, _ in entries])
        lay = build_layout(entries, [0, 0], e.rt.device, pad_rows_to=pad)
        assert lay.n_rows == (10 if pad == 1 else 16)
        got.append(e.model.forward(StepContext(e.rt, e.ops, lay, e.model.position, e.cache)))
        for s in slots:
            e.free_slot(s)
    assert torch.equal(got[0], got[1])


def test_stored_32bit_weights_stay_32bit_in_a_bfloat16_run(model_dirs):
    e = _engine(model_dirs, "C", "bfloat16")          # tiny C: bf16 tables, matrices kept in fp32
    assert e.model.params["layers.0.ffn.fc.weight"].dtype == torch.float32
    assert e.model.params["embedding.table"].dtype == torch.bfloat16
    assert e.cache.groups[0].storage.dtype == torch.bfloat16
    e = _engine(model_dirs, "A", "bfloat16")
    assert e.model.params["layers.0.ffn.fc.weight"].dtype == torch.bfloat16
    assert e.model.params["final_norm.weight"].dtype == torch.float32


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_steps_of_a_shape_that_comes_again_are_replayed_and_change_nothing(model_dirs, name, dtype):
    """Steps of one shape (same numbers of rows, sequences and wanted places) with other
    tokens, in other slots, at other lengths: from the second on they are replayed from a
    recorded CUDA graph.  Each must equal the plain implementation and, bit for bit, an engine
    that never records."""
    e = _engine(model_dirs, name, dtype, n_slots=6)
    plain = _engine(model_dirs, name, dtype, n_slots=6)
    plain.step_graphs.capacity = 0            # never records
    V = e.spec.vocab_size
    # prompts: three steps of shape (20 + 7 tokens, wanted: 2 + 1), in different slots
    held = []
    for r in range(3):
        for eng in (e, plain):
            eng._slots = [eng.alloc_slot() for _ in range(2)]
        assert e._slots == plain._slots
        a, b = random_tokens(V, 20, seed=50 + r), random_tokens(V, 7, seed=60 + r)
        req = [(e._slots[0], a, [3, 19]), (e._slots[1], b, [6])]
        out, ref = e.step(req), plain.step(req)
        assert torch.equal(out, ref), f"prompt step {r}"
        assert_close(out, torch.cat([plain_logits(model_dirs[name], a)[[3, 19]],
                                     plain_logits(model_dirs[name], b)[[6]]]), dtype, f"prompts {r}")
        held.append((list(e._slots), [a, b]))
    assert e.step_graphs.captures == 1 and e.step_graphs.replays == 2
    # one token each for all six sequences, many times over: lengths cross a page boundary
    # and the power-of-two range of the longest sequence changes on the way
    seqs = [(s, list(t)) for slots, toks in held for s, t in zip(slots, toks)]
    n_dec = min(60, e.spec.max_seq_len - 20)
    new = [random_tokens(V, n_dec, seed=70 + i) for i in range(len(seqs))]
    for t in range(n_dec):
        req = [(s, [new[i][t]], [0]) for i, (s, _) in enumerate(seqs)]
        out, ref = e.step(req), plain.step(req)
        assert torch.equal(out, ref), f"decode step {t}"
        for i, (_, toks) in enumerate(seqs):
            toks.append(new[i][t])
        if t in (0, 1, 2, n_dec // 2, n_dec - 1):
            want = torch.stack([plain_logits(model_dirs[name], toks)[-1] for _, toks in seqs])
            assert_close(out, want, dtype, f"decode step {t}")
    assert e.step_graphs.replays >= 2 + n_dec - 4 and plain.step_graphs.replays == 0
    e.ops.check_device_errors()


def test_recorded_steps_are_dropped_least_recently_used_first(model_dirs):
    """With room for one recording, two shapes taking turns are recorded again and again and
    still give what the plain launches give."""
    e = _engine(model_dirs, "A", "bfloat16", n_slots=4)
    plain = _engine(model_dirs, "A", "bfloat16", n_slots=4)
    e.step_graphs.capacity = 1
    plain.step_graphs.capacity = 0
    V = e.spec.vocab_size
    for r in range(6):
        n = 9 if r % 2 == 0 else 14                       # two shapes, alternating
        toks = random_tokens(V, n, seed=200 + r)
        for eng in (e, plain):
            eng._s = eng.alloc_slot()
        out, ref = e.step([(e._s, toks, [n - 1])]), plain.step([(plain._s, toks, [n - 1])])
        assert torch.equal(out, ref)
        assert_close(out, plain_logits(model_dirs["A"], toks)[-1:], "bfloat16", f"step {r}")
        for eng in (e, plain):
            eng.free_slot(eng._s)
    assert len(e.step_graphs._graphs) == 1 and e.step_graphs.captures >= 3


@pytest.mark.parametrize("name", ["A", "C"])
def test_kernels_that_start_before_their_predecessor_ends_change_nothing(model_dirs, name):
    """With programmatic dependent launch a kernel is set up, and fetches weights, while the
    kernel before it is finishing.  Whatever it reads of that kernel's work it must read after
    its wait: a prompt, then eighty single-token steps (plain launches, recorded steps and
    their replays, page boundaries), give the same bits with the overlap on and off."""
    from nimbus_infer_rs_b200.csrc import ops as ops_mod
    ops = ops_mod.backend()
    was = ops.overlap
    runs = {}
    try:
        for on in (True, False):
            ops.set_overlap(on)
            e = _engine(model_dirs, name, "bfloat16")
            toks = random_tokens(e.spec.vocab_size, 150, seed=9)
            slots = [e.alloc_slot(), e.alloc_slot()]
            outs = [e.step([(slots[0], toks[:37], list(range(37))), (slots[1], toks[5:20], [14])])]
            for i in range(80):
                outs.append(e.step([(slots[0], [toks[37 + i]], [0]), (slots[1], [toks[20 + i]], [0])]))
            runs[on] = torch.cat(outs).cpu()
            for s in slots:
                e.free_slot(s)
    finally:
        ops.set_overlap(was)
    assert torch.equal(runs[True], runs[False])
    ref = plain_logits(model_dirs[name], toks[:37])
    assert_close(runs[True][:37], ref[:37], "bfloat16", f"{name} prompt")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_a_poisoned_cache_page_does_not_reach_another_request(model_dirs, name, dtype):
    """Pages go back to the pool and are handed out again uncleared.  Here every row of every
    page is NaN (keys) or infinite (values) before each batch, as if earlier requests had
    overflowed: prompts of unequal lengths in one step, then single tokens across a page end,
    must give the plain implementation's logits, because no kernel may let a row that holds
    no key of the sequence into a sum (a zero probability times infinity is not zero)."""
    e = _engine(model_dirs, name, dtype, cache_tokens=8 * PAGE, n_slots=3)
    V = e.spec.vocab_size
    for batch in range(2):
        for g in e.cache.groups:
            g.storage[:, 0] = float("nan")
            g.storage[:, 1] = float("inf")
        seqs = [random_tokens(V, n, seed=300 + 10 * batch + i) for i, n in enumerate((70, 9, 61))]
        slots = [e.alloc_slot() for _ in seqs]
        outs = [e.step([(s, t[:-6], list(range(len(t) - 6))) for s, t in zip(slots, seqs)])]
        for i in range(6):
            outs.append(e.step([(s, [t[len(t) - 6 + i]], [0]) for s, t in zip(slots, seqs)]))
        for s in slots:
            e.free_slot(s)
        o = 0
        for j, t in enumerate(seqs):
            n = len(t) - 6
            ref = plain_logits(model_dirs[name], t)
            assert_close(outs[0][o:o + n], ref[:n], dtype, f"{name} batch {batch} prompt {j}")
            assert_close(torch.cat([st[j:j + 1] for st in outs[1:]]), ref[n:], dtype,
                         f"{name} batch {batch} decode {j}")
            o += n
    e.ops.check_device_errors()
