"""The reference project's own test checkpoint (tests/fixtures/tiny-gpt2: its config keys with
``head_dim: null`` and ``n_kv_heads: null``, 44 tensors stored in F32 under its names, no
linear biases) through the engine, against the plain implementation, in the three cuttings and
both precisions; and the reference's two end-to-end properties (tests/engine.rs:14-23 greedy
generation is deterministic, tests/engine.rs:25-57 generation with the cache gives the tokens
of re-running the whole sequence every step)."""
from pathlib import Path

import pytest
import torch

import plain_gpt2 as P
from gpu_helpers import DTYPES, assert_close, assert_greedy_matches, random_tokens
from nimbus_infer_rs_b200 import Engine, SamplingParams

pytestmark = pytest.mark.gpu
FIXTURE = Path(__file__).resolve().parent / "fixtures" / "tiny-gpt2"


@pytest.fixture(scope="module")
def plain():
    return P.PlainWeights(FIXTURE)


def test_the_fixture_loads_as_the_reference_describes_it():
    e = Engine.load(FIXTURE, dtype="float32", cache_tokens=256)
    info = e.inspect()
    assert info["n_params"] == 878_848 and info["name"] == "tiny-gpt2"
    assert (info["layers"], info["d_model"], info["heads"], info["vocab"]) == (4, 128, 4, 448)
    assert e.model.params["layers.0.mixer.qkv.bias"] is None       # no linear biases in the file
    # a file without a single bf16 matrix is a full-precision checkpoint: a bfloat16 run rounds
    # its matrices (they then run on the tensor cores), vectors stay 32-bit
    e16 = Engine.load(FIXTURE, dtype="bfloat16", cache_tokens=256)
    assert e16.model.params["layers.0.ffn.fc.weight"].dtype == torch.bfloat16
    assert e16.model.params["final_norm.weight"].dtype == torch.float32
    kept = Engine.load(FIXTURE, dtype="bfloat16", cache_tokens=256, cast_weights=False)
    assert kept.model.params["layers.0.ffn.fc.weight"].dtype == torch.float32


@pytest.mark.parametrize("dtype", DTYPES)
def test_fixture_alone_whole_and_last_32_one_by_one(plain, dtype):
    e = Engine.load(FIXTURE, dtype=dtype, cache_tokens=1024)
    for n in (1, 40, 130, 256):
        toks = random_tokens(448, n, seed=n)
        ref = P.forward_logits(plain, toks)
        s = e.alloc_slot()
        out = e.step([(s, toks, list(range(n)))])
        e.free_slot(s)
        assert_close(out, ref, dtype, f"fixture whole, {n} tokens")
        if n > 32:
            s = e.alloc_slot()
            head = n - 32
            outs = [e.step([(s, toks[:head], [head - 1])])]
            outs += [e.step([(s, [toks[t]], [0])]) for t in range(head, n)]
            e.free_slot(s)
            assert_close(torch.cat(outs), ref[head - 1:], dtype, f"fixture last 32 of {n}")
    e.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_fixture_unequal_batches_one_after_another(plain, dtype):
    e = Engine.load(FIXTURE, dtype=dtype, cache_tokens=5 * 64, n_slots=3)
    seed = 0
    for batch in ([(5, 12), (70, 9), (1, 30)], [(64, 3), (13, 20)], [(2, 70), (100, 0), (33, 31)]):
        reqs = []
        for plen, ndec in batch:
            seed += 1
            reqs.append({"toks": random_tokens(448, plen + ndec, seed=500 + seed), "plen": plen,
                         "got": [], "slot": e.alloc_slot()})
        outs = e.step([(r["slot"], r["toks"][:r["plen"]], list(range(r["plen"]))) for r in reqs])
        o = 0
        for r in reqs:
            r["got"].append(outs[o:o + r["plen"]])
            o += r["plen"]
            r["pos"] = r["plen"]
        live = list(reqs)
        while True:
            for r in [r for r in live if r["pos"] >= len(r["toks"])]:
                e.free_slot(r["slot"])
                live.remove(r)
            if not live:
                break
            outs = e.step([(r["slot"], [r["toks"][r["pos"]]], [0]) for r in live])
            for i, r in enumerate(live):
                r["got"].append(outs[i:i + 1])
                r["pos"] += 1
        for ri, r in enumerate(reqs):
            assert_close(torch.cat(r["got"]), P.forward_logits(plain, r["toks"]), dtype,
                         f"fixture batch request {ri}")
    assert e.cache.slots.n_free == 3
    e.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_references_two_end_to_end_properties(plain, dtype):
    e = Engine.load(FIXTURE, dtype=dtype, cache_tokens=1024)
    prompt = random_tokens(448, 9, seed=42)
    params = SamplingParams(max_new_tokens=24, temperature=0.0)
    a = e.generate([prompt], params)[0]
    b = e.generate([prompt], params)[0]
    assert len(a) == 24 and a == b                                  # tests/engine.rs:14-23
    cached = e.generate([prompt], SamplingParams(max_new_tokens=8, temperature=0.0))[0]
    assert cached == a[:8]
    assert_greedy_matches(cached, plain, prompt, dtype)             # tests/engine.rs:25-57
    if dtype == "float32":
        assert cached == P.greedy_generate(plain, prompt, 8)
