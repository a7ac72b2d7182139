"""Real layer sizes (GPT-2 small, medium and XL widths and head counts, the full vocabulary,
two layers) against the plain implementation, in 32-bit and in bfloat16, cut three ways: each
request alone and whole; two unequal prompts in one step and then eight single-token steps of
the batch; and the bfloat16 engine beside the float32 engine.  These are the kernels the
benchmark runs: the tensor-core products at K = 768 ... 6400, the tensor-core prefill
attention with heads of 64, the weight-streaming products with the folded norm, the head over
50,257 columns."""
import pytest
import torch

import plain_gpt2 as P
from gpu_helpers import DTYPES, TOL, assert_close, random_tokens
from nimbus_infer_rs_b200 import Engine
from nimbus_infer_rs_b200.config import GPT2Config, preset_json
from nimbus_infer_rs_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

LAYERS, CONTEXT = 2, 192
LENGTHS = (138, 45)          # the last 8 tokens of each are decoded one by one
_made = {}


def _model(tmp_path_factory, preset):
    """The preset's widths with two layers and a short context, as a model folder; with what
    the plain implementation says about the two test sequences."""
    if preset not in _made:
        obj = dict(preset_json(preset), n_layer=LAYERS, n_positions=CONTEXT)
        cfg = GPT2Config.from_json(obj)
        d = write_random_model(tmp_path_factory.mktemp(preset), cfg, 4, std=0.02, bias_std=0.01,
                               gamma_jitter=0.02)
        W = P.PlainWeights(d)
        seqs = [random_tokens(cfg.vocab_size, n, seed=i + 1) for i, n in enumerate(LENGTHS)]
        _made[preset] = (d, seqs, [P.forward_logits(W, t) for t in seqs])
    return _made[preset]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("preset", ["gpt2", "gpt2-medium", "gpt2-xl"])
def test_real_widths_against_the_plain_implementation(tmp_path_factory, preset, dtype):
    d, seqs, refs = _model(tmp_path_factory, preset)
    e = Engine.load(d, dtype=dtype, cache_tokens=1024)
    # each request alone and whole
    for t, ref in zip(seqs, refs):
        s = e.alloc_slot()
        out = e.step([(s, t, list(range(len(t))))])
        e.free_slot(s)
        assert_close(out, ref, dtype, f"{preset} alone, {len(t)} tokens")
    # both prompts in one step (all but the last 8 tokens), then one token each, 8 times
    slots = [e.alloc_slot() for _ in seqs]
    whole = e.step([(s, t[:-8], list(range(len(t) - 8))) for s, t in zip(slots, seqs)])
    steps = [e.step([(s, [t[len(t) - 8 + i]], [0]) for s, t in zip(slots, seqs)]) for i in range(8)]
    for s in slots:
        e.free_slot(s)
    o = 0
    for j, (t, ref) in enumerate(zip(seqs, refs)):
        n = len(t) - 8
        assert_close(whole[o:o + n], ref[:n], dtype, f"{preset} batch prompt {j}")
        assert_close(torch.cat([st[j:j + 1] for st in steps]), ref[n:], dtype,
                     f"{preset} batch decode {j}")
        o += n
    e.ops.check_device_errors()


@pytest.mark.parametrize("preset", ["gpt2", "gpt2-xl"])
def test_bfloat16_follows_float32_at_real_sizes(tmp_path_factory, preset):
    d, seqs, _ = _model(tmp_path_factory, preset)
    outs = {}
    for dtype in DTYPES:
        e = Engine.load(d, dtype=dtype, cache_tokens=1024)
        slots = [e.alloc_slot() for _ in seqs]
        outs[dtype] = e.step([(s, t, [len(t) - 2, len(t) - 1]) for s, t in zip(slots, seqs)])
        e.ops.check_device_errors()
    a, b = outs["bfloat16"].double(), outs["float32"].double()
    assert float((a - b).abs().max() / b.abs().max()) <= TOL["bfloat16"]


@pytest.mark.parametrize("clusters", [1, 0])
def test_a_decode_session_at_real_head_sizes_and_a_long_context(tmp_path_factory, clusters):
    """GPT-2 small's widths and heads (two layers), contexts of 700, 130 and 64 tokens in a
    model of 1,024 positions: the decode session's replayed graph cuts every sequence's 16
    possible pages into splits that merge inside a thread-block cluster (or, with `clusters`
    off, through scratch memory), the long sequence reads eleven pages, the short one crosses
    a page end on its first step.  The logits the session holds after each of 6 steps are the
    plain implementation's."""
    from nimbus_infer_rs_b200.engine.decode import DecodeSession
    obj = dict(preset_json("gpt2"), n_layer=LAYERS, n_positions=1024)
    cfg = GPT2Config.from_json(obj)
    d = write_random_model(tmp_path_factory.mktemp("gpt2_long"), cfg, 5, std=0.02, bias_std=0.01,
                           gamma_jitter=0.02)
    W = P.PlainWeights(d)
    n_steps = 6
    seqs = [random_tokens(cfg.vocab_size, n + n_steps, seed=40 + i) for i, n in enumerate((700, 130, 64))]
    refs = [P.forward_logits(W, t) for t in seqs]
    e = Engine.load(d, dtype="bfloat16", cache_tokens=4096)
    was = e.ops.decode_clusters
    e.ops.set_decode_clusters(clusters)
    try:
        slots = [e.alloc_slot() for _ in seqs]
        e.step([(s, t[:-n_steps - 1], []) for s, t in zip(slots, seqs)])
        session = DecodeSession(e, slots, [t[-n_steps - 1] for t in seqs])
        for k in range(n_steps):
            session.step([t[len(t) - n_steps - 1 + k] for t in seqs])      # the token each row runs now
            session.read_tokens()
            want = torch.stack([ref[len(t) - n_steps - 1 + k] for ref, t in zip(refs, seqs)])
            assert_close(session.logits.clone(), want, "bfloat16", f"long session step {k}")
        assert session._graph is not None
        session.close()
        for s in slots:
            e.free_slot(s)
        e.ops.check_device_errors()
    finally:
        e.ops.set_decode_clusters(was)
