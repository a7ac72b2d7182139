"""Real layer sizes (GPT-2 small and XL widths, full vocabulary, a few layers): the bfloat16
engine against the float32 engine on the same seeded weights, whole prompts against token by
token.  The plain implementation is too slow at these sizes; the float32 path, itself checked
against it on the tiny models, is the yardstick here."""
import pytest
import torch

from gpu_helpers import TOL, random_tokens
from nimbus_infer_rs_b200 import Engine
from nimbus_infer_rs_b200.config import GPT2Config

pytestmark = pytest.mark.gpu

SIZES = {
    "small": {"vocab_size": 50257, "n_positions": 320, "n_embd": 768, "n_layer": 3, "n_head": 12,
              "activation_function": "gelu_new", "model_type": "gpt2"},
    "xl": {"vocab_size": 50257, "n_positions": 200, "n_embd": 1600, "n_layer": 2, "n_head": 25,
           "activation_function": "gelu_new", "model_type": "gpt2"},
}


def _rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max())


@pytest.mark.parametrize("name", list(SIZES))
def test_bfloat16_follows_float32_at_real_sizes(name):
    cfg = GPT2Config.from_json(SIZES[name])
    opts = dict(seed=4, cache_tokens=1024, std=0.02, bias_std=0.01, gamma_jitter=0.02)
    e32 = Engine.random(cfg, dtype="float32", **opts)
    e16 = Engine.random(cfg, dtype="bfloat16", **opts)
    n = cfg.max_seq_len - 8
    seqs = [random_tokens(cfg.vocab_size, n, seed=1), random_tokens(cfg.vocab_size, 37, seed=2)]
    out = {}
    for tag, e in (("f32", e32), ("b16", e16)):
        slots = [e.alloc_slot() for _ in seqs]
        whole = e.step([(s, t[:-8], list(range(len(t) - 8))) for s, t in zip(slots, seqs)])
        steps = [e.step([(s, [t[len(t) - 8 + i]], [0]) for s, t in zip(slots, seqs)])
                 for i in range(8)]
        out[tag] = (whole, torch.cat(steps))
        # the same positions again, each sequence alone and whole: cutting changes nothing
        for s in slots:
            e.free_slot(s)
        s = e.alloc_slot()
        alone = e.step([(s, seqs[1], list(range(len(seqs[1]))))])
        e.free_slot(s)
        first = len(seqs[0]) - 8
        cut = torch.cat([whole[first:], torch.cat(steps)[1::2]])
        assert _rel(cut, alone) <= (2 * TOL["float32"] if tag == "f32" else TOL["bfloat16"]), tag
        e.ops.check_device_errors()
    assert _rel(out["b16"][0], out["f32"][0]) <= TOL["bfloat16"]
    assert _rel(out["b16"][1], out["f32"][1]) <= TOL["bfloat16"]
