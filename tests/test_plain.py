"""The plain implementation itself: the reference's unit-test values and the golden file."""
import json
from pathlib import Path

import pytest
import torch

import plain_gpt2 as P

GOLDEN = Path(__file__).parent / "golden"


def test_gelu_values_of_the_reference():       # src/ops.rs:66-73
    for x, want in [(0.0, 0.0), (1.0, 0.841192), (-1.0, -0.158808), (3.0, 2.996363)]:
        assert abs(float(P.gelu_tanh(torch.tensor(x, dtype=torch.float64))) - want) < 1e-4
    assert abs(float(P.gelu_erf(torch.tensor(1.0, dtype=torch.float64))) - 0.8413447) < 1e-6


def test_softmax_is_stable_and_sums_to_one():  # src/ops.rs:56-64
    p = P.softmax_row(torch.tensor([1000.0, 1001.0, 999.0]))
    assert abs(float(p.sum()) - 1) < 1e-6 and p[1] > p[0] > 0 and torch.isfinite(p).all()


def test_layer_norm_normalises():              # src/ops.rs:75-85
    y = P.layer_norm(torch.tensor([[1.0, 2.0, 3.0, 4.0]]), torch.ones(4), torch.zeros(4), 1e-5)
    assert abs(float(y.mean())) < 1e-5 and abs(float((y ** 2).mean()) - 1) < 1e-3


def test_causality_and_float32_agreement(model_dirs):
    W = P.PlainWeights(model_dirs["C"])
    toks = list(range(3, 40))
    full = P.forward_logits(W, toks)
    part = P.forward_logits(W, toks[:20])
    assert torch.allclose(full[:20], part, atol=1e-10)           # later tokens change nothing
    f32 = P.forward_logits(W, toks, dtype=torch.float32)
    assert (f32.double() - full).abs().max() < 2e-5 * full.abs().max()


def test_both_naming_schemes_read_the_same(model_dirs, tmp_path):
    from nimbus_infer_rs_b200.config import GPT2Config
    from nimbus_infer_rs_b200.models.gpt2 import random_tensors as gpt2_tensors
    from nimbus_infer_rs_b200.weights import write_safetensors
    from tiny_configs import TINY_A
    cfg = GPT2Config.from_json(TINY_A)
    for scheme in ("nimbus", "checkpoint"):
        d = tmp_path / scheme
        d.mkdir()
        (d / "config.json").write_text(json.dumps(TINY_A))
        write_safetensors(d / "model.safetensors", gpt2_tensors(cfg, 4, bias_std=0.01, scheme=scheme))
    a = P.forward_logits(P.PlainWeights(tmp_path / "nimbus"), [1, 2, 3, 4])
    b = P.forward_logits(P.PlainWeights(tmp_path / "checkpoint"), [1, 2, 3, 4])
    assert torch.allclose(a, b, atol=1e-12)


@pytest.mark.parametrize("name", ["A", "B"])
def test_golden_outputs(name, tmp_path):
    """The committed outputs of tests/golden/make_golden.py are reproduced."""
    from make_golden_lib import build_case
    case = json.loads((GOLDEN / f"tiny_{name}.json").read_text())
    got = build_case(name, tmp_path)
    assert got["greedy"] == case["greedy"]
    for k in ("last_logits_head", "last_logits_tail"):
        assert torch.allclose(torch.tensor(got[k]), torch.tensor(case[k]), atol=1e-9)
    assert got["argmax"] == case["argmax"]
