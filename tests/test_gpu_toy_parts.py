"""Generality of the assembly, shown with toy parts that exist only in this file: a position
encoding that turns queries and keys, a feed-forward that routes every token to one of a few
experts, and an architecture whose layers differ -- full and windowed attention with cache
groups of their own, and layers that read another layer's keys and values.  Everything is
registered, built, loaded from a model folder and stepped without a change to the package,
and compared with a float64 computation of whole sequences written out below."""
import json
from dataclasses import dataclass

import pytest
import torch

import plain_gpt2 as P
from nimbus_infer_rs_b200 import Engine, LayerSpec, ModelSpec, PartSpec, register_part
from nimbus_infer_rs_b200.cache import PAGE
from nimbus_infer_rs_b200.config import Architecture, register_architecture
from nimbus_infer_rs_b200.engine.model import Model, Runtime
from nimbus_infer_rs_b200.parts import MATRIX, FeedForward, ParamSpec, Position
from nimbus_infer_rs_b200.weights import write_safetensors
from nimbus_infer_rs_b200.weights.loader import WeightPlan, take

pytestmark = pytest.mark.gpu
THETA = 0.37


@register_part("position", "toy_single_angle", replace=True)
class ToySingleAngle(Position):
    """Turns every (even, odd) pair of each query and key head by ``position * theta``: one
    angle for all pairs.  Nothing is added to the embedding."""

    def __init__(self, theta: float, max_positions: int):
        self.theta, self.max_positions = float(theta), int(max_positions)
        self.table = None

    def rotate(self, ctx, qkv, mixer):
        n = mixer.q_width + mixer.kv_width
        ang = ctx.layout.row_pos.clamp(min=0).to(torch.float32) * self.theta
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        x = qkv[:, :n].float().reshape(qkv.shape[0], n // 2, 2)
        a, b = x[..., 0], x[..., 1]
        qkv[:, :n] = torch.stack((a * c - b * s, a * s + b * c), dim=-1).reshape(
            qkv.shape[0], n).to(qkv.dtype)


@register_part("ffn", "toy_top1_experts", replace=True)
class ToyTop1Experts(FeedForward):
    """Each token goes to the expert with the largest router logit (fp32); an expert is
    ``relu(h @ up.T) @ down.T``."""

    def __init__(self, width: int, hidden: int, n_experts: int):
        self.width, self.hidden, self.n_experts = int(width), int(hidden), int(n_experts)
        self.router = self.up = self.down = None

    def param_specs(self):
        return {"router": ParamSpec((self.n_experts, self.width), MATRIX),
                "up": ParamSpec((self.n_experts * self.hidden, self.width), MATRIX),
                "down": ParamSpec((self.n_experts * self.width, self.hidden), MATRIX)}

    def forward(self, ctx, h, residual):
        hf = h.float()
        choice = (hf @ self.router.float().t()).argmax(dim=1)
        for e in range(self.n_experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            up = self.up.float()[e * self.hidden:(e + 1) * self.hidden]
            down = self.down.float()[e * self.width:(e + 1) * self.width]
            residual[rows] += torch.relu(hf[rows] @ up.t()) @ down.t()


@dataclass(frozen=True)
class MixedConfig:
    architecture = "toy_mixed_lm"
    vocab_size: int
    width: int
    max_len: int
    hidden: int
    n_experts: int

    @classmethod
    def from_json(cls, obj):
        return cls(*(int(obj[k]) for k in ("vocab_size", "width", "max_len", "hidden", "n_experts")))


# layer: (query heads, key/value heads, head size, window, layer whose cache it reads)
LAYERS = [(4, 2, 16, 0, None), (2, 1, 32, 70, None), (4, 2, 16, 0, 0), (2, 1, 32, 40, 1)]


def _spec(c: MixedConfig) -> ModelSpec:
    norm = PartSpec("layernorm", {"width": c.width, "eps": 1e-5})
    layers = []
    for i, (h, hk, hd, window, src) in enumerate(LAYERS):
        mixer = PartSpec("causal_attention", {"width": c.width, "n_heads": h, "n_kv_heads": hk,
                                              "head_dim": hd, "scale": hd ** -0.5,
                                              "window": window, "bias": False})
        ffn = (PartSpec("dense_mlp", {"width": c.width, "hidden": c.hidden,
                                      "activation": "gelu_tanh", "bias": False}) if i % 2 == 0 else
               PartSpec("toy_top1_experts", {"width": c.width, "hidden": c.hidden,
                                             "n_experts": c.n_experts}))
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm_mixer=norm, norm_ffn=norm,
                                cache_from=src))
    return ModelSpec("toy_mixed_lm", c.vocab_size, c.width, c.max_len,
                     position=PartSpec("toy_single_angle", {"theta": THETA,
                                                            "max_positions": c.max_len}),
                     layers=tuple(layers), final_norm=norm, tie_head=True)


def _plan(c, spec, names):
    specs = Model(spec, Runtime(torch.device("cpu"), torch.float32)).param_specs()
    return WeightPlan({path: take(path, s.shape, s.optional) for path, s in specs.items()})


def _turn(x, n_heads, hd):
    """x [T, n_heads * hd]: pairs turned by position * THETA, as the toy encoding does."""
    T = x.shape[0]
    ang = torch.arange(T, dtype=torch.float64) * THETA
    c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
    p = x.reshape(T, n_heads * hd // 2, 2)
    a, b = p[..., 0], p[..., 1]
    return torch.stack((a * c - b * s, a * s + b * c), dim=-1).reshape(T, n_heads * hd)


def _reference(t, c: MixedConfig, toks):
    f = {k: v.double() for k, v in t.items()}
    T = len(toks)
    x = f["embedding.table"][torch.tensor(toks)]
    kept = {}                                         # layer -> (keys, values) it wrote
    for li, (H, Hk, hd, window, src) in enumerate(LAYERS):
        p = f"layers.{li}."
        h = P.layer_norm(x, f[p + "norm_mixer.weight"], f[p + "norm_mixer.bias"], 1e-5)
        qkv = h @ f[p + "mixer.qkv.weight"].t()
        q = _turn(qkv[:, :H * hd], H, hd).view(T, H, hd)
        if src is None:
            k = _turn(qkv[:, H * hd:(H + Hk) * hd], Hk, hd).view(T, Hk, hd)
            v = qkv[:, (H + Hk) * hd:].view(T, Hk, hd)
            kept[li] = (k, v)
        else:
            k, v = kept[src]
        o = torch.zeros(T, H, hd, dtype=torch.float64)
        for tkn in range(T):
            lo = max(0, tkn + 1 - window) if window else 0
            for hh in range(H):
                g = hh // (H // Hk)
                sc = (k[lo:tkn + 1, g] @ q[tkn, hh]) * hd ** -0.5
                o[tkn, hh] = torch.softmax(sc, 0) @ v[lo:tkn + 1, g]
        x = x + o.view(T, H * hd) @ f[p + "mixer.out.weight"].t()
        h = P.layer_norm(x, f[p + "norm_ffn.weight"], f[p + "norm_ffn.bias"], 1e-5)
        if li % 2 == 0:
            x = x + P.gelu_tanh(h @ f[p + "ffn.fc.weight"].t()) @ f[p + "ffn.proj.weight"].t()
        else:
            choice = (h @ f[p + "ffn.router"].t()).argmax(dim=1)
            add = torch.zeros_like(x)
            for tkn in range(T):
                e = int(choice[tkn])
                up = f[p + "ffn.up"][e * c.hidden:(e + 1) * c.hidden]
                down = f[p + "ffn.down"][e * c.width:(e + 1) * c.width]
                add[tkn] = down @ torch.relu(up @ h[tkn])
            x = x + add
    x = P.layer_norm(x, f["final_norm.weight"], f["final_norm.bias"], 1e-5)
    return x @ f["embedding.table"].t()


def _close(got, ref, tol=2e-5):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert (got - ref).abs().max() <= tol * ref.abs().max()


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    register_architecture(Architecture("toy_mixed_lm", MixedConfig, _spec, _plan), replace=True)
    cfg_json = {"architecture": "toy_mixed_lm", "vocab_size": 131, "width": 48, "max_len": 256,
                "hidden": 72, "n_experts": 3}
    c = MixedConfig.from_json(cfg_json)
    specs = Model(_spec(c), Runtime(torch.device("cpu"), torch.float32)).param_specs()
    g = torch.Generator().manual_seed(3)
    tensors = {}
    for path, s in specs.items():
        std = 0.25 if len(s.shape) > 1 else 0.1
        if path.endswith("router"):
            std = 2.0                                  # clear choices: no near ties
        tensors[path] = torch.randn(*s.shape, generator=g) * std + (
            1.0 if path.endswith(("norm_mixer.weight", "norm_ffn.weight", "final_norm.weight"))
            else 0.0)
    folder = tmp_path_factory.mktemp("toy_mixed")
    (folder / "config.json").write_text(json.dumps(cfg_json))
    write_safetensors(folder / "model.safetensors", tensors)
    g2 = torch.Generator().manual_seed(4)
    seqs = [torch.randint(0, 131, (n,), generator=g2).tolist() for n in (200, 7, 150)]
    refs = [_reference(tensors, c, s) for s in seqs]
    return folder, seqs, refs


def test_groups_and_readers_of_the_toy_architecture(toy):
    folder, _, _ = toy
    e = Engine.load(folder, dtype="float32", cache_tokens=512, n_slots=2)
    # entries 0 and 1 keep keys and values (two groups: all keys / a window); 2 and 3 read them
    assert [g.layers for g in e.cache.groups] == [[0], [1]]
    assert [g.request.window for g in e.cache.groups] == [0, 70]
    assert e.model.kv_source(2) == 0 and e.model.kv_source(3) == 1
    assert not e.graph_safe                           # the toy parts work on the host


def test_toy_architecture_whole_sequences(toy):
    folder, seqs, refs = toy
    e = Engine.load(folder, dtype="float32", cache_tokens=512, n_slots=2)
    for s_, r in zip(seqs, refs):
        slot = e.alloc_slot()
        out = e.step([(slot, s_, list(range(len(s_))))])
        e.free_slot(slot)
        _close(out, r)


def test_toy_architecture_in_steps_with_pages_given_back(toy):
    """Prompts of unequal length in one step, then token by token; the shorter request ends
    first and its slot is used again.  The window group holds three pages at most while the
    group without a window holds them all."""
    folder, seqs, refs = toy
    e = Engine.load(folder, dtype="float32", cache_tokens=512, n_slots=2)
    full, win = e.cache.groups
    a, b = e.alloc_slot(), e.alloc_slot()
    cut = (100, 3)
    got = [[], []]
    out = e.step([(a, seqs[0][:cut[0]], list(range(cut[0]))), (b, seqs[1][:cut[1]], list(range(cut[1])))])
    got[0].append(out[:cut[0]]); got[1].append(out[cut[0]:])
    pos = list(cut)
    while pos[1] < len(seqs[1]):
        out = e.step([(a, [seqs[0][pos[0]]], [0]), (b, [seqs[1][pos[1]]], [0])])
        got[0].append(out[0:1]); got[1].append(out[1:2])
        pos[0] += 1; pos[1] += 1
    e.free_slot(b)
    _close(torch.cat(got[1]), refs[1])
    # the third request starts in the slot that was given back, while the first goes on
    # alone for a while (a batch has started: nobody joins it)
    while pos[0] < len(seqs[0]):
        out = e.step([(a, [seqs[0][pos[0]]], [0])])
        got[0].append(out)
        pos[0] += 1
        assert len(win.pages_of(a)) <= 3
        assert len(full.pages_of(a)) == (pos[0] + PAGE - 1) // PAGE
    _close(torch.cat(got[0]), refs[0])
    assert len(win.pages_of(a)) < len(full.pages_of(a))          # pages were given back
    b2 = e.alloc_slot()
    assert b2 == b
    out = e.step([(b2, seqs[2], list(range(len(seqs[2]))))])
    _close(out, refs[2])
    e.free_slot(a)
    e.free_slot(b2)
    assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)


def test_a_reader_must_want_what_the_owner_keeps():
    c = MixedConfig(131, 48, 256, 72, 3)
    spec = _spec(c)
    bad = list(spec.layers)
    wide = PartSpec("causal_attention", {**spec.layers[3].mixer.args, "window": 90})
    bad[3] = LayerSpec(mixer=wide, ffn=bad[3].ffn, norm_mixer=bad[3].norm_mixer,
                       norm_ffn=bad[3].norm_ffn, cache_from=1)
    m = Model(ModelSpec("toy_mixed_lm", 131, 48, 256, spec.position, tuple(bad), spec.final_norm),
              Runtime(torch.device("cpu"), torch.float32))
    with pytest.raises(ValueError, match="reads the cache of layer 1"):
        m.storage_requests()
