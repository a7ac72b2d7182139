"""Each part of a model alone against plain torch, and the generality of the assembly: a toy
mixer with state of its own and a toy architecture around it are defined HERE, registered,
built, loaded and stepped without any change to the package."""
import json
from dataclasses import dataclass

import pytest
import torch

import plain_gpt2 as P
from nimbus_infer_rs_b200 import Engine, LayerSpec, ModelSpec, PartSpec, register_part
from nimbus_infer_rs_b200.cache import SequenceCache
from nimbus_infer_rs_b200.config import Architecture, register_architecture
from nimbus_infer_rs_b200.config.base import Field, positive, read_fields
from nimbus_infer_rs_b200.csrc import ops as ops_mod
from nimbus_infer_rs_b200.engine.batch import build_layout
from nimbus_infer_rs_b200.engine.context import StepContext
from nimbus_infer_rs_b200.engine.model import Runtime
from nimbus_infer_rs_b200.parts import (MATRIX, Mixer, ParamSpec, StateRequest, bind_params,
                                        build_part, collect_param_specs)
from nimbus_infer_rs_b200.weights import write_safetensors
from nimbus_infer_rs_b200.weights.loader import WeightPlan, take

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
PREC = [("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 2e-2)]


def _ctx(act_dtype, entries=None, pos0=None, cache=None, position=None):
    rt = Runtime(DEV, act_dtype)
    lay = build_layout(entries, pos0, DEV) if entries is not None else None
    return StepContext(rt, ops_mod.backend(), lay, position or build_part("position", PartSpec("none")),
                       cache)


def _bind_random(part, act_dtype, seed, std=0.2):
    g = torch.Generator().manual_seed(seed)
    params = {}
    for name, spec in collect_param_specs(part).items():
        t = torch.randn(*spec.shape, generator=g) * (std if len(spec.shape) > 1 else 0.5)
        dt = act_dtype if spec.role in ("matrix", "table") else torch.float32
        params[name] = t.to(dt).to(DEV)
    bind_params(part, params, None)
    return {k: v.double().cpu() for k, v in params.items()}


def _close(got, ref, tol):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert (got - ref).abs().max() <= tol * ref.abs().max()


@pytest.mark.parametrize("prec, dt, tol", PREC)
def test_norm_part(prec, dt, tol):
    part = build_part("norm", PartSpec("layernorm", {"width": 104, "eps": 2e-4}))
    w = _bind_random(part, dt, 1)
    x = torch.randn(9, 104, device=DEV)
    got = part.forward(_ctx(dt), x)
    assert got.dtype == dt
    _close(got, P.layer_norm(x.double().cpu(), w["weight"], w["bias"], 2e-4), tol)


@pytest.mark.parametrize("prec, dt, tol", PREC)
@pytest.mark.parametrize("act", ["gelu_tanh", "gelu_erf", "none"])
def test_feed_forward_part(prec, dt, tol, act):
    part = build_part("ffn", PartSpec("dense_mlp", {"width": 72, "hidden": 200, "activation": act}))
    w = _bind_random(part, dt, 2)
    h = torch.randn(11, 72, device=DEV).to(dt)
    x = torch.randn(11, 72, device=DEV)
    ref_mid = h.double().cpu() @ w["fc.weight"].t() + w["fc.bias"]
    ref_mid = {"gelu_tanh": P.gelu_tanh, "gelu_erf": P.gelu_erf, "none": lambda v: v}[act](ref_mid)
    ref = x.double().cpu() + ref_mid @ w["proj.weight"].t() + w["proj.bias"]
    part.forward(_ctx(dt), h, x)
    _close(x, ref, tol)


@pytest.mark.parametrize("prec, dt, tol", PREC)
def test_embedding_position_and_head_parts(prec, dt, tol):
    from nimbus_infer_rs_b200.parts import LMHead, TokenEmbedding
    emb = TokenEmbedding(301, 40)
    pos = build_part("position", PartSpec("learned_absolute", {"max_positions": 50, "width": 40}))
    we, wp = _bind_random(emb, dt, 3), _bind_random(pos, dt, 4)
    ctx = _ctx(dt, [(0, [5, 300, 7], []), (1, [9], [])], [10, 49], position=pos)
    x = emb.forward(ctx, pos)
    ref = torch.stack([we["table"][5] + wp["table"][10], we["table"][300] + wp["table"][11],
                       we["table"][7] + wp["table"][12], we["table"][9] + wp["table"][49]])
    _close(x, ref, 1e-6)
    head = LMHead(301, 40, tied=True)
    head.tie(emb.table)
    h = torch.randn(4, 40, device=DEV).to(dt)
    _close(head.forward(ctx, h), h.double().cpu() @ we["table"].t(), tol)
    own = LMHead(301, 40, tied=False)
    wo = _bind_random(own, dt, 5)
    _close(own.forward(ctx, h), h.double().cpu() @ wo["weight"].t(), tol)


@pytest.mark.parametrize("prec, dt, tol", PREC)
@pytest.mark.parametrize("H, Hk, hd, window", [(4, 4, 16, 0), (6, 2, 32, 0), (3, 1, 48, 20)])
def test_attention_part_alone(prec, dt, tol, H, Hk, hd, window):
    """A prompt step, then decode steps, for two sequences of unequal length, against dense
    causal attention with the same weights."""
    width = 56
    part = build_part("mixer", PartSpec("causal_attention", {
        "width": width, "n_heads": H, "n_kv_heads": Hk, "head_dim": hd, "scale": 0.3,
        "window": window}))
    w = _bind_random(part, dt, 6)
    cache = SequenceCache({0: part.cache_request()}, {}, cache_tokens=512, max_seq_len=200,
                          dtype=dt, device=DEV)
    lens = [70, 9]
    hs = [torch.randn(n, width).to(dt) for n in lens]

    def dense(h):
        h = h.double()
        qkv = h @ w["qkv.weight"].t() + w["qkv.bias"]
        n = h.shape[0]
        q = qkv[:, :H * hd].view(n, H, hd)
        k = qkv[:, H * hd:(H + Hk) * hd].view(n, Hk, hd)
        v = qkv[:, (H + Hk) * hd:].view(n, Hk, hd)
        out = torch.zeros(n, H, hd, dtype=torch.float64)
        for t in range(n):
            lo = max(0, t + 1 - window) if window else 0
            for head in range(H):
                s = (k[lo:t + 1, head // (H // Hk)] @ q[t, head]) * 0.3
                out[t, head] = torch.softmax(s, 0) @ v[lo:t + 1, head // (H // Hk)]
        return out.view(n, H * hd) @ w["out.weight"].t() + w["out.bias"]

    refs = [dense(h) for h in hs]
    slots = [cache.alloc_slot() for _ in lens]
    split = [60, 3]                                    # prompt part of each; the rest is decoded
    entries = [(s, [0] * n, []) for s, n in zip(slots, split)]
    cache.reserve([(s, n) for s, n in zip(slots, split)])
    ctx = _ctx(dt, entries, [0, 0], cache)
    ctx.kv = cache.layer_kv(0)
    x = torch.zeros(sum(split), width, device=DEV)
    part.forward(ctx, torch.cat([h[:n] for h, n in zip(hs, split)]).to(DEV), x)
    for s, n in zip(slots, split):
        cache.advance(s, n)
    _close(x, torch.cat([r[:n] for r, n in zip(refs, split)]), tol)
    pos = list(split)
    while any(p < n for p, n in zip(pos, lens)):
        live = [i for i in range(2) if pos[i] < lens[i]]
        cache.reserve([(slots[i], 1) for i in live])
        ctx = _ctx(dt, [(slots[i], [0], []) for i in live], [pos[i] for i in live], cache)
        ctx.kv = cache.layer_kv(0)
        x = torch.zeros(len(live), width, device=DEV)
        part.forward(ctx, torch.stack([hs[i][pos[i]] for i in live]).to(DEV), x)
        _close(x, torch.stack([refs[i][pos[i]] for i in live]), tol)
        for i in live:
            cache.advance(slots[i], 1)
            pos[i] += 1


@pytest.mark.parametrize("prec, dt, tol", PREC)
def test_block_part(prec, dt, tol, model_dirs):
    """The pre-norm arrangement with the real parts equals the plain block."""
    e = Engine.load(model_dirs["B"], dtype=prec, cache_tokens=256)
    W = P.PlainWeights(model_dirs["B"])
    toks = list(range(40, 60))
    s = e.alloc_slot()
    ent = e._check_entries([(s, toks, [])])
    e.cache.reserve([(s, len(toks))])
    ctx = StepContext(e.rt, e.ops, build_layout(ent, [0], DEV), e.model.position, e.cache)
    x = e.model.embedding.forward(ctx, e.model.position)
    cast = P._Cast(W, lambda t: t.double())
    ref = P.embed(toks, cast["wte"], cast["wpe"])
    _close(x, ref, 1e-6)
    layer = e.model.layers[0]
    ctx.kv, ctx.state, ctx.writes_cache = e.model.storage_of(e.cache, 0)
    layer.block.forward(ctx, x, layer)
    _close(x, P.block(ref, cast, 0, W.cfg), tol)


# ---------------------------------------------------------------------------------------
# a toy mixer with state of its own, and a toy architecture, defined in this test
# ---------------------------------------------------------------------------------------
@register_part("mixer", "toy_decay_state", replace=True)
class ToyDecayMixer(Mixer):
    """state <- decay * state + h_t @ W_in ; residual_t += state @ W_out.  The state is a
    fixed-size row per sequence in the cache's state area; there is no key/value cache."""

    def __init__(self, width: int, state_size: int, decay: float):
        self.width, self.state_size, self.decay = width, state_size, decay
        self.w_in = self.w_out = None

    def param_specs(self):
        return {"w_in": ParamSpec((self.state_size, self.width), MATRIX),
                "w_out": ParamSpec((self.width, self.state_size), MATRIX)}

    def state_request(self):
        return StateRequest(self.state_size)

    def forward(self, ctx, h, residual):
        lay = ctx.layout
        u = h.float() @ self.w_in.float().t()
        r = 0
        for slot, n in zip(lay.seq_slots_host, lay.seq_lens):
            for i in range(n):
                ctx.state[slot] = self.decay * ctx.state[slot] + u[r + i]
                residual[r + i] += ctx.state[slot] @ self.w_out.float().t()
            r += n


@dataclass(frozen=True)
class ToyConfig:
    architecture = "toy_state_lm"
    vocab_size: int
    width: int
    n_layers: int
    state_size: int
    decay: float
    max_len: int

    @classmethod
    def from_json(cls, obj):
        v, _ = read_fields(obj, (
            Field("vocab_size", int, ("vocab_size",), required=True, check=positive),
            Field("width", int, ("width",), required=True, check=positive),
            Field("n_layers", int, ("n_layers",), required=True, check=positive),
            Field("state_size", int, ("state_size",), required=True, check=positive),
            Field("decay", float, ("decay",), 0.5),
            Field("max_len", int, ("max_len",), 64, check=positive)))
        return cls(**v)


def _toy_spec(c: ToyConfig) -> ModelSpec:
    norm = PartSpec("layernorm", {"width": c.width, "eps": 1e-5})
    layers = []
    for i in range(c.n_layers):
        # different mixers in different layers of one model: state mixer, then attention
        mixer = (PartSpec("toy_decay_state", {"width": c.width, "state_size": c.state_size,
                                              "decay": c.decay}) if i % 2 == 0 else
                 PartSpec("causal_attention", {"width": c.width, "n_heads": 2, "n_kv_heads": 1,
                                               "head_dim": 16, "scale": 0.25, "bias": False}))
        layers.append(LayerSpec(mixer=mixer, norm_mixer=norm, norm_ffn=norm, ffn=PartSpec(
            "dense_mlp", {"width": c.width, "hidden": 2 * c.width, "activation": "gelu_erf",
                          "bias": False})))
    return ModelSpec("toy_state_lm", c.vocab_size, c.width, c.max_len,
                     position=PartSpec("none", {"max_positions": c.max_len}),
                     layers=tuple(layers), final_norm=norm, tie_head=True,
                     schedule=tuple(range(c.n_layers)) + (0,))     # layer 0 runs twice


def _toy_plan(c, spec, names):
    from nimbus_infer_rs_b200.engine.model import Model
    specs = Model(spec, Runtime(torch.device("cpu"), torch.float32)).param_specs()
    return WeightPlan({path: take(path, s.shape, s.optional) for path, s in specs.items()})


def _toy_reference(t, c: ToyConfig, toks):
    """Plain float64 computation of the toy model on one whole sequence."""
    f = {k: v.double() for k, v in t.items()}
    x = f["embedding.table"][torch.tensor(toks)]
    for li in list(range(c.n_layers)) + [0]:
        p = f"layers.{li}."
        h = P.layer_norm(x, f[p + "norm_mixer.weight"], f[p + "norm_mixer.bias"], 1e-5)
        if li % 2 == 0:
            # storage belongs to the schedule entry: the second run of layer 0 has a state
            # of its own, which also starts from zero
            s = torch.zeros(c.state_size, dtype=torch.float64)
            outs = []
            for tkn in range(len(toks)):
                s = c.decay * s + f[p + "mixer.w_in"] @ h[tkn]
                outs.append(f[p + "mixer.w_out"] @ s)
            x = x + torch.stack(outs)
        else:
            qkv = h @ f[p + "mixer.qkv.weight"].t()
            q, k, v = qkv[:, :32].view(-1, 2, 16), qkv[:, 32:48], qkv[:, 48:]
            o = torch.zeros(len(toks), 2, 16, dtype=torch.float64)
            for tkn in range(len(toks)):
                for hd in range(2):
                    sc = (k[:tkn + 1] @ q[tkn, hd]) * 0.25
                    o[tkn, hd] = torch.softmax(sc, 0) @ v[:tkn + 1]
            x = x + o.view(len(toks), 32) @ f[p + "mixer.out.weight"].t()
        h = P.layer_norm(x, f[p + "norm_ffn.weight"], f[p + "norm_ffn.bias"], 1e-5)
        x = x + P.gelu_erf(h @ f[p + "ffn.fc.weight"].t()) @ f[p + "ffn.proj.weight"].t()
    x = P.layer_norm(x, f["final_norm.weight"], f["final_norm.bias"], 1e-5)
    return x @ f["embedding.table"].t()


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    register_architecture(Architecture("toy_state_lm", ToyConfig, _toy_spec, _toy_plan),
                          replace=True)
    cfg_json = {"architecture": "toy_state_lm", "vocab_size": 97, "width": 40, "n_layers": 3,
                "state_size": 24, "decay": 0.6, "max_len": 96}
    c = ToyConfig.from_json(cfg_json)
    from nimbus_infer_rs_b200.engine.model import Model
    specs = Model(_toy_spec(c), Runtime(torch.device("cpu"), torch.float32)).param_specs()
    g = torch.Generator().manual_seed(0)
    tensors = {p: (torch.randn(*s.shape, generator=g) * (0.3 if len(s.shape) > 1 else 0.2)
                   + (1.0 if p.endswith("norm_mixer.weight") else 0.0)) for p, s in specs.items()}
    (tmp_path / "config.json").write_text(json.dumps(cfg_json))
    write_safetensors(tmp_path / "model.safetensors", tensors)

    e = Engine.load(tmp_path, dtype="float32", cache_tokens=256, n_slots=2)
    assert sorted(e.cache.state) == [0, 2, 3] and len(e.cache.groups) == 1   # schedule entries
    assert e.cache.groups[0].layers == [1]
    seqs = [[3, 9, 27, 81, 50, 53, 62, 89, 73, 25] * 7, [5, 6], [96] * 33]
    refs = [_toy_reference(tensors, c, s) for s in seqs]
    # whole
    for s_, r in zip(seqs, refs):
        slot = e.alloc_slot()
        out = e.step([(slot, s_, list(range(len(s_))))])
        e.free_slot(slot)
        _close(out, r, 2e-5)
    # a batch of two, prompts then token by token, then the third in a reused slot: its state
    # must start from zero although the slot's row held the previous sequence's state
    slots = [e.alloc_slot(), e.alloc_slot()]
    outs = [[], []]
    first = e.step([(slots[0], seqs[0][:60], [59]), (slots[1], seqs[1][:1], [0])])
    outs[0].append(first[0:1]); outs[1].append(first[1:2])
    o = e.step([(slots[0], [seqs[0][60]], [0]), (slots[1], [seqs[1][1]], [0])])
    outs[0].append(o[0:1]); outs[1].append(o[1:2])
    e.free_slot(slots[1])
    for t in seqs[0][61:]:
        outs[0].append(e.step([(slots[0], [t], [0])]))
    _close(torch.cat(outs[0]), refs[0][59:], 2e-5)
    _close(torch.cat(outs[1]), refs[1], 2e-5)
    slot = e.alloc_slot()
    assert slot == slots[1]
    out = e.step([(slot, seqs[2], list(range(33)))])
    _close(out, refs[2], 2e-5)
