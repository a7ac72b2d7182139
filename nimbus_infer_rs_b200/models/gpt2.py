"""GPT-2 as data: how its configuration maps onto parts, and where its parameters are found
in a weight file.  This is the only file that knows the architecture.

Structure (src/model.rs:271-325): learned absolute positions added to the token embedding;
``n_layers`` pre-norm blocks of LayerNorm → causal attention → residual, LayerNorm → GELU
MLP → residual; a final LayerNorm; logits through the token embedding (tied) or ``lm_head``.

Two naming schemes are read:

* the reference's (src/engine.rs:110-225): ``wte``, ``wpe``, ``h.N.norm1.{weight,bias}``,
  ``h.N.attn.{q,k,v,o}.{weight,bias}``, ``h.N.mlp.{fc,proj}.{weight,bias}``,
  ``h.N.norm2.*``, ``norm_f.*``, ``lm_head.weight``; every linear weight stored
  ``(in, out)`` (src/engine.rs:93);
* published GPT-2 checkpoints: ``wte.weight``, ``wpe.weight``, ``h.N.ln_1``,
  ``h.N.attn.c_attn`` (queries, keys, values side by side), ``h.N.attn.c_proj``, ``h.N.ln_2``,
  ``h.N.mlp.c_fc``, ``h.N.mlp.c_proj``, ``ln_f``, optionally under ``transformer.``; linear
  weights stored ``(in, out)``, ``lm_head.weight`` stored ``(vocab, width)``.  The mask
  buffers ``h.N.attn.bias`` / ``h.N.attn.masked_bias`` are no weights
  (scripts/remap_gpt2_safetensors.py:28-34).
"""
from __future__ import annotations

import torch

from ..config.gpt2 import GPT2Config
from ..config.registry import Architecture, register_architecture
from ..engine.spec import LayerSpec, ModelSpec
from ..parts.base import PartSpec
from ..weights.loader import (Recipe, Source, WeightPlan, concat_optional_vectors,
                              concat_transposed, take, take_transposed)


def build_spec(cfg: GPT2Config) -> ModelSpec:
    norm = PartSpec("layernorm", {"width": cfg.d_model, "eps": cfg.norm_eps})
    layers = []
    for i in range(cfg.n_layers):
        layers.append(LayerSpec(
            mixer=PartSpec("causal_attention", {
                "width": cfg.d_model, "n_heads": cfg.n_heads, "n_kv_heads": cfg.n_kv_heads,
                "head_dim": cfg.head_dim, "scale": cfg.attn_scale(i)}),
            ffn=PartSpec("dense_mlp", {"width": cfg.d_model, "hidden": cfg.d_mlp,
                                       "activation": cfg.activation}),
            norm_mixer=norm, norm_ffn=norm, block=PartSpec("pre_norm")))
    return ModelSpec(
        architecture="gpt2", vocab_size=cfg.vocab_size, width=cfg.d_model,
        max_seq_len=cfg.max_seq_len,
        position=PartSpec("learned_absolute", {"max_positions": cfg.max_seq_len,
                                               "width": cfg.d_model}),
        layers=tuple(layers), final_norm=norm, tie_head=cfg.tie_embeddings)


def _head_recipe(name: str, vocab: int, width: int, stored_in_out: bool) -> Recipe:
    """``lm_head.weight`` in either orientation; when both sizes are equal the scheme's own
    orientation decides."""
    def combine(ts):
        t = ts[0]
        if tuple(t.shape) == (vocab, width) and not (vocab == width and stored_in_out):
            return t
        return t.t().contiguous()
    return Recipe([Source(name, ((vocab, width), (width, vocab)))], combine)


def weight_plan(cfg: GPT2Config, spec: ModelSpec, names: set[str]) -> WeightPlan:
    d, m, V, P = cfg.d_model, cfg.d_mlp, cfg.vocab_size, cfg.max_seq_len
    hq, hk = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    prefix = "transformer." if any(n.startswith("transformer.") for n in names) else ""
    checkpoint_style = (prefix + "wte.weight") in names or (
        "wte" not in names and any(".ln_1." in n or ".c_attn." in n for n in names))
    r: dict[str, Recipe] = {}
    ignored: set[str] = set()

    if not checkpoint_style:
        r["embedding.table"] = take("wte", (V, d))
        r["position.table"] = take("wpe", (P, d))
        for i in range(cfg.n_layers):
            p, L = f"h.{i}.", f"layers.{i}."
            for ours, theirs in (("norm_mixer", "norm1"), ("norm_ffn", "norm2")):
                r[f"{L}{ours}.weight"] = take(f"{p}{theirs}.weight", (d,))
                r[f"{L}{ours}.bias"] = take(f"{p}{theirs}.bias", (d,))
            r[f"{L}mixer.qkv.weight"] = concat_transposed([
                (f"{p}attn.q.weight", (d, hq)), (f"{p}attn.k.weight", (d, hk)),
                (f"{p}attn.v.weight", (d, hk))])
            r[f"{L}mixer.qkv.bias"] = concat_optional_vectors([
                (f"{p}attn.q.bias", hq), (f"{p}attn.k.bias", hk), (f"{p}attn.v.bias", hk)])
            r[f"{L}mixer.out.weight"] = take_transposed(f"{p}attn.o.weight", (hq, d))
            r[f"{L}mixer.out.bias"] = take(f"{p}attn.o.bias", (d,), optional=True)
            r[f"{L}ffn.fc.weight"] = take_transposed(f"{p}mlp.fc.weight", (d, m))
            r[f"{L}ffn.fc.bias"] = take(f"{p}mlp.fc.bias", (m,), optional=True)
            r[f"{L}ffn.proj.weight"] = take_transposed(f"{p}mlp.proj.weight", (m, d))
            r[f"{L}ffn.proj.bias"] = take(f"{p}mlp.proj.bias", (d,), optional=True)
        r["final_norm.weight"] = take("norm_f.weight", (d,))
        r["final_norm.bias"] = take("norm_f.bias", (d,))
        if not cfg.tie_embeddings:
            r["head.weight"] = _head_recipe("lm_head.weight", V, d, stored_in_out=True)
        return WeightPlan(r, ignored)

    t = prefix
    r["embedding.table"] = take(f"{t}wte.weight", (V, d))
    r["position.table"] = take(f"{t}wpe.weight", (P, d))
    for i in range(cfg.n_layers):
        p, L = f"{t}h.{i}.", f"layers.{i}."
        for ours, theirs in (("norm_mixer", "ln_1"), ("norm_ffn", "ln_2")):
            r[f"{L}{ours}.weight"] = take(f"{p}{theirs}.weight", (d,))
            r[f"{L}{ours}.bias"] = take(f"{p}{theirs}.bias", (d,))
        r[f"{L}mixer.qkv.weight"] = take_transposed(f"{p}attn.c_attn.weight", (d, hq + 2 * hk))
        r[f"{L}mixer.qkv.bias"] = take(f"{p}attn.c_attn.bias", (hq + 2 * hk,), optional=True)
        r[f"{L}mixer.out.weight"] = take_transposed(f"{p}attn.c_proj.weight", (hq, d))
        r[f"{L}mixer.out.bias"] = take(f"{p}attn.c_proj.bias", (d,), optional=True)
        r[f"{L}ffn.fc.weight"] = take_transposed(f"{p}mlp.c_fc.weight", (d, m))
        r[f"{L}ffn.fc.bias"] = take(f"{p}mlp.c_fc.bias", (m,), optional=True)
        r[f"{L}ffn.proj.weight"] = take_transposed(f"{p}mlp.c_proj.weight", (m, d))
        r[f"{L}ffn.proj.bias"] = take(f"{p}mlp.c_proj.bias", (d,), optional=True)
        ignored.update({f"{p}attn.bias", f"{p}attn.masked_bias"})
    r["final_norm.weight"] = take(f"{t}ln_f.weight", (d,))
    r["final_norm.bias"] = take(f"{t}ln_f.bias", (d,))
    if cfg.tie_embeddings:
        ignored.add("lm_head.weight")   # a stored copy of the tied table
    else:
        r["head.weight"] = _head_recipe("lm_head.weight", V, d, stored_in_out=False)
    return WeightPlan(r, ignored)


def random_tensors(cfg: GPT2Config, seed: int, *, std: float = 0.02, bias_std: float = 0.0,
                 gamma_jitter: float = 0.0, beta_std: float = 0.0,
                 dtype: torch.dtype = torch.bfloat16, scheme: str = "nimbus") -> dict:
    """Random GPT-2 tensors under the names of ``scheme``: ``"nimbus"`` (the reference's,
    src/engine.rs:110-225) or ``"checkpoint"`` (published GPT-2 files: fused ``c_attn``).

    The reference's fixture has matrices and embeddings ~N(0, 0.02), norm weights 1, norm
    biases 0 and no linear biases (benchmarks/cross_engine.py:43-64); here the standard
    deviations are arguments so that tests can give biases and norm weights a spread too.
    Values are drawn in fp32 from a seeded CPU generator, one tensor after another in a fixed
    order, then rounded to the storage type: matrices and tables are stored in ``dtype``
    (bfloat16 by default, the serving precision), vectors in fp32."""
    if scheme not in ("nimbus", "checkpoint"):
        raise ValueError("scheme must be 'nimbus' or 'checkpoint'")
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    d, m, V, P = cfg.d_model, cfg.d_mlp, cfg.vocab_size, cfg.max_seq_len
    hq, hk = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim

    def mat(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(dtype)

    def vec(n, s, mean=0.0):
        if s > 0:
            return torch.randn(n, generator=g, dtype=torch.float32) * s + mean
        return torch.full((n,), mean, dtype=torch.float32)

    out: dict[str, torch.Tensor] = {}
    ck = scheme == "checkpoint"
    out["wte.weight" if ck else "wte"] = mat(V, d)
    out["wpe.weight" if ck else "wpe"] = mat(P, d)
    for i in range(cfg.n_layers):
        p = f"h.{i}."
        n1, n2 = ("ln_1", "ln_2") if ck else ("norm1", "norm2")
        out[f"{p}{n1}.weight"] = vec(d, gamma_jitter, 1.0)
        out[f"{p}{n1}.bias"] = vec(d, beta_std)
        q, k, v = mat(d, hq), mat(d, hk), mat(d, hk)       # stored (in, out)
        if ck:
            out[f"{p}attn.c_attn.weight"] = torch.cat([q, k, v], dim=1).contiguous()
            if bias_std > 0:
                out[f"{p}attn.c_attn.bias"] = vec(hq + 2 * hk, bias_std)
            out[f"{p}attn.c_proj.weight"] = mat(hq, d)
            if bias_std > 0:
                out[f"{p}attn.c_proj.bias"] = vec(d, bias_std)
        else:
            out[f"{p}attn.q.weight"], out[f"{p}attn.k.weight"], out[f"{p}attn.v.weight"] = q, k, v
            if bias_std > 0:
                out[f"{p}attn.q.bias"] = vec(hq, bias_std)
                out[f"{p}attn.k.bias"] = vec(hk, bias_std)
                out[f"{p}attn.v.bias"] = vec(hk, bias_std)
            out[f"{p}attn.o.weight"] = mat(hq, d)
            if bias_std > 0:
                out[f"{p}attn.o.bias"] = vec(d, bias_std)
        out[f"{p}{n2}.weight"] = vec(d, gamma_jitter, 1.0)
        out[f"{p}{n2}.bias"] = vec(d, beta_std)
        fc, pj = ("mlp.c_fc", "mlp.c_proj") if ck else ("mlp.fc", "mlp.proj")
        out[f"{p}{fc}.weight"] = mat(d, m)
        if bias_std > 0:
            out[f"{p}{fc}.bias"] = vec(m, bias_std)
        out[f"{p}{pj}.weight"] = mat(m, d)
        if bias_std > 0:
            out[f"{p}{pj}.bias"] = vec(d, bias_std)
    nf = "ln_f" if ck else "norm_f"
    out[f"{nf}.weight"] = vec(d, gamma_jitter, 1.0)
    out[f"{nf}.bias"] = vec(d, beta_std)
    if not cfg.tie_embeddings:
        out["lm_head.weight"] = mat(V, d) if ck else mat(d, V)
    return out


def _recognises(obj: dict) -> bool:
    """A config.json in the reference's style is GPT-2 when its three switches say so
    (src/config.rs:56-58 are the defaults)."""
    return (obj.get("norm", "layernorm") == "layernorm"
            and obj.get("pos_encoding", "learned") == "learned"
            and obj.get("activation", "gelu") != "swiglu")


ARCHITECTURE = register_architecture(Architecture(
    name="gpt2", config_cls=GPT2Config, build_spec=build_spec, weight_plan=weight_plan,
    aliases=("GPT2LMHeadModel", "GPT2Model", "gpt-2"), recognises=_recognises,
    random_tensors=random_tensors), replace=True)
