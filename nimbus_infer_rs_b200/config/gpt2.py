"""Typed configuration of the GPT-2 decoder.

Keys, meanings and defaults follow the reference's ``ModelConfig``
(src/config.rs:8-25 fields, :45-66 defaults, :69-133 parsing, :142-173 checks and
derived values).  The spellings used by published GPT-2 checkpoints (``n_embd``,
``n_layer``, ``n_head``, ``n_inner``, ``n_positions``, ``layer_norm_epsilon``,
``activation_function``, ``tie_word_embeddings``, ``scale_attn_weights``) are
accepted as aliases of the same fields.

Two options go beyond the reference: ``activation`` may be the exact (erf) GELU,
and ``scale_attn_by_inverse_layer_idx`` divides a layer's scores by its 1-based
index.  A missing ``d_mlp`` means four times ``d_model`` (for the default width that
is the reference's default of 3072, src/config.rs:52).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict, replace
from pathlib import Path
from typing import Any

from .base import ConfigError, Field, load_json, positive, read_fields

ACT_TANH = "gelu_tanh"
ACT_ERF = "gelu_erf"

# The reference's spelling "gelu" is the tanh form (src/config.rs:104, src/ops.rs:21-24).
_NIMBUS_ACTIVATIONS = {
    "gelu": ACT_TANH,
    "gelu_new": ACT_TANH,
    "gelu_tanh": ACT_TANH,
    "gelu_pytorch_tanh": ACT_TANH,
    "gelu_erf": ACT_ERF,
    "gelu_exact": ACT_ERF,
}
# In checkpoint-style configs "gelu" is the exact form and "gelu_new" the tanh form.
_CHECKPOINT_ACTIVATIONS = dict(_NIMBUS_ACTIVATIONS, gelu=ACT_ERF)

_NIMBUS_KEYS = ("d_model", "n_layers", "n_heads", "d_mlp", "max_seq_len", "norm",
                "pos_encoding", "tie_embeddings", "norm_eps")

_FIELDS = (
    Field("vocab_size", int, ("vocab_size",), 50257, check=positive),
    Field("n_layers", int, ("n_layers", "n_layer", "num_hidden_layers"), 12, check=positive),
    Field("n_heads", int, ("n_heads", "n_head", "num_attention_heads"), 12, check=positive),
    Field("d_model", int, ("d_model", "n_embd", "hidden_size"), 768, check=positive),
    Field("d_mlp", int, ("d_mlp", "n_inner", "intermediate_size"), None, check=positive),
    Field("max_seq_len", int, ("max_seq_len", "n_positions", "n_ctx",
                               "max_position_embeddings"), 1024, check=positive),
    Field("head_dim", int, ("head_dim",), None, check=positive),
    Field("n_kv_heads", int, ("n_kv_heads", "num_key_value_heads"), None, check=positive),
    Field("norm", str, ("norm",), "layernorm"),
    Field("pos_encoding", str, ("pos_encoding",), "learned"),
    Field("tie_embeddings", bool, ("tie_embeddings", "tie_word_embeddings"), True),
    Field("norm_eps", float, ("norm_eps", "layer_norm_epsilon", "layer_norm_eps"), 1e-5,
          check=positive),
    Field("scale_attn_by_head_dim", bool, ("scale_attn_by_head_dim", "scale_attn_weights"),
          True),
    Field("scale_attn_by_inverse_layer_idx", bool, ("scale_attn_by_inverse_layer_idx",),
          False),
    Field("name", str, ("name", "_name_or_path"), "model"),
)


@dataclass(frozen=True)
class GPT2Config:
    architecture = "gpt2"

    vocab_size: int
    n_layers: int
    n_heads: int
    d_model: int
    d_mlp: int
    max_seq_len: int
    head_dim: int
    n_kv_heads: int
    activation: str
    tie_embeddings: bool
    norm_eps: float
    scale_attn_by_head_dim: bool
    scale_attn_by_inverse_layer_idx: bool
    name: str = "model"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_json(cls, obj: dict) -> "GPT2Config":
        values, _ = read_fields(obj, _FIELDS)
        if values["norm"] != "layernorm":
            raise ConfigError(
                f"architecture not supported: gpt2 needs norm 'layernorm', got {values['norm']!r}")
        if values["pos_encoding"] != "learned":
            raise ConfigError(
                "architecture not supported: gpt2 needs pos_encoding 'learned', got "
                f"{values['pos_encoding']!r}")
        values.pop("norm")
        values.pop("pos_encoding")
        values["activation"] = _read_activation(obj)
        if values["d_mlp"] is None:
            values["d_mlp"] = 4 * values["d_model"]
        if values["head_dim"] is None:
            # src/config.rs:142-156
            if values["d_model"] % values["n_heads"] != 0:
                raise ConfigError(
                    "d_model must be divisible by n_heads when head_dim is unset "
                    f"({values['d_model']} % {values['n_heads']} != 0)")
            values["head_dim"] = values["d_model"] // values["n_heads"]
        if values["n_kv_heads"] is None:
            values["n_kv_heads"] = values["n_heads"]
        cfg = cls(**values)
        cfg.validate()
        return cfg

    @classmethod
    def load(cls, path: str | Path) -> "GPT2Config":
        return cls.from_json(load_json(path))

    def validate(self) -> None:
        if self.n_heads % self.n_kv_heads != 0:  # src/config.rs:146-150
            raise ConfigError(
                f"n_heads must be divisible by n_kv_heads ({self.n_heads} % {self.n_kv_heads})")
        if self.activation not in (ACT_TANH, ACT_ERF):
            raise ConfigError(f"unknown activation {self.activation!r}")
        for f in ("vocab_size", "n_layers", "n_heads", "d_model", "d_mlp", "max_seq_len",
                  "head_dim", "n_kv_heads"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"{f} must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("norm_eps must be positive")

    # ------------------------------------------------------------ derived values
    @property
    def kv_group_size(self) -> int:
        """Query heads per key/value head (src/config.rs:171-173)."""
        return self.n_heads // self.n_kv_heads

    def attn_scale(self, layer_idx: int) -> float:
        """Score scale of one layer: ``head_dim**-0.5`` if enabled (src/config.rs:162-168),
        further divided by ``layer_idx + 1`` under ``scale_attn_by_inverse_layer_idx``."""
        s = float(self.head_dim) ** -0.5 if self.scale_attn_by_head_dim else 1.0
        if self.scale_attn_by_inverse_layer_idx:
            s /= float(layer_idx + 1)
        return s

    def n_params(self, with_linear_biases: bool = True) -> int:
        """Parameter count as the reference counts it (src/model.rs:216-244)."""
        d, m, hq, hk = self.d_model, self.d_mlp, self.n_heads * self.head_dim, \
            self.n_kv_heads * self.head_dim
        per_layer = d * hq + 2 * d * hk + hq * d + 2 * d * m + 4 * d
        if with_linear_biases:
            per_layer += hq + 2 * hk + d + m + d
        total = self.vocab_size * d + self.max_seq_len * d + self.n_layers * per_layer + 2 * d
        if not self.tie_embeddings:
            total += self.vocab_size * d
        return total

    # ------------------------------------------------------------------ writing
    def to_json(self) -> dict[str, Any]:
        """The reference's key names, so that the folder loads there too; the exact
        GELU and the per-layer scale use spellings the reference ignores or rejects."""
        d = asdict(self)
        d["activation"] = "gelu" if self.activation == ACT_TANH else "gelu_erf"
        d["norm"] = "layernorm"
        d["pos_encoding"] = "learned"
        d["model_type"] = "gpt2"
        return d

    def replace(self, **kw) -> "GPT2Config":
        cfg = replace(self, **kw)
        cfg.validate()
        return cfg


def _read_activation(obj: dict) -> str:
    if obj.get("activation_function") is not None:
        raw, table, key = obj["activation_function"], _CHECKPOINT_ACTIVATIONS, "activation_function"
    elif obj.get("activation") is not None:
        nimbus_style = any(k in obj for k in _NIMBUS_KEYS)
        raw, key = obj["activation"], "activation"
        table = _NIMBUS_ACTIVATIONS if nimbus_style else _CHECKPOINT_ACTIVATIONS
    else:
        return ACT_TANH  # src/config.rs:57
    if not isinstance(raw, str):
        raise ConfigError(f"{key}: expected a string, got {raw!r}")
    if raw == "swiglu":
        raise ConfigError("architecture not supported: gpt2 has a GELU feed-forward, got 'swiglu'")
    if raw not in table:
        raise ConfigError(f"{key}: unknown activation {raw!r} (accepted: {sorted(table)})")
    return table[raw]
