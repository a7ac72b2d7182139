"""Interfaces of the parts a model is assembled from, and their registries.

A *part* is built from a :class:`PartSpec` (a kind name plus keyword arguments: all of
its sizes and constants) and knows nothing about the model it sits in.  There are five
families, each with its own registry:

=============  ===========================================================================
family         interface
=============  ===========================================================================
``norm``       ``forward(ctx, x_f32[rows, width], rows=None) -> act[rows', width]``
``position``   ``table`` (rows added to the token embedding, or ``None``) and
               ``rotate(ctx, qkv)`` (applied to queries and keys before they are cached)
``mixer``      ``forward(ctx, h, residual)``: mixes tokens of a sequence; ``residual`` (the
               fp32 stream) receives ``+= mixer(h)``.  Declares what it keeps per sequence
               with ``cache_request()`` (growing keys/values) and ``state_request()``
               (fixed size); the storage of the running schedule entry is on the context
               (``ctx.kv``, ``ctx.state``, ``ctx.writes_cache``).
``ffn``        ``forward(ctx, h, residual)``: per-token feed-forward, ``residual += ffn(h)``
``block``      ``forward(ctx, x, layer)``: the arrangement of norms, mixer and feed-forward
               around the residual stream of one layer
=============  ===========================================================================

Every part lists its parameters with :meth:`Part.param_specs` (shape and role) and gets the
loaded device tensors through :meth:`Part.bind`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

MATRIX = "matrix"   # linear weight held as [out, in]; element type follows the run precision
TABLE = "table"     # rows gathered by index (embeddings); element type as for matrices
VECTOR = "vector"   # biases and norm weights; always held in fp32
INDEX = "index"     # integer tables; held as int32


@dataclass(frozen=True)
class ParamSpec:
    shape: tuple[int, ...]
    role: str = MATRIX
    optional: bool = False


@dataclass(frozen=True)
class PartSpec:
    """Which part, with which sizes and constants."""
    kind: str
    args: dict = field(default_factory=dict)

    def with_args(self, **kw) -> "PartSpec":
        return PartSpec(self.kind, {**self.args, **kw})


@dataclass(frozen=True)
class KVRequest:
    """Growing per-sequence storage a mixer needs: keys and values for every cached token.
    ``window`` > 0 means only the last ``window`` tokens are ever read."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size per-sequence storage: ``n_elements`` fp32 values, zeroed when a slot is
    handed out."""
    n_elements: int


class Part:
    """Base of all parts."""
    family: str = ""
    kind: str = ""
    #: True if ``forward`` only launches work on the current CUDA stream from device-resident
    #: data (no host reads of the batch, no synchronisation), so that a step can be captured
    #: in a CUDA graph.  A part that does not say so keeps the engine on plain launches.
    graph_safe: bool = False

    def param_specs(self) -> dict[str, ParamSpec]:
        return {}

    def bind(self, params: dict[str, torch.Tensor | None], runtime) -> None:
        """Receive the loaded tensors (``None`` for absent optional ones)."""
        for name, t in params.items():
            setattr(self, name.replace(".", "_"), t)

    def children(self) -> dict[str, "Part"]:
        """Sub-parts whose parameters are listed under ``<name>.``."""
        return {}


class Norm(Part):
    family = "norm"

    def forward(self, ctx, x: torch.Tensor, rows: torch.Tensor | None = None,
                n_rows: int | None = None) -> torch.Tensor:
        raise NotImplementedError

    def defer(self, ctx, x: torch.Tensor):
        """The normalised rows, possibly not computed yet: a consumer that can fuse the norm
        into its first kernel takes a :class:`DeferredNorm` apart, any other calls
        ``.tensor()``.  The default computes right away."""
        return self.forward(ctx, x)


class DeferredNorm:
    """``norm(x)`` that has not been computed: ``x`` fp32 rows, ``args`` what the fused kernel
    needs.  ``tensor()`` computes it the plain way."""

    def __init__(self, ctx, norm: Norm, x: torch.Tensor, args: tuple):
        self.ctx, self.norm, self.x, self.args = ctx, norm, x, args
        self.shape = x.shape
        self.device = x.device

    def tensor(self) -> torch.Tensor:
        return self.norm.forward(self.ctx, self.x)


class Position(Part):
    family = "position"
    #: rows added to the token embedding at a token's position, or None
    table: torch.Tensor | None = None
    #: the longest sequence this encoding can address, or None if unbounded
    max_positions: int | None = None

    def rotate(self, ctx, qkv: torch.Tensor, mixer) -> None:
        """Hook for encodings that act on queries and keys, in place, before keys are written
        to the cache.  ``qkv``: the step's rows [n_rows, q_width + 2 * kv_width] (queries, keys,
        values side by side); ``mixer`` gives ``n_heads``, ``n_kv_heads``, ``head_dim``,
        ``q_width`` and ``kv_width``; a row's position is ``ctx.layout.row_pos``."""
        return None


class Mixer(Part):
    family = "mixer"
    #: True if ``forward`` takes ``h`` as a :class:`DeferredNorm` (its first linear map fuses
    #: the norm); otherwise it always gets a tensor
    accepts_deferred_norm: bool = False

    def cache_request(self) -> KVRequest | None:
        return None

    def state_request(self) -> StateRequest | None:
        return None

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        """``ctx.kv``: the paged key/value store of this schedule entry (or of the entry it
        reads from, then ``ctx.writes_cache`` is False); ``ctx.state``: fp32 tensor
        [n_slots, n_elements] or None.  Storage belongs to the schedule entry, not to the
        layer: a layer that runs twice keeps two caches."""
        raise NotImplementedError


class FeedForward(Part):
    family = "ffn"
    accepts_deferred_norm: bool = False

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    family = "block"

    def forward(self, ctx, x: torch.Tensor, layer) -> None:
        raise NotImplementedError


_REGISTRIES: dict[str, dict[str, Callable[..., Part]]] = {
    "norm": {}, "position": {}, "mixer": {}, "ffn": {}, "block": {},
}


def register_part(family: str, kind: str, factory: Callable[..., Part] | None = None, *,
                  replace: bool = False):
    """Register ``factory(**args) -> Part`` under ``family``/``kind``.  Usable as a decorator
    on a class: ``@register_part("mixer", "my_mixer")``."""
    if family not in _REGISTRIES:
        raise ValueError(f"unknown part family {family!r} (have {sorted(_REGISTRIES)})")

    def _do(f):
        if kind in _REGISTRIES[family] and not replace:
            raise ValueError(f"{family} part {kind!r} is already registered")
        _REGISTRIES[family][kind] = f
        if isinstance(f, type):
            f.kind = kind
        return f

    return _do(factory) if factory is not None else _do


def build_part(family: str, spec: PartSpec) -> Part:
    try:
        factory = _REGISTRIES[family][spec.kind]
    except KeyError:
        raise ValueError(
            f"no {family} part named {spec.kind!r} (registered: {sorted(_REGISTRIES[family])})"
        ) from None
    part = factory(**spec.args)
    if not part.kind:
        part.kind = spec.kind
    return part


def registered_parts(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])


def collect_param_specs(part: Part, prefix: str = "") -> dict[str, ParamSpec]:
    """All parameters of a part and its children, keyed by dotted path."""
    out = {prefix + n: s for n, s in part.param_specs().items()}
    for cname, child in part.children().items():
        out.update(collect_param_specs(child, f"{prefix}{cname}."))
    return out


def bind_params(part: Part, params: dict[str, Any], runtime, prefix: str = "") -> None:
    own = {n: params.get(prefix + n) for n in part.param_specs()}
    part.bind(own, runtime)
    for cname, child in part.children().items():
        bind_params(child, params, runtime, f"{prefix}{cname}.")
