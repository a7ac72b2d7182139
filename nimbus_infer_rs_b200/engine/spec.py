"""The description of a model as data: which parts, layer by layer, and in which order.

An architecture's ``build_spec(config)`` returns a :class:`ModelSpec`; the engine builds the
model from it without knowing the architecture.  Layers may differ from one another
(another mixer, another feed-forward), ``schedule`` lists the layers in the order they run
(a layer may be named twice), and a layer with ``cache_from`` set reads the key/value cache
of that other layer instead of keeping its own.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerSpec:
    mixer: PartSpec
    ffn: PartSpec
    norm_mixer: PartSpec
    norm_ffn: PartSpec
    block: PartSpec = PartSpec("pre_norm")
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_seq_len: int
    position: PartSpec
    layers: tuple[LayerSpec, ...]
    final_norm: PartSpec
    tie_head: bool = True
    schedule: tuple[int, ...] | None = None

    def run_order(self) -> tuple[int, ...]:
        order = self.schedule if self.schedule is not None else tuple(range(len(self.layers)))
        for i in order:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"schedule names layer {i}, but there are {len(self.layers)}")
        return tuple(order)

    def validate(self) -> None:
        self.run_order()
        for i, l in enumerate(self.layers):
            if l.cache_from is not None:
                if not 0 <= l.cache_from < len(self.layers) or l.cache_from == i:
                    raise ValueError(f"layer {i}: cache_from={l.cache_from} is not another layer")
                if self.layers[l.cache_from].cache_from is not None:
                    raise ValueError(f"layer {i}: cache_from must name a layer with its own cache")
