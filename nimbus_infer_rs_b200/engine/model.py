"""A model assembled from a :class:`ModelSpec`: embedding, position encoding, layers in
schedule order, final norm, output head.  It owns no architecture knowledge.

The forward pass follows src/model.rs:271-325: embed (+ position), every scheduled layer on
the fp32 residual stream, then the final norm and the head -- here only on the rows whose
logits were asked for (the reference norms every row and takes logits of the last one).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import ParamSpec, bind_params, build_part, collect_param_specs
from ..parts.embedding import LMHead, TokenEmbedding
from .spec import ModelSpec

PRECISIONS = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
              "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


@dataclass
class Runtime:
    """What every part may ask about the run: device and element type of activations and
    caches (``bfloat16``: the serving precision; ``float32``: everything in true 32-bit)."""
    device: torch.device
    act_dtype: torch.dtype

    @property
    def precision(self) -> str:
        return "float32" if self.act_dtype == torch.float32 else "bfloat16"


class Layer:
    def __init__(self, index: int, spec):
        self.index = index
        self.spec = spec
        self.block = build_part("block", spec.block)
        self.norm_mixer = build_part("norm", spec.norm_mixer)
        self.mixer = build_part("mixer", spec.mixer)
        self.norm_ffn = build_part("norm", spec.norm_ffn)
        self.ffn = build_part("ffn", spec.ffn)

    def parts(self):
        return {"norm_mixer": self.norm_mixer, "mixer": self.mixer,
                "norm_ffn": self.norm_ffn, "ffn": self.ffn}


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = runtime
        self.embedding = TokenEmbedding(spec.vocab_size, spec.width)
        self.position = build_part("position", spec.position)
        self.layers = [Layer(i, ls) for i, ls in enumerate(spec.layers)]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = LMHead(spec.vocab_size, spec.width, spec.tie_head)
        self.run_order = spec.run_order()
        self.params: dict[str, torch.Tensor | None] = {}

    # ------------------------------------------------------------------ parameters
    def _named_parts(self):
        yield "embedding.", self.embedding
        yield "position.", self.position
        for l in self.layers:
            for name, part in l.parts().items():
                yield f"layers.{l.index}.{name}.", part
        yield "final_norm.", self.final_norm
        yield "head.", self.head

    def param_specs(self) -> dict[str, ParamSpec]:
        out: dict[str, ParamSpec] = {}
        for prefix, part in self._named_parts():
            out.update(collect_param_specs(part, prefix))
        return out

    def bind(self, params: dict[str, torch.Tensor | None]) -> None:
        self.params = params
        for prefix, part in self._named_parts():
            bind_params(part, params, self.rt, prefix)
        if self.spec.tie_head:
            self.head.tie(self.embedding.table)

    def graph_safe(self) -> bool:
        """True if every part of the model may run under CUDA-graph capture."""
        parts = [self.embedding, self.position, self.final_norm, self.head]
        for l in self.layers:
            parts += [l.block, l.norm_mixer, l.mixer, l.norm_ffn, l.ffn]
        return all(getattr(p, "graph_safe", False) for p in parts)

    def n_params(self) -> int:
        return sum(t.numel() for t in self.params.values() if t is not None)

    def weight_bytes(self) -> int:
        """Bytes of the tensors a decode step reads: every parameter once, except that of the
        embedding tables only the rows of the step's tokens are read (the tied table is
        counted because the head reads all of it)."""
        total = 0
        for name, t in self.params.items():
            if t is None:
                continue
            if name == "position.table" or (name == "embedding.table" and not self.spec.tie_head):
                continue
            total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, ctx) -> torch.Tensor:
        """The fp32 residual stream after the last scheduled layer, [rows, width]."""
        x = self.embedding.forward(ctx, self.position)
        for entry, li in enumerate(self.run_order):
            layer = self.layers[li]
            ctx.kv, ctx.state, ctx.writes_cache = self.storage_of(ctx.cache, entry)
            layer.block.forward(ctx, x, layer)
        return x

    def storage_requests(self):
        """What each schedule entry keeps per sequence: ``({entry: KVRequest}, {entry:
        StateRequest})``.  An entry of a layer with ``cache_from`` keeps no keys/values."""
        kv, st = {}, {}
        for entry, li in enumerate(self.run_order):
            layer = self.layers[li]
            r = layer.mixer.cache_request()
            if layer.spec.cache_from is None:
                if r is not None:
                    kv[entry] = r
            else:
                # the reader must want what the owner keeps: same heads and head size, and no
                # keys from before the owner's window
                own = self.layers[layer.spec.cache_from].mixer.cache_request()
                ok = (r is not None and own is not None and r.n_kv_heads == own.n_kv_heads
                      and r.head_dim == own.head_dim
                      and (own.window == 0 or 0 < r.window <= own.window))
                if not ok:
                    raise ValueError(
                        f"layer {li} reads the cache of layer {layer.spec.cache_from}, which "
                        f"keeps {own}, but asks for {r}")
            s = layer.mixer.state_request()
            if s is not None:
                st[entry] = s
        return kv, st

    def kv_source(self, entry: int) -> int:
        """The schedule entry whose key/value store ``entry`` uses: itself, or the latest
        earlier run of the layer named by ``cache_from``."""
        src = self.layers[self.run_order[entry]].spec.cache_from
        if src is None:
            return entry
        for e in range(entry - 1, -1, -1):
            if self.run_order[e] == src:
                return e
        raise ValueError(f"schedule entry {entry}: layer {src}, whose cache it reads, has not "
                         "run before it")

    def storage_of(self, cache, entry: int):
        src = self.kv_source(entry)
        return cache.layer_kv(src), cache.layer_state(entry), src == entry

    def logits(self, ctx, x: torch.Tensor, rows: torch.Tensor, n_rows: int) -> torch.Tensor:
        """Final norm and head on the selected rows → fp32 [n_rows, vocab]."""
        if ctx.layout.want_all_rows and n_rows == x.shape[0]:
            # every row is wanted, in order (a decode step): no gather, and the norm may be
            # folded into the head's product
            return self.head.forward(ctx, self.final_norm.defer(ctx, x))
        h = self.final_norm.forward(ctx, x, rows, n_rows)
        return self.head.forward(ctx, h)

    def forward(self, ctx) -> torch.Tensor | None:
        x = self.forward_hidden(ctx)
        lay = ctx.layout
        if lay.n_want == 0:
            return None
        return self.logits(ctx, x, lay.want_rows, lay.n_want)
