"""Arrangements of norms, mixer and feed-forward around the residual stream."""
from __future__ import annotations

from .base import Block, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """``x += mixer(norm_mixer(x)); x += ffn(norm_ffn(x))`` (src/model.rs:297-300 with
    :345-357, :437-439, :448-460, :485-487).  ``x`` is the fp32 residual stream."""
    graph_safe = True

    def __init__(self):
        pass

    def forward(self, ctx, x, layer) -> None:
        mixer, ffn = layer.mixer, layer.ffn
        h = layer.norm_mixer.defer(ctx, x) if mixer.accepts_deferred_norm \
            else layer.norm_mixer.forward(ctx, x)
        mixer.forward(ctx, h, x)
        h = layer.norm_ffn.defer(ctx, x) if ffn.accepts_deferred_norm \
            else layer.norm_ffn.forward(ctx, x)
        ffn.forward(ctx, h, x)
