"""Normalisation parts."""
from __future__ import annotations

import torch

from .base import VECTOR, DeferredNorm, Norm, ParamSpec, register_part


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * weight + bias`` per row with biased variance, statistics
    in fp32 (src/ops.rs:32-40).  Weight and bias are both required (src/engine.rs:141-152)."""
    graph_safe = True

    def __init__(self, width: int, eps: float):
        self.width = int(width)
        self.eps = float(eps)
        self.weight = None
        self.bias = None

    def param_specs(self):
        return {"weight": ParamSpec((self.width,), VECTOR),
                "bias": ParamSpec((self.width,), VECTOR)}

    def defer(self, ctx, x):
        return DeferredNorm(ctx, self, x, (self.weight, self.bias, self.eps, ctx.rt.act_dtype))

    def forward(self, ctx, x, rows=None, n_rows=None):
        n = x.shape[0] if rows is None else (rows.numel() if n_rows is None else n_rows)
        out = torch.empty((n, self.width), device=x.device, dtype=ctx.rt.act_dtype)
        ctx.ops.layernorm(x, self.weight, self.bias, self.eps, out, rows)
        return out
