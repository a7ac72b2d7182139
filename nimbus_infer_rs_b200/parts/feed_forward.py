"""Per-token feed-forward parts."""
from __future__ import annotations

import torch

from ..csrc.ops import ACTIVATIONS
from .base import FeedForward, register_part
from .linear import Linear


@register_part("ffn", "dense_mlp")
class DenseMLP(FeedForward):
    """``residual += act(h @ Wfc + bfc) @ Wproj + bproj`` (src/model.rs:462-473,485-487).
    ``activation`` is ``gelu_tanh`` (src/ops.rs:21-24), ``gelu_erf`` or ``none``; ``hidden`` is
    a plain number, not derived from the width (src/config.rs:13)."""
    graph_safe = True
    accepts_deferred_norm = True

    def __init__(self, width: int, hidden: int, activation: str, bias: bool = True):
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} (have {sorted(ACTIVATIONS)})")
        self.width, self.hidden = int(width), int(hidden)
        self.activation = activation
        self.act_code = ACTIVATIONS[activation]
        self.fc = Linear(self.width, self.hidden, bias)
        self.proj = Linear(self.hidden, self.width, bias)

    def children(self):
        return {"fc": self.fc, "proj": self.proj}

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        mid = self.fc(ctx, h, act=self.act_code)
        self.proj(ctx, mid, residual=residual)
