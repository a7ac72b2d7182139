"""Causal self-attention over the paged key/value cache."""
from __future__ import annotations

import torch

from .base import KVRequest, Mixer, register_part
from .linear import Linear


@register_part("mixer", "causal_attention")
class CausalSelfAttention(Mixer):
    """Multi-head attention with ``n_kv_heads`` shared key/value heads (query head ``h`` reads
    key/value head ``h // (n_heads // n_kv_heads)``, src/model.rs:342,390).

    One fused projection gives queries, keys and values (the reference runs three products,
    src/model.rs:360-365; the weights are concatenated at load).  Keys and values of this
    step's tokens are appended to the cache first; every query row then attends to keys
    ``0..p`` of its own sequence, ``p`` being its absolute position (src/model.rs:401-419), or
    to the last ``window`` of them.  Scores are ``dot(q, k) * scale``; softmax in fp32.
    The output projection adds its result into the residual stream (src/model.rs:434-439).
    """
    graph_safe = True
    accepts_deferred_norm = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 window: int = 0, bias: bool = True):
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.head_dim, self.scale, self.window = int(head_dim), float(scale), int(window)
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be divisible by n_kv_heads")
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.qkv = Linear(self.width, self.q_width + 2 * self.kv_width, bias)
        self.out = Linear(self.q_width, self.width, bias)

    def children(self):
        return {"qkv": self.qkv, "out": self.out}

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        lay, kv = ctx.layout, ctx.kv
        qkv = self.qkv(ctx, h, out_dtype=kv.k.dtype)
        ctx.position.rotate(ctx, qkv, self)
        append = (self.q_width, self.q_width + self.kv_width) if ctx.writes_cache else None
        attn = torch.empty((lay.n_rows, self.q_width), device=h.device, dtype=ctx.rt.act_dtype)
        ctx.ops.attention(qkv, 0, lay, kv, self.n_heads, attn, self.scale, self.window, append)
        self.out(ctx, attn, residual=residual)
