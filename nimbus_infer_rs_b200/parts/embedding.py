"""Token embedding and output head."""
from __future__ import annotations

import torch

from .base import MATRIX, TABLE, DeferredNorm, ParamSpec, Part


class TokenEmbedding(Part):
    """``x[i] = table[token_i] (+ position_table[pos_i])`` into the fp32 residual stream
    (src/model.rs:285-295)."""
    graph_safe = True
    family = "embedding"
    kind = "token_embedding"

    def __init__(self, vocab_size: int, width: int):
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.table = None

    def param_specs(self):
        return {"table": ParamSpec((self.vocab_size, self.width), TABLE)}

    def forward(self, ctx, position) -> torch.Tensor:
        lay = ctx.layout
        x = torch.empty((lay.n_rows, self.width), device=self.table.device, dtype=torch.float32)
        ctx.ops.embed_pos(lay.tokens, lay.row_pos, self.table, position.table, x)
        return x


class LMHead(Part):
    """``logits = h @ W.T`` without bias, fp32 result; ``W`` is the token embedding table when
    tied (src/model.rs:317-325)."""
    graph_safe = True
    family = "head"
    kind = "lm_head"

    def __init__(self, vocab_size: int, width: int, tied: bool):
        self.vocab_size = int(vocab_size)
        self.width = int(width)
        self.tied = bool(tied)
        self.weight = None

    def param_specs(self):
        if self.tied:
            return {}
        return {"weight": ParamSpec((self.vocab_size, self.width), MATRIX)}

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, ctx, h) -> torch.Tensor:
        """``h``: activation rows, or a :class:`DeferredNorm` of fp32 rows."""
        norm = None
        if isinstance(h, DeferredNorm):
            h, norm = h.x, h.args
        logits = torch.empty((h.shape[0], self.vocab_size), device=h.device, dtype=torch.float32)
        ctx.ops.linear(h, self.weight, None, logits, 0, None, norm)
        return logits
