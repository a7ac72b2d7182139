"""A linear map with optional bias: the building block of mixers, feed-forwards and heads.

The weight is held as ``[out_features, in_features]`` (each output is one contiguous row,
as the reference keeps it after its load-time transpose, src/engine.rs:93-101), which is
the K-major operand layout of the tensor-core kernels.  The epilogue (bias, activation,
residual add) runs inside the matrix-product kernel.
"""
from __future__ import annotations

import torch

from .base import MATRIX, VECTOR, DeferredNorm, ParamSpec, Part


class Linear(Part):
    graph_safe = True
    family = "linear"
    kind = "linear"

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.has_bias = bool(bias)
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def param_specs(self):
        specs = {"weight": ParamSpec((self.out_features, self.in_features), MATRIX)}
        if self.has_bias:
            # a bias is optional per tensor (src/engine.rs:153-161)
            specs["bias"] = ParamSpec((self.out_features,), VECTOR, optional=True)
        return specs

    def __call__(self, ctx, x: torch.Tensor, *, out: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None, act: int = 0,
                 residual: torch.Tensor | None = None) -> torch.Tensor:
        """``act(x @ W.T + b)``; with ``residual`` (fp32) the result is added into it in place."""
        norm = None
        if isinstance(x, DeferredNorm):       # the kernel applies the norm to the rows it loads
            x, norm = x.x, x.args
        if residual is not None:
            out = residual
        elif out is None:
            out = torch.empty((x.shape[0], self.out_features), device=x.device,
                              dtype=out_dtype or ctx.rt.act_dtype)
        ctx.ops.linear(x, self.weight, self.bias, out, act, residual, norm)
        return out
