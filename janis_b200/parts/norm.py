"""RMS norm with a weight offset.

y = x / sqrt(mean(x^2) + eps) * (offset + w).  Gemma2 stores w and uses 1 + w
(`gemma/gemma.go:22-28`); offset 0 is the usual RMS norm (`qwen/norm.go:10-27`).
eps lies inside the root, added to the mean (`cpu/cpu_ops.go:145-162`).  The
sum of squares, the root and offset + w are float32 whatever the model's dtype.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Norm, Runtime, StepContext


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, weight_name: str, offset: float = 0.0, init_std: float = 0.1):
        self.width = width
        self.eps = float(eps)
        self.offset = float(offset)
        self.weight_name = weight_name
        self.init_std = init_std
        self.weight = None          # float32: offset + w

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.width,), init_std=self.init_std)}

    def load(self, store, rt: Runtime):
        self.weight = (store.get(self.weight_name).to(torch.float32) + self.offset).contiguous()

    def forward(self, x, ctx: StepContext, out, rows=None):
        return ctx.rt.ops.rmsnorm(x, self.weight, self.eps, out, rows)

    def residual_add(self, h, r, ctx: StepContext, next_norm: Norm | None = None, out=None):
        """h += self(r); out = next_norm(h) when a next norm is given."""
        if next_norm is None:
            ctx.rt.ops.add_rmsnorm(h, r, self.weight, self.eps)
            return None
        if isinstance(next_norm, RMSNorm):
            return ctx.rt.ops.add_rmsnorm(h, r, self.weight, self.eps, next_norm.weight, next_norm.eps, out)
        ctx.rt.ops.add_rmsnorm(h, r, self.weight, self.eps)
        return next_norm.forward(h, ctx, out)


def plain_residual_add(h, r, ctx: StepContext, next_norm: Norm | None = None, out=None):
    """h += r for blocks without a norm after the sublayer; out = next_norm(h) when given."""
    if isinstance(next_norm, RMSNorm):
        return ctx.rt.ops.add_rmsnorm(h, r, None, 0.0, next_norm.weight, next_norm.eps, out)
    ctx.rt.ops.add_rmsnorm(h, r, None, 0.0)
    return next_norm.forward(h, ctx, out) if next_norm is not None else None
