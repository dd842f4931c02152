"""RMSNorm over the last dimension, fused with the residual sum that precedes it.

Formula (upstream src/tinyserve/layers.py:35-38): in 32-bit ``y = x * rsqrt(mean(x^2) +
eps)``; ``y`` is cast to the model dtype and THEN multiplied by the weight (a plain weight,
not ``1 + w``). Here ``x`` is the 32-bit residual stream plus the pending sub-layer output,
which the same kernel adds and writes back.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from .base import EVERY_STEP, LazyNormed, Norm, ResidualStream, StepContext, TensorSpec, register_norm


class RMSNorm(Norm):
    recordable = EVERY_STEP

    def __init__(self, name: str, size: int, eps: float) -> None:
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + self.name, (self.size,), init="one_plus_normal")]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[prefix + self.name]

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        out = ctx.arena.take((stream.resid.shape[0], self.size), ctx.dtype)
        ops.add_rms_norm(stream.resid, stream.delta, self.weight, self.eps, out)
        if stream.delta is not None:
            stream.delta = None
            stream.sumsq = None          # the stream has changed
        return out

    def lazy(self, stream: ResidualStream, ctx: StepContext) -> "torch.Tensor | LazyNormed":
        if stream.delta is None and stream.sumsq is not None:
            return LazyNormed(stream, self.weight, self.eps, lambda: self.forward(stream, ctx))
        return self.forward(stream, ctx)

    def forward_rows(self, stream: ResidualStream, rows: torch.Tensor, num_rows: int,
                     ctx: StepContext) -> torch.Tensor:
        out = ctx.arena.take((num_rows, self.size), ctx.dtype)
        ops.add_rms_norm(stream.resid, stream.delta, self.weight, self.eps, out, rows=rows)
        return out


register_norm("rms_norm", RMSNorm)
