"""Dense gated feed-forward (SwiGLU).

``y = (silu(x Wgate^T) * (x Wup^T)) Wdown^T`` with ``silu(z) = z * sigmoid(z)`` and no
biases (upstream src/tinyserve/layers.py:94-115); gate and up come from one product with
the merged ``[2 * intermediate, hidden]`` matrix, gate rows first
(src/tinyserve/model.py:178-179, src/tinyserve/weights.py:104-129).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from .base import (EVERY_STEP, FeedForward, LazyNormed, ResidualStream, StepContext, TensorSpec, project, project_to_stream,
                   register_feed_forward)


class SwiGLU(FeedForward):
    recordable = EVERY_STEP

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int) -> None:
        self.prefix = prefix
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, h, i = prefix + self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(p + "gate_up_proj.weight", (2 * i, h),
                       merged_from=(p + "gate_proj.weight", p + "up_proj.weight"),
                       merged_rows=(i, i)),
            TensorSpec(p + "down_proj.weight", (h, i)),
        ]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p = prefix + self.prefix
        self.w_gate_up = tensors[p + "gate_up_proj.weight"]
        self.w_down = tensors[p + "down_proj.weight"]

    takes_lazy_input = True
    adds_to_stream = True

    def streamed_weights(self) -> list[torch.Tensor]:
        return [self.w_gate_up, self.w_down]

    def forward(self, x: "torch.Tensor | LazyNormed", ctx: StepContext,
                stream: ResidualStream | None = None) -> torch.Tensor | None:
        t = x.shape[0]
        act = ctx.arena.take((t, self.intermediate_size), ctx.dtype)
        project(x, self.w_gate_up, act, ctx, swiglu=True)
        return project_to_stream(act, self.w_down, stream, ctx)


register_feed_forward("swiglu", SwiGLU)
