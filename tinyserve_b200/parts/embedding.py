"""Token embedding (a row gather with no scaling, upstream src/tinyserve/model.py:192) and
the output head (``logits = float32(x W^T)`` with ``W`` the embedding table when tied,
src/tinyserve/model.py:129-130,208).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from .base import EMBEDDINGS, EVERY_STEP, HEADS, Part, StepContext, TensorSpec


class TokenEmbedding(Part):
    recordable = EVERY_STEP

    def __init__(self, name: str, vocab_size: int, hidden_size: int) -> None:
        self.name, self.vocab_size, self.hidden_size = name, int(vocab_size), int(hidden_size)
        self.table: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(prefix + self.name, (self.vocab_size, self.hidden_size))]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[prefix + self.name]

    def forward(self, ctx: StepContext) -> torch.Tensor:
        """The 32-bit residual stream ``[T, hidden]`` of this step's tokens."""
        out = ctx.arena.take((ctx.num_tokens, self.hidden_size), torch.float32)
        ops.embed(ctx.tokens, self.table, out)
        return out


class LMHead(Part):
    recordable = EVERY_STEP

    def __init__(self, name: str, tied: bool, vocab_size: int, hidden_size: int,
                 ignored_when_tied: str | None = None) -> None:
        self.name, self.tied = name, bool(tied)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.ignored_when_tied = ignored_when_tied
        self.weight: torch.Tensor | None = None

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        # When tied this names the embedding table, which the embedding declares as well;
        # equal declarations are one tensor.
        return [TensorSpec(prefix + self.name, (self.vocab_size, self.hidden_size))]

    def ignorable_tensors(self, prefix: str) -> set[str]:
        # A tied checkpoint may still ship a copy of the table under the head's name.
        return {prefix + self.ignored_when_tied} if self.tied and self.ignored_when_tied else set()

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[prefix + self.name]

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """``x [R, hidden]`` in the model dtype -> ``out [R, vocab]`` float32."""
        ops.gemm(x, self.weight, out)
        return out


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("lm_head", LMHead)
