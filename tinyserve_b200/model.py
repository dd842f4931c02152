"""The generic decoder: a model is the parts its ``ModelSpec`` names, run in the order the
spec lists. There is no per-architecture model class; an architecture is a typed
configuration that produces a spec (``tinyserve_b200.architectures``).

One forward pass (after upstream src/tinyserve/model.py:181-200): embed the step's tokens
into the 32-bit residual stream, run every call of the order through its block, select the
wanted rows, apply the final norm to those rows only and multiply by the output head into
32-bit logits.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

import torch

from . import parts as _parts  # noqa: F401  (registers the built-in parts)
from .config.base import LayerSpec, ModelConfig, ModelSpec
from .parts.base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
    Block, KVNeed, PositionEncoding, ResidualStream, StateNeed, StepContext, TensorSpec,
)
from .weights.loader import load_tensors, merge_specs
from .weights.random_init import random_bound_tensors


@dataclass
class Layer:
    spec: LayerSpec
    block: Block
    position: PositionEncoding | None


class ModelParts:
    """The parts of a model, built from a spec but not yet holding weights."""

    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.embedding = EMBEDDINGS.build(spec.embedding.kind, **spec.embedding.args)
        self.final_norm = NORMS.build(spec.final_norm.kind, **spec.final_norm.args)
        self.head = HEADS.build(spec.head.kind, **spec.head.args)
        self._positions: dict[Any, PositionEncoding] = {}
        self.layers: list[Layer] = []
        for ls in spec.layers:
            mixer = MIXERS.build(ls.mixer.kind, **ls.mixer.args)
            ffn = FEED_FORWARDS.build(ls.feed_forward.kind, **ls.feed_forward.args)
            n1 = NORMS.build(ls.mixer_norm.kind, **ls.mixer_norm.args)
            n2 = NORMS.build(ls.feed_forward_norm.kind, **ls.feed_forward_norm.args)
            block = BLOCKS.build(ls.block, mixer, ffn, n1, n2)
            pos = None
            if ls.position is not None:
                cand = POSITION_ENCODINGS.build(ls.position.kind, **ls.position.args)
                pos = self._positions.setdefault(cand.key(), cand)
            self.layers.append(Layer(ls, block, pos))
        self._check_order()

    def _check_order(self) -> None:
        for n, call in enumerate(self.spec.order):
            src = call.reads_cache_of
            if src is None:
                continue
            mine = self.layers[call.layer].block.mixer.cache_need()
            theirs = self.layers[self.spec.order[src].layer].block.mixer.cache_need()
            same = (isinstance(mine, KVNeed) and isinstance(theirs, KVNeed)
                    and (mine.num_kv_heads, mine.head_dim) == (theirs.num_kv_heads, theirs.head_dim))
            if not same:
                raise ValueError(
                    f"order[{n}] reads the cache of call {src}, whose layout differs: {mine} vs {theirs}")

    # ---- weights
    def _each_part(self):
        yield "", self.embedding
        for layer in self.layers:
            b = layer.block
            for part in (b.mixer_norm, b.mixer, b.feed_forward_norm, b.feed_forward):
                yield layer.spec.prefix, part
        yield "", self.final_norm
        yield "", self.head

    def tensor_specs(self) -> list[TensorSpec]:
        specs: list[TensorSpec] = []
        for prefix, part in self._each_part():
            specs.extend(part.tensor_specs(prefix))
        return list(merge_specs(specs).values())

    def ignorable_tensors(self) -> set[str]:
        out: set[str] = set()
        for prefix, part in self._each_part():
            out |= part.ignorable_tensors(prefix)
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for prefix, part in self._each_part():
            part.bind(prefix, tensors)

    # ---- cache
    def cache_needs(self) -> list[KVNeed | StateNeed | None]:
        """One entry per call of the order: what that call keeps between steps (``None``
        for a call that keeps nothing or that reads another call's cache)."""
        needs: list[KVNeed | StateNeed | None] = []
        for call in self.spec.order:
            if call.reads_cache_of is not None:
                needs.append(None)
            else:
                needs.append(self.layers[call.layer].block.mixer.cache_need())
        return needs


def build_parts(spec: ModelSpec) -> ModelParts:
    return ModelParts(spec)


class DecoderModel:
    """Parts with weights on a device, in one dtype, ready to run steps."""

    def __init__(self, config: ModelConfig, tensors: Mapping[str, torch.Tensor],
                 dtype: torch.dtype, device: torch.device | str) -> None:
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        self.config = config
        self.spec = config.to_spec()
        self.parts = build_parts(self.spec)
        self.dtype = dtype
        self.device = torch.device(device)
        self.tensors = dict(tensors)
        self.parts.bind(self.tensors)

    @classmethod
    def from_folder(cls, model_dir: str | Path, dtype: torch.dtype,
                    device: torch.device | str = "cuda") -> "DecoderModel":
        from .config.registry import load_config

        config = load_config(model_dir)
        parts = build_parts(config.to_spec())
        tensors = load_tensors(model_dir, parts.tensor_specs(), dtype, device,
                               ignorable=parts.ignorable_tensors())
        return cls(config, tensors, dtype, device)

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int, dtype: torch.dtype,
                    device: torch.device | str = "cuda") -> "DecoderModel":
        """Random weights made on the device (no folder); see ``weights.random_init``."""
        parts = build_parts(config.to_spec())
        tensors = random_bound_tensors(parts.tensor_specs(), seed, dtype, device)
        return cls(config, tensors, dtype, device)

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def cache_needs(self) -> list[KVNeed | StateNeed | None]:
        return self.parts.cache_needs()

    def weight_bytes(self) -> int:
        seen: set[int] = set()
        total = 0
        for t in self.tensors.values():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def forward(self, ctx: StepContext, caches: list[Any], want_rows: torch.Tensor | None,
                num_want: int) -> torch.Tensor | None:
        """Run this step's tokens; return float32 logits ``[num_want, vocab]`` at ``want_rows``
        (flat row indices into the step's tokens), or ``None`` if nothing is wanted."""
        parts = self.parts
        stream = ResidualStream(parts.embedding.forward(ctx))
        for n, call in enumerate(self.spec.order):
            layer = parts.layers[call.layer]
            tables = None
            if layer.position is not None:
                key = layer.position.key()
                if key not in ctx.position_tables:
                    ctx.position_tables[key] = layer.position.prepare(ctx)
                tables = ctx.position_tables[key]
            src = call.reads_cache_of
            entry = caches[n if src is None else src]
            layer.block.forward(stream, ctx, entry, src is None, tables)
        ctx.arena.step_region()
        if num_want == 0:
            return None
        hn = parts.final_norm.forward_rows(stream, want_rows, num_want, ctx)
        logits = ctx.arena.take_step((num_want, self.spec.vocab_size), torch.float32)
        return parts.head.forward(hn, logits)
