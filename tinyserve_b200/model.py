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
    BLOCKS, EMBEDDINGS, HEADS, NORMS, PART_FAMILIES, POSITION_ENCODINGS,
    Block, CacheNeed, PagedNeed, PositionEncoding, ResidualStream, StepContext, TensorSpec,
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
        for n, ls in enumerate(spec.layers):
            block = self._build_block(n, ls)
            pos = None
            if ls.position is not None:
                cand = POSITION_ENCODINGS.build(ls.position.kind, **ls.position.args)
                pos = self._positions.setdefault(cand.key(), cand)
            self.layers.append(Layer(ls, block, pos))
        # One cache user per (call of the order, mixer role of its block), in that order: the
        # cache manager gets their needs as a flat list and hands back one entry for each.
        self.cache_users: list[tuple[int, str]] = []
        self._user_index: dict[tuple[int, str], int] = {}
        for n, call in enumerate(spec.order):
            for role in self.layers[call.layer].block.mixers():
                self._user_index[(n, role)] = len(self.cache_users)
                self.cache_users.append((n, role))
        self._check_order()

    @staticmethod
    def _build_block(n: int, ls: LayerSpec) -> Block:
        """The block class names its roles; every role is built from the registry of its family."""
        block_cls = BLOCKS.get(ls.block)
        roles = getattr(block_cls, "roles", None)
        if not roles:
            raise TypeError(f"block {ls.block!r} names no roles (a Block subclass with a ``roles`` mapping is needed)")
        optional = getattr(block_cls, "optional_roles", frozenset())
        unknown = set(ls.parts) - set(roles)
        missing = set(roles) - set(ls.parts) - set(optional)
        if unknown or missing:
            raise ValueError(f"layer {n} ({ls.block!r}): parts for unknown roles {sorted(unknown)}, "
                             f"no parts for roles {sorted(missing)}; the block's roles are {dict(roles)}")
        parts = {}
        for role, family in roles.items():
            if role not in ls.parts:
                continue
            if family not in PART_FAMILIES:
                raise ValueError(f"block {ls.block!r}: role {role!r} names the unknown family {family!r}")
            parts[role] = PART_FAMILIES[family].build(ls.parts[role].kind, **ls.parts[role].args)
        return block_cls(parts)

    def _check_order(self) -> None:
        for n, call in enumerate(self.spec.order):
            src = call.reads_cache_of
            if src is None:
                continue
            mine = {r: m.cache_need() for r, m in self.layers[call.layer].block.mixers().items()}
            theirs = {r: m.cache_need() for r, m in self.layers[self.spec.order[src].layer].block.mixers().items()}
            for role, need in mine.items():
                other = theirs.get(role)
                same = (isinstance(need, PagedNeed) and type(other) is type(need)
                        and {**vars(need), "window": None} == {**vars(other), "window": None})
                if not same:
                    raise ValueError(
                        f"order[{n}] reads the cache of call {src}, whose layout differs: {need} vs {other}")

    # ---- weights
    def _each_part(self):
        yield "", self.embedding
        for layer in self.layers:
            for part in layer.block.parts.values():
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
    def cache_needs(self) -> list[CacheNeed | None]:
        """One entry per cache user (a call of the order and a mixer role of its block; with one
        mixer per block, one entry per call): what it keeps between steps (``None`` for a
        mixer that keeps nothing or a call that reads another call's cache)."""
        needs: list[CacheNeed | None] = []
        for n, role in self.cache_users:
            call = self.spec.order[n]
            if call.reads_cache_of is not None:
                needs.append(None)
            else:
                needs.append(self.layers[call.layer].block.parts[role].cache_need())
        return needs

    def caches_of_call(self, n: int, entries: list[Any]) -> dict[str, Any]:
        """The cache entries that call ``n`` of the order works on, by mixer role: its own, or
        those of the call whose cache it reads."""
        call = self.spec.order[n]
        src = n if call.reads_cache_of is None else call.reads_cache_of
        out = {}
        for role in self.layers[call.layer].block.mixers():
            entry = entries[self._user_index[(src, role)]]
            if entry is not None:
                out[role] = entry
        return out

    def recordable(self, kind: str) -> bool:
        """Whether steps of this kind ("decode", "prefill") can be recorded: every part allows it."""
        parts = [part for _, part in self._each_part()] + [l.position for l in self.layers if l.position is not None]
        return all(kind in part.recordable for part in parts)


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

    def cache_needs(self) -> list[CacheNeed | None]:
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
            ctx.upcoming_caches = parts.caches_of_call(n + 1, caches) if n + 1 < len(self.spec.order) else {}
            layer.block.forward(stream, ctx, parts.caches_of_call(n, caches), call.reads_cache_of is None, tables)
        ctx.arena.step_region()
        for join in ctx.at_step_end:
            join()
        ctx.at_step_end.clear()
        if num_want == 0:
            return None
        hn = parts.final_norm.forward_rows(stream, want_rows, num_want, ctx)
        logits = ctx.arena.take_step((num_want, self.spec.vocab_size), torch.float32)
        return parts.head.forward(hn, logits)
