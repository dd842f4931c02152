"""Interfaces of the parts a layer is assembled from, and the registries that name them.

A part knows its own sizes and constants (constructor arguments) and nothing about the
model it sits in. Parts declare the checkpoint tensors they need (``tensor_specs``), receive
them (``bind``) and run on the tokens of one step (``forward``) given a ``StepContext``.

Kinds of part and what each must provide:

* ``Norm``: ``forward(stream, ctx) -> normalised [T, size]`` in the model dtype. ``stream``
  is the residual stream (32-bit) with the previous sub-layer's output still pending; the
  norm folds that output into the stream before normalising, so the residual sum is made
  in 32-bit and costs no extra pass. ``forward_rows`` does the same for selected rows only
  without changing the stream (used before the output head).
* ``PositionEncoding``: ``prepare(ctx)`` once per step returns whatever tables the mixers
  of this step need (for rotary encodings: cos/sin per token). The mixer applies them.
* ``Mixer``: ``cache_need()`` says what it keeps between steps (pages of keys/values for
  all or a window of the positions, a fixed-size state slot, or nothing);
  ``forward(x, ctx, cache, writes_cache) -> [T, hidden]``.
* ``FeedForward``: ``forward(x, ctx) -> [T, hidden]``.
* ``Block``: arranges one mixer, one feed-forward and their norms around the stream.

Registering a class under a name (``register_mixer("my_mixer", MyMixer)`` and so on) is all
it takes to make it available to a ``LayerSpec``; nothing else in the framework changes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch


# --------------------------------------------------------------------------- tensors
@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs, by its full checkpoint name.

    ``merged_from`` lists checkpoint tensors whose rows, stacked in that order, make this
    tensor; a checkpoint may store either the merged tensor or all of its sources.
    ``init`` names the law of the random-weights mode: ``"normal"`` is N(0, std),
    ``"one_plus_normal"`` is 1 + N(0, std). ``keep_32bit`` marks tensors that stay 32-bit
    when the checkpoint stores them so, whatever the run's dtype; integer tables are always
    kept as int32.
    """

    name: str
    shape: tuple[int, ...]
    init: str = "normal"
    std: float = 0.02
    merged_from: tuple[str, ...] = ()
    merged_rows: tuple[int, ...] = ()
    keep_32bit: bool = False
    integer: bool = False


# ------------------------------------------------------------------------ cache needs
@dataclass(frozen=True)
class KVNeed:
    """Pages of keys and values: ``num_kv_heads x head_dim`` per token, for every position
    (``window=None``) or only the last ``window`` positions."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A slot of fixed size per request: ``shape`` elements of ``dtype``, zero at the
    request's first token, carried from step to step."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class KVCacheEntry:
    """The cache one call of a layer owns: ``k``/``v`` are ``[pages, kv_heads, page_size,
    head_dim]``; ``group`` finds this call's block tables and slots in the step context."""

    group: int
    k: torch.Tensor
    v: torch.Tensor
    page_size: int


@dataclass
class StateCacheEntry:
    """``state`` is ``[slots, *shape]``; row ``ctx.state_slots[b]`` belongs to request b."""

    state: torch.Tensor


# ----------------------------------------------------------------------- step context
@dataclass
class KVGroupContext:
    """Per step and per page group: ``block_tables [B, W]`` and ``slots [T]`` (int32).
    ``slots[t] = page * page_size + offset`` of the new token t."""

    page_size: int
    block_tables: torch.Tensor
    slots: torch.Tensor


@dataclass
class StepContext:
    """Everything about one step that the parts may read. Built once per step."""

    num_tokens: int
    num_seqs: int
    query_lens: list[int]            # host: new tokens of each request in this step
    context_lens: list[int]          # host: tokens of each request, the new ones included
    tokens: torch.Tensor             # [T] int32
    positions: torch.Tensor          # [T] int32
    cu_query_lens: torch.Tensor      # [B + 1] int32
    context_lens_dev: torch.Tensor   # [B] int32
    decode_seqs: torch.Tensor        # [Nd] int32: requests that bring exactly one token
    prefill_seqs: torch.Tensor       # [Np] int32: requests that bring more
    num_decode: int
    num_prefill: int
    max_query_len: int
    max_context_len: int
    kv: dict[int, KVGroupContext]
    state_slots: torch.Tensor | None  # [B] int32
    state_slots_host: list[int]
    arena: "Any"
    dtype: torch.dtype
    position_tables: dict[Any, Any] = field(default_factory=dict)
    # Weights that the kernels after the current mixer will stream (set by the block): a mixer
    # with a long kernel that leaves memory bandwidth idle may have them fetched into L2 beside it.
    upcoming_weights: list[torch.Tensor] = field(default_factory=list)


class ResidualStream:
    """The residual stream of one step: ``resid`` is 32-bit ``[T, hidden]``; ``delta`` is the
    last sub-layer's output in the model dtype, not yet added. ``sumsq``, when set, holds the
    sums of squares of the rows of ``resid`` in parts, left by the product that last added to the
    stream (``ops.gemm_to_stream``) together with ``resid16``, a copy of the stream in the model
    dtype; both are valid only while ``delta`` is None."""

    __slots__ = ("resid", "delta", "sumsq", "resid16", "_sumsq_buf", "_resid16_buf")

    def __init__(self, resid: torch.Tensor, delta: torch.Tensor | None = None) -> None:
        self.resid = resid
        self.delta = delta
        self.sumsq: torch.Tensor | None = None
        self.resid16: torch.Tensor | None = None
        self._sumsq_buf: torch.Tensor | None = None
        self._resid16_buf: torch.Tensor | None = None

    def fusion_buffers(self, ctx: "StepContext") -> tuple[torch.Tensor, torch.Tensor]:
        """Scratch for the stream's copy in the model dtype and for the parts of the rows' sums
        of squares (one float per column)."""
        if self._sumsq_buf is None:
            self._sumsq_buf = ctx.arena.take_step((self.resid.shape[1],), torch.float32)
            self._resid16_buf = ctx.arena.take_step(tuple(self.resid.shape), ctx.dtype)
        return self._resid16_buf, self._sumsq_buf


class LazyNormed:
    """A normalised activation that is not computed yet: a part that can apply the norm while
    it loads the stream (``project`` below) reads ``stream``, ``weight`` and ``eps``; any other
    use calls ``tensor()``, which runs the norm's own kernel once."""

    __slots__ = ("stream", "weight", "eps", "_make", "_tensor")

    def __init__(self, stream: ResidualStream, weight: torch.Tensor, eps: float,
                 make: Callable[[], torch.Tensor]) -> None:
        self.stream, self.weight, self.eps, self._make = stream, weight, eps, make
        self._tensor: torch.Tensor | None = None

    @property
    def shape(self) -> torch.Size:
        return self.stream.resid.shape

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self._make()
        return self._tensor


def project(x: "torch.Tensor | LazyNormed", w: torch.Tensor, out: torch.Tensor, ctx: "StepContext",
            swiglu: bool = False) -> None:
    """``out = x @ w^T`` (``swiglu``: ``silu(x Wgate^T) * (x Wup^T)`` with ``w`` the merged
    matrix). A lazy ``x`` is normalised inside the product where the kernels allow it."""
    from ..kernels import ops

    if isinstance(x, LazyNormed):
        m, k = x.shape
        st = x.stream
        if st.delta is None and st.sumsq is not None and ops.can_stream_fuse(m, w.shape[0], k, k, w.dtype, w.device):
            ops.gemm_normed(st.resid16, st.sumsq, x.weight, x.eps, w, out, swiglu)
            return
        x = x.tensor()
    if swiglu:
        ops.gemm_swiglu(x, w, out, ctx.arena)
    else:
        ops.gemm(x, w, out)


def project_to_stream(x: torch.Tensor, w: torch.Tensor, stream: ResidualStream | None,
                      ctx: "StepContext") -> torch.Tensor | None:
    """A sub-layer's output product. With a ``stream`` and few rows the product adds its result
    to the stream itself and returns None; otherwise it returns ``x @ w^T`` for the caller to
    leave pending on the stream."""
    from ..kernels import ops

    m, k = x.shape
    n = w.shape[0]
    if (stream is not None and stream.delta is None and x.dtype == torch.bfloat16
            and ops.can_stream_fuse(m, n, k, n, x.dtype, x.device)):
        copy, parts = stream.fusion_buffers(ctx)
        ops.gemm_to_stream(x, w, stream.resid, copy, parts)
        stream.resid16, stream.sumsq = copy, parts
        return None
    out = ctx.arena.take((m, n), ctx.dtype)
    ops.gemm(x, w, out)
    return out


# ------------------------------------------------------------------------- interfaces
class Part:
    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        return []

    def ignorable_tensors(self, prefix: str) -> set[str]:
        return set()

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        pass


class Norm(Part):
    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def lazy(self, stream: ResidualStream, ctx: StepContext) -> "torch.Tensor | LazyNormed":
        """For parts that declare ``takes_lazy_input``: the norm as a ``LazyNormed`` where the
        stream allows it, else its result."""
        return self.forward(stream, ctx)

    def forward_rows(self, stream: ResidualStream, rows: torch.Tensor, num_rows: int,
                     ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def key(self) -> Any:
        """Encodings with equal keys share one set of tables per step."""
        raise NotImplementedError

    def prepare(self, ctx: StepContext) -> Any:
        raise NotImplementedError


class Mixer(Part):
    # True if ``forward`` reads nothing of the step on the host (no lengths, no slot lists):
    # only then can a decode step with this mixer be recorded once and replayed as a graph.
    graph_safe: bool = False
    # True if ``forward`` accepts a ``LazyNormed`` for ``x`` (and hands it to ``project``).
    takes_lazy_input: bool = False
    # True if ``forward`` has a keyword ``stream`` and may add its output to it (returning None).
    adds_to_stream: bool = False

    def cache_need(self) -> KVNeed | StateNeed | None:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Any, writes_cache: bool,
                position: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    takes_lazy_input: bool = False     # as for Mixer
    adds_to_stream: bool = False

    def streamed_weights(self) -> list[torch.Tensor]:
        """The weight tensors that ``forward`` reads once from end to end, in the order of use
        (what is worth fetching into L2 ahead of it); empty if it is not that simple."""
        return []

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block:
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Any, writes_cache: bool,
                position: Any) -> None:
        raise NotImplementedError


# -------------------------------------------------------------------------- registries
class _Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._items: dict[str, Callable[..., Any]] = {}

    def register(self, name: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
        if not replace and name in self._items and self._items[name] is not factory:
            raise ValueError(f"{self.what} {name!r} is already registered")
        self._items[name] = factory

    def build(self, kind: str, /, *args: Any, **kwargs: Any) -> Any:
        if kind not in self._items:
            raise KeyError(f"unknown {self.what} {kind!r}; known: {sorted(self._items)}")
        return self._items[kind](*args, **kwargs)

    def names(self) -> list[str]:
        return sorted(self._items)


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITION_ENCODINGS = _Registry("position encoding")
BLOCKS = _Registry("block")
EMBEDDINGS = _Registry("embedding")
HEADS = _Registry("output head")


def register_mixer(name: str, factory: Callable[..., Mixer], **kw: Any) -> None:
    MIXERS.register(name, factory, **kw)


def register_feed_forward(name: str, factory: Callable[..., FeedForward], **kw: Any) -> None:
    FEED_FORWARDS.register(name, factory, **kw)


def register_norm(name: str, factory: Callable[..., Norm], **kw: Any) -> None:
    NORMS.register(name, factory, **kw)


def register_position_encoding(name: str, factory: Callable[..., PositionEncoding], **kw: Any) -> None:
    POSITION_ENCODINGS.register(name, factory, **kw)


def register_block(name: str, factory: Callable[..., Block], **kw: Any) -> None:
    BLOCKS.register(name, factory, **kw)
