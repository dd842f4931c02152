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
* ``PositionEncoding``: ``prepare(ctx)`` once per step returns the step's position data, an
  object with one method, ``qk_rotation()``: the rotation the mixer applies to its queries and
  keys (``Rotation``: cos/sin per token, how many elements of a head turn, how they pair up),
  or ``None`` if queries and keys stay as they are.
* ``Mixer``: ``cache_need()`` says what it keeps between steps, as a ``CacheNeed``: a
  ``PagedNeed`` (pages per token: ``KVNeed`` is keys and values for all or a window of the
  positions; a mixer may define its own), a ``SlotNeed`` (``StateNeed``: a fixed-size state per
  request), or nothing; ``forward(x, ctx, cache, writes_cache) -> [T, hidden]``.
* ``FeedForward``: ``forward(x, ctx) -> [T, hidden]``.
* ``Block``: names the roles it wants filled (``roles``: role -> family of part) and arranges
  those parts around the stream; ``PreNormBlock`` wants a mixer, a feed-forward and their norms.

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
class CacheNeed:
    """What one call of a mixer keeps between steps. The cache manager knows two families and
    serves any subclass of them through the methods below, so a mixer with a cache of another
    shape (one latent vector per token, keys of another width than the values, ...) defines its
    own frozen dataclass deriving ``PagedNeed`` or ``SlotNeed`` and nothing in the manager changes."""


class PagedNeed(CacheNeed):
    """Memory per token, in pages. Calls whose needs compare equal share a page group (one pool
    of pages, one block table per request). ``window``: only the last ``window`` positions are
    ever read again (pages behind it are given back early); ``None`` keeps every position."""

    window: int | None = None

    def bytes_per_token(self, element_size: int) -> int:
        raise NotImplementedError

    def allocate(self, num_calls: int, num_pages: int, page_size: int, dtype: torch.dtype,
                 device: torch.device) -> torch.Tensor:
        """The storage of a whole group: ``num_pages`` already counts the pad page (the last one,
        never handed out, where fixed-shape padding rows may write). Zero-filled."""
        raise NotImplementedError

    def entry(self, storage: torch.Tensor, call_in_group: int, group: int, page_size: int) -> Any:
        """What the mixer's ``forward`` receives as ``cache`` for one call: views into ``storage``
        and ``group``, the key of this call's block tables and slots in ``StepContext.kv``."""
        raise NotImplementedError


class SlotNeed(CacheNeed):
    """Memory of fixed size per request, in slots: zero at the request's first token, carried from
    step to step, lost (recomputed) on preemption. One extra slot after the pool is never handed
    out; fixed-shape padding rows of a recorded step use it."""

    def allocate(self, num_slots: int, device: torch.device) -> torch.Tensor:
        """``[num_slots, ...]`` zero-filled; ``num_slots`` already counts the pad slot."""
        raise NotImplementedError

    def entry(self, storage: torch.Tensor) -> Any:
        raise NotImplementedError


@dataclass(frozen=True)
class KVNeed(PagedNeed):
    """Pages of keys and values: ``num_kv_heads x head_dim`` per token, for every position
    (``window=None``) or only the last ``window`` positions. Storage
    ``[call, k|v, page, kv_head, offset, head_dim]``: the keys of one (page, kv head) are one
    contiguous run of ``page_size * head_dim`` elements, the unit a bulk copy moves."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None

    def bytes_per_token(self, element_size: int) -> int:
        return 2 * self.num_kv_heads * self.head_dim * element_size

    def allocate(self, num_calls, num_pages, page_size, dtype, device):
        return torch.zeros((num_calls, 2, num_pages, self.num_kv_heads, page_size, self.head_dim), dtype=dtype, device=device)

    def entry(self, storage, call_in_group, group, page_size):
        return KVCacheEntry(group, storage[call_in_group, 0], storage[call_in_group, 1], page_size)


@dataclass(frozen=True)
class StateNeed(SlotNeed):
    """A slot of fixed size per request: ``shape`` elements of ``dtype``."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def allocate(self, num_slots, device):
        return torch.zeros((num_slots, *self.shape), dtype=self.dtype, device=device)

    def entry(self, storage):
        return StateCacheEntry(storage)


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
    """``state`` is ``[slots + 1, *shape]``; row ``ctx.state_slots[b]`` belongs to request b (the
    last row is the pad slot of recorded steps' padding rows)."""

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
    # The cache entries of the next call of the order, by mixer role (set by the model): a mixer may
    # have their pages fetched into L2 once its own kernel has gone over the memory.
    upcoming_caches: Mapping[str, Any] = field(default_factory=dict)
    # Side branches that a part has opened and that nothing later in the step reads from (such a
    # prefetch): functions that join them, called once at the end of the step.
    at_step_end: list[Callable[[], None]] = field(default_factory=list)


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
        of squares (up to 16 rows x a part per 8 columns: two floats per column)."""
        if self._sumsq_buf is None:
            self._sumsq_buf = ctx.arena.take_step((2 * self.resid.shape[1],), torch.float32)
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
        copy, scratch = stream.fusion_buffers(ctx)
        stream.sumsq = ops.gemm_to_stream(x, w, stream.resid, copy, scratch)
        stream.resid16 = copy
        return None
    out = ctx.arena.take((m, n), ctx.dtype)
    ops.gemm(x, w, out)
    return out


# ------------------------------------------------------------------------- interfaces
EVERY_STEP = frozenset({"decode", "prefill"})


class Part:
    # The kinds of step in which the part reads nothing of the step on the host (no lengths, no
    # slot lists, no result of a device computation) and launches the same work whatever the step's
    # values: "decode" (every request brings one token) and/or "prefill" (one request brings a
    # fixed number of tokens). Only such steps can be recorded once and replayed as a graph; one
    # part that does not allow a kind switches its recording off for the whole model. The default
    # allows nothing; the built-in parts allow both (``EVERY_STEP``). A mixer with state of its own
    # can allow "decode" by indexing its state with ``ctx.state_slots`` on the device.
    recordable: frozenset = frozenset()

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


@dataclass
class Rotation:
    """A rotation of the first ``rotary_dim`` elements of every query and key head by the
    token's angles: ``cos``/``sin`` are ``[T, rotary_dim / 2]`` float32 on the device; pairs are
    ``(i, i + rotary_dim / 2)`` or, ``interleaved``, neighbours ``(2i, 2i + 1)``."""

    cos: torch.Tensor
    sin: torch.Tensor
    rotary_dim: int
    interleaved: bool = False

    def qk_rotation(self) -> "Rotation":
        return self


class PositionEncoding(Part):
    def key(self) -> Any:
        """Encodings with equal keys share one set of tables per step."""
        raise NotImplementedError

    def prepare(self, ctx: StepContext) -> Any:
        """Once per step: the step's position data, an object with the method ``qk_rotation()``
        that returns the ``Rotation`` a mixer applies to its queries and keys, or ``None`` when
        they stay as they are (a ``Rotation`` is such an object itself)."""
        raise NotImplementedError


class Mixer(Part):
    # True if ``forward`` accepts a ``LazyNormed`` for ``x`` (and hands it to ``project``).
    takes_lazy_input: bool = False
    # True if ``forward`` has a keyword ``stream`` and may add its output to it (returning None).
    adds_to_stream: bool = False

    def cache_need(self) -> CacheNeed | None:
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
    """Arranges the parts of one layer around the residual stream. A block class names the roles
    it wants filled: ``roles`` maps a role (a name of the block's own choosing, the key under which
    ``LayerSpec.parts`` gives the part) to the family the part comes from ("mixer",
    "feed_forward" or "norm"); roles in ``optional_roles`` may be left out. The model builds the
    parts in the order of ``roles`` (which is also the order of their tensors) and hands them
    over as a dict. A block with a third norm, two mixers side by side or no feed-forward at all
    is another ``Block`` class and a ``register_block`` call."""

    roles: Mapping[str, str] = {}
    optional_roles: frozenset = frozenset()

    def __init__(self, parts: Mapping[str, Part]) -> None:
        self.parts = dict(parts)

    def mixers(self) -> dict[str, Mixer]:
        """The parts that may keep a cache, by role."""
        return {role: p for role, p in self.parts.items() if isinstance(p, Mixer)}

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, Any], writes_cache: bool,
                position: Any) -> None:
        """``caches[role]`` is the cache entry of the mixer in that role for this call of the
        layer (absent if it keeps nothing)."""
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

    def get(self, kind: str) -> Callable[..., Any]:
        if kind not in self._items:
            raise KeyError(f"unknown {self.what} {kind!r}; known: {sorted(self._items)}")
        return self._items[kind]

    def build(self, kind: str, /, *args: Any, **kwargs: Any) -> Any:
        return self.get(kind)(*args, **kwargs)

    def names(self) -> list[str]:
        return sorted(self._items)


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITION_ENCODINGS = _Registry("position encoding")
BLOCKS = _Registry("block")
EMBEDDINGS = _Registry("embedding")
HEADS = _Registry("output head")
# the families a block's roles may name
PART_FAMILIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}


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
