"""The step function: run a batch of (request, its next tokens) through the model, from the
cache that earlier steps left, and return the logits at the wanted places.

A batch is any mix of portions of prompts and single decoded tokens, flattened request
after request without padding (after upstream src/tinyserve/batch.py:60-115 and
src/tinyserve/model.py:259-329). The caller has already reserved room for the new tokens
in each request's cache (``CacheManager.append``); this function only reads the tables. All
per-step integers (tokens, positions, slots, block tables, lengths, wanted rows) are packed
on the host into ONE pinned buffer and reach the device in one copy.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..model import DecoderModel
from ..kernels import ops
from ..parts.base import KVGroupContext, StepContext
from .arena import Arena


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclass
class StepEntry:
    """One request's share of a step: the request's cache and its next tokens, which must be
    the LAST ``len(tokens)`` positions already reserved in that cache."""

    cache: RequestCache
    tokens: Sequence[int]


def default_buckets(max_batch: int) -> list[int]:
    """Batch sizes a decode graph is recorded for: 1, 2, 4, ... and ``max_batch`` itself
    (after upstream src/tinyserve/cuda_graphs.py:40-49)."""
    out, b = [], 1
    while b < max_batch:
        out.append(b)
        b *= 2
    out.append(max_batch)
    return out


class DecodeGraph:
    """One recorded decode step for a fixed number of rows.

    Every per-step integer lives at a fixed place of one device buffer that the recorded
    kernels read; a step copies this step's values there and replays. Rows beyond the live
    requests are one-token requests on the pad page, whose results nobody reads (after
    upstream src/tinyserve/batch.py:118-206). The graph has scratch memory of its own, which
    never moves once recorded."""

    def __init__(self, runner: "ModelRunner", rows: int, max_context: int) -> None:
        self.rows = rows
        cache, dev = runner.cache, runner.device
        groups = cache.groups
        self.width = -(-max_context // cache.page_size)
        off = 0

        def section(n: int) -> slice:
            nonlocal off
            s = slice(off, off + n)
            off = _round_up(off + n, 4)
            return s

        n = rows
        self.s_tokens, self.s_pos, self.s_cu, self.s_ctx = section(n), section(n), section(n + 1), section(n)
        self.s_dec, self.s_pre, self.s_rows, self.s_state = section(n), section(n), section(n), section(n)
        self.s_slots = [section(n) for _ in groups]
        self.s_tables = [section(n * self.width) for _ in groups]
        self.size = off
        self.host = torch.empty(off, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(off, dtype=torch.int32, device=dev)
        self.copied = torch.cuda.Event()
        self.arena = Arena(dev)
        buf = self.host_np
        buf[:] = 0
        buf[self.s_cu] = np.arange(n + 1)
        buf[self.s_dec] = np.arange(n)
        buf[self.s_rows] = np.arange(n)
        self._fill_padding(runner, 0)
        self.dev.copy_(self.host)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self._row_owner: dict[tuple[int, int], tuple[int, int, int]] = {}   # (group, row) -> what its table row holds
        self._live_rows = 0

    def _fill_padding(self, runner: "ModelRunner", live: int) -> None:
        buf, n = self.host_np, self.rows
        buf[self.s_tokens][live:] = 0
        buf[self.s_pos][live:] = 0
        buf[self.s_ctx][live:] = 1
        buf[self.s_state][live:] = runner.cache.state_pool.pad_slot      # a row of state that belongs to nobody
        for g, ss, st in zip(runner.cache.groups, self.s_slots, self.s_tables):
            buf[ss][live:] = g.pad_page * g.page_size
            buf[st].reshape(n, self.width)[live:, 0] = g.pad_page

    def context(self, runner: "ModelRunner") -> StepContext:
        n, dev, w = self.rows, self.dev, self.width
        cache = runner.cache
        kv = {g.index: KVGroupContext(g.page_size, dev[st].view(n, w), dev[ss])
              for g, ss, st in zip(cache.groups, self.s_slots, self.s_tables)}
        cap = w * cache.page_size
        return StepContext(
            num_tokens=n, num_seqs=n, query_lens=[1] * n, context_lens=[cap] * n,
            tokens=dev[self.s_tokens], positions=dev[self.s_pos], cu_query_lens=dev[self.s_cu],
            context_lens_dev=dev[self.s_ctx], decode_seqs=dev[self.s_dec], prefill_seqs=dev[self.s_pre],
            num_decode=n, num_prefill=0, max_query_len=1, max_context_len=cap, kv=kv,
            state_slots=dev[self.s_state] if cache.has_state else None, state_slots_host=[0] * n,
            arena=self.arena, dtype=runner.model.dtype)

    def record(self, runner: "ModelRunner") -> None:
        model, caches = runner.model, runner.cache.entries

        def run() -> torch.Tensor:
            self.arena.begin_step()
            with ops.stream_scope():
                return model.forward(self.context(runner), caches, self.dev[self.s_rows], self.rows)

        # Twice without recording: the first sizes the scratch memory, the second shows that
        # it no longer moves; then the same launches are recorded.
        run()
        run()
        reserved = self.arena.reserved_bytes
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph):
            logits = run()
        self.num_kernels = ops.launch_count - before
        ops.launch_count = before          # recorded, not run
        if self.arena.reserved_bytes != reserved:
            raise RuntimeError("scratch memory moved while a decode graph was being recorded")
        self.graph, self.logits = graph, logits

    def fill(self, runner: "ModelRunner", entries: Sequence[StepEntry]) -> None:
        self.copied.synchronize()          # the last copy must have left the host buffer
        buf, n, b = self.host_np, self.rows, len(entries)
        buf[self.s_tokens][:b] = [e.tokens[0] for e in entries]
        totals = [e.cache.num_tokens for e in entries]
        buf[self.s_ctx][:b] = totals
        buf[self.s_pos][:b] = np.asarray(totals, dtype=np.int32) - 1
        buf[self.s_state][:b] = [e.cache.state_slot for e in entries]
        owners = self._row_owner
        for g, ss, st in zip(runner.cache.groups, self.s_slots, self.s_tables):
            ps = g.page_size
            slots, table = buf[ss], buf[st].reshape(n, self.width)
            for i, e in enumerate(entries):
                bt = e.cache.tables[g.index]
                pages = bt.pages
                p = totals[i] - 1
                slots[i] = pages[p // ps] * ps + p % ps
                # A row that still belongs to the same request with as many pages as it had is
                # already right in the buffer (decoding adds a page every page_size steps).
                key = (e.cache.uid, len(pages), bt._first_live)
                if owners.get((g.index, i)) != key:
                    arr = bt.pages_array()
                    table[i, : arr.shape[0]] = arr
                    owners[(g.index, i)] = key
        if b != self._live_rows:
            self._fill_padding(runner, b)
            for key in [k for k in owners if k[1] >= b]:
                del owners[key]
            self._live_rows = b
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()


class PrefillGraph:
    """One recorded step of ONE request that brings exactly ``tokens`` new tokens (a portion of
    a long prompt, as chunked prefill cuts them) on top of any context up to ``max_context``.
    A step of a few thousand tokens launches some 250 kernels whose host-side cost is as long
    as their run time at small model sizes; replayed from a recording it costs one launch. The
    logits of the portion's last token are always computed (a mid-prompt portion ignores them)."""

    def __init__(self, runner: "ModelRunner", tokens: int, max_context: int) -> None:
        self.tokens = t = tokens
        cache, dev = runner.cache, runner.device
        groups = cache.groups
        self.width = -(-max_context // cache.page_size)
        off = 0

        def section(n: int) -> slice:
            nonlocal off
            s = slice(off, off + n)
            off = _round_up(off + n, 4)
            return s

        self.s_tokens, self.s_pos, self.s_cu, self.s_ctx = section(t), section(t), section(2), section(1)
        self.s_dec, self.s_pre, self.s_rows, self.s_state = section(1), section(1), section(1), section(1)
        self.s_slots = [section(t) for _ in groups]
        self.s_tables = [section(self.width) for _ in groups]
        self.host = torch.empty(off, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(off, dtype=torch.int32, device=dev)
        self.copied = torch.cuda.Event()
        self.arena = Arena(dev)
        buf = self.host_np
        buf[:] = 0
        buf[self.s_cu] = [0, t]
        buf[self.s_ctx] = t
        buf[self.s_pos] = np.arange(t)
        buf[self.s_rows] = t - 1
        for g, ss, st in zip(groups, self.s_slots, self.s_tables):
            # until the first fill: every token on the pad page
            buf[ss] = g.pad_page * g.page_size + np.arange(t) % g.page_size
            buf[st] = g.pad_page
        self.dev.copy_(self.host)
        self._arange = np.arange(t, dtype=np.int64)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None

    def context(self, runner: "ModelRunner") -> StepContext:
        t, dev, w = self.tokens, self.dev, self.width
        cache = runner.cache
        kv = {g.index: KVGroupContext(g.page_size, dev[st].view(1, w), dev[ss])
              for g, ss, st in zip(cache.groups, self.s_slots, self.s_tables)}
        cap = w * cache.page_size
        return StepContext(
            num_tokens=t, num_seqs=1, query_lens=[t], context_lens=[cap],
            tokens=dev[self.s_tokens], positions=dev[self.s_pos], cu_query_lens=dev[self.s_cu],
            context_lens_dev=dev[self.s_ctx], decode_seqs=dev[self.s_dec], prefill_seqs=dev[self.s_pre],
            num_decode=0, num_prefill=1, max_query_len=t, max_context_len=cap, kv=kv,
            state_slots=dev[self.s_state] if cache.has_state else None, state_slots_host=[0],
            arena=self.arena, dtype=runner.model.dtype)

    def record(self, runner: "ModelRunner") -> None:
        model, caches = runner.model, runner.cache.entries

        def run() -> torch.Tensor:
            self.arena.begin_step()
            with ops.stream_scope():
                return model.forward(self.context(runner), caches, self.dev[self.s_rows], 1)

        run()
        run()
        reserved = self.arena.reserved_bytes
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph):
            logits = run()
        self.num_kernels = ops.launch_count - before
        ops.launch_count = before          # recorded, not run
        if self.arena.reserved_bytes != reserved:
            raise RuntimeError("scratch memory moved while a prefill graph was being recorded")
        self.graph, self.logits = graph, logits

    def fill(self, runner: "ModelRunner", entry: StepEntry) -> None:
        self.copied.synchronize()          # the last copy must have left the host buffer
        buf, t = self.host_np, self.tokens
        total = entry.cache.num_tokens
        first = total - t
        buf[self.s_tokens] = entry.tokens
        buf[self.s_pos] = self._arange + first
        buf[self.s_ctx] = total
        buf[self.s_state] = entry.cache.state_slot
        for g, ss, st in zip(runner.cache.groups, self.s_slots, self.s_tables):
            ps = g.page_size
            arr = entry.cache.tables[g.index].pages_array()
            buf[st][: arr.shape[0]] = arr
            pos = self._arange + first
            buf[ss] = arr[pos // ps].astype(np.int64) * ps + pos % ps
        self.dev.copy_(self.host, non_blocking=True)
        self.copied.record()


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager) -> None:
        self.model = model
        self.cache = cache
        self.device = model.device
        self.arena = Arena(self.device)
        # choose the launch-overlap mask per step (prefill or decode); a caller that sets the
        # mask itself (measurements) turns this off
        self.tune_launch_overlap = True
        self.graphs: dict[int, DecodeGraph] = {}
        self.prefill_graphs: dict[int, PrefillGraph] = {}
        self.graph_max_context = 0
        self.num_graph_steps = 0
        self._host: torch.Tensor | None = None     # pinned int32 staging buffer
        self._host_np: np.ndarray | None = None
        self._dev: torch.Tensor | None = None
        self._copied: torch.cuda.Event | None = None   # the staging buffer's last copy
        self.num_steps = 0

    # ------------------------------------------------------------------ staging
    def _staging(self, n: int) -> None:
        if self._copied is not None:
            # The host buffer is about to be rewritten: its last copy must have left it.
            self._copied.synchronize()
        if self._host is None or self._host.numel() < n:
            cap = max(_round_up(n, 1024), 4096)
            pin = self.device.type == "cuda"
            self._host = torch.empty(cap, dtype=torch.int32, pin_memory=pin)
            self._host_np = self._host.numpy()
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)

    def build_context(self, entries: Sequence[StepEntry], want: Sequence[Sequence[int]] | None
                      ) -> tuple[StepContext, torch.Tensor | None, int]:
        """Pack the step's integers and make the ``StepContext``. ``want[b]`` lists the
        places among request b's tokens whose logits are asked for; ``None`` asks for the
        last token of every request."""
        if not entries:
            raise ValueError("a step needs at least one request")
        groups = self.cache.groups
        b = len(entries)
        query_lens = [len(e.tokens) for e in entries]
        totals = [e.cache.num_tokens for e in entries]
        for n, total in zip(query_lens, totals):
            if not 0 < n <= total:
                raise ValueError(f"{n} new tokens but the request's cache holds {total} positions")
        t = sum(query_lens)
        if want is None:
            want = [[n - 1] for n in query_lens]
        if len(want) != b:
            raise ValueError(f"{b} requests but {len(want)} lists of wanted places")
        rows: list[int] = []
        start = 0
        for n, places in zip(query_lens, want):
            for p in places:
                if not 0 <= p < n:
                    raise ValueError(f"wanted place {p} is not among the request's {n} tokens")
                rows.append(start + p)
            start += n
        r = len(rows)
        widths = [max(len(e.cache.tables[g.index].pages) for e in entries) for g in groups]

        # ---- layout of the packed buffer (every section starts on a 16-byte boundary)
        off = 0

        def section(n: int) -> slice:
            nonlocal off
            s = slice(off, off + n)
            off = _round_up(off + n, 4)
            return s

        s_tokens, s_pos = section(t), section(t)
        s_cu, s_ctx = section(b + 1), section(b)
        s_dec, s_pre = section(b), section(b)
        s_rows, s_state = section(r), section(b)
        s_slots = [section(t) for _ in groups]
        s_tables = [section(b * w) for w in widths]
        self._staging(off)
        buf = self._host_np

        # ---- fill
        tok = buf[s_tokens]
        pos = buf[s_pos]
        cu = buf[s_cu]
        cu[0] = 0
        at = 0
        dec: list[int] = []
        pre: list[int] = []
        for i, (e, n, total) in enumerate(zip(entries, query_lens, totals)):
            tok[at: at + n] = e.tokens
            pos[at: at + n] = np.arange(total - n, total, dtype=np.int32)
            at += n
            cu[i + 1] = at
            (dec if n == 1 else pre).append(i)
        buf[s_ctx] = totals
        buf[s_dec][: len(dec)] = dec
        buf[s_pre][: len(pre)] = pre
        buf[s_rows] = rows
        buf[s_state] = [e.cache.state_slot for e in entries]
        for g, ss, st, w in zip(groups, s_slots, s_tables, widths):
            ps = g.page_size
            slots = buf[ss]
            table = buf[st].reshape(b, w)
            table[:] = 0
            at = 0
            for i, (e, n, total) in enumerate(zip(entries, query_lens, totals)):
                pages = e.cache.tables[g.index].pages_array()
                table[i, : pages.shape[0]] = pages
                p = pos[at: at + n]
                slots[at: at + n] = pages[p // ps] * ps + p % ps
                at += n

        dev = self._dev
        dev[:off].copy_(self._host[:off], non_blocking=True)
        if self.device.type == "cuda":
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()

        self.arena.begin_step()
        kv = {
            g.index: KVGroupContext(g.page_size, dev[st].view(b, w), dev[ss])
            for g, ss, st, w in zip(groups, s_slots, s_tables, widths)
        }
        ctx = StepContext(
            num_tokens=t, num_seqs=b, query_lens=query_lens, context_lens=totals,
            tokens=dev[s_tokens], positions=dev[s_pos], cu_query_lens=dev[s_cu],
            context_lens_dev=dev[s_ctx], decode_seqs=dev[s_dec], prefill_seqs=dev[s_pre],
            num_decode=len(dec), num_prefill=len(pre), max_query_len=max(query_lens),
            max_context_len=max(totals), kv=kv,
            state_slots=dev[s_state] if self.cache.has_state else None,
            state_slots_host=[e.cache.state_slot for e in entries],
            arena=self.arena, dtype=self.model.dtype,
        )
        return ctx, (dev[s_rows] if r else None), r

    # ------------------------------------------------------------------- graphs
    @torch.inference_mode()
    def record_decode_graphs(self, max_batch: int, max_context: int, buckets: Sequence[int] | None = None) -> None:
        """Record one decode step per batch-size bucket. Afterwards a step in which every
        request brings exactly one token, asks for that token's logits, and fits the largest
        bucket and ``max_context`` is replayed from the recording instead of being launched
        kernel by kernel."""
        if self.device.type != "cuda":
            raise RuntimeError("decode graphs need a CUDA device")
        if not self.model.parts.recordable("decode"):
            raise RuntimeError("a mixer of this model reads the step on the host; its decode step cannot be recorded")
        self.graph_max_context = max_context
        for rows in sorted(set(buckets or default_buckets(max_batch))):
            if self.tune_launch_overlap:
                ops.use_pdl_mask(ops.decode_pdl_mask(rows))
            g = DecodeGraph(self, rows, max_context)
            g.record(self)
            self.graphs[rows] = g

    @torch.inference_mode()
    def record_prefill_graph(self, tokens: int, max_context: int) -> None:
        """Record the step of one request that brings exactly ``tokens`` tokens. Afterwards such
        a step (whose request holds at most ``max_context`` tokens, and that wants no logits or
        those of its last token) is replayed from the recording."""
        if self.device.type != "cuda":
            raise RuntimeError("prefill graphs need a CUDA device")
        if not self.model.parts.recordable("prefill"):
            raise RuntimeError("a mixer of this model reads the step on the host; its prompt portions cannot be recorded")
        if self.tune_launch_overlap:
            ops.use_pdl_mask(ops.PREFILL_PDL_MASK)
        g = PrefillGraph(self, tokens, max_context)
        g.record(self)
        self.prefill_graphs[tokens] = g
        self.prefill_graph_max_context = max_context

    def _prefill_graph_for(self, entries: Sequence[StepEntry], want: Sequence[Sequence[int]] | None) -> PrefillGraph | None:
        if not self.prefill_graphs or len(entries) != 1:
            return None
        e = entries[0]
        g = self.prefill_graphs.get(len(e.tokens))
        if g is None or e.cache.num_tokens > self.prefill_graph_max_context:
            return None
        if want is not None and list(want[0]) not in ([], [len(e.tokens) - 1]):
            return None
        return g

    def _graph_for(self, entries: Sequence[StepEntry], want: Sequence[Sequence[int]] | None) -> DecodeGraph | None:
        if not self.graphs or len(entries) > max(self.graphs):
            return None
        for e in entries:
            if len(e.tokens) != 1 or e.cache.num_tokens > self.graph_max_context:
                return None
        if want is not None and any(list(w) != [0] for w in want):
            return None
        return self.graphs[min(r for r in self.graphs if r >= len(entries))]

    # --------------------------------------------------------------------- step
    def replays(self, entries: Sequence[StepEntry], want: Sequence[Sequence[int]] | None = None) -> bool:
        """Whether :meth:`step` would replay a recorded decode step for these entries."""
        return self._graph_for(entries, want) is not None

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], want: Sequence[Sequence[int]] | None = None,
             tokens_from: torch.Tensor | None = None) -> torch.Tensor | None:
        """Run one step. Returns float32 logits ``[wanted, vocab]`` in the order of the entries
        and of their wanted places (a view into step scratch: use it before the next step),
        or ``None`` when nothing is wanted. ``tokens_from`` (int32 on the device, one per entry;
        only for steps that :meth:`replays` accepts): the entries' tokens are taken from there
        instead of from the host, so a step can be launched before the host knows them."""
        graph = self._graph_for(entries, want)
        if tokens_from is not None and graph is None:
            raise ValueError("tokens on the device can only feed a recorded decode step")
        if graph is not None:
            graph.fill(self, entries)
            if tokens_from is not None:
                graph.dev[graph.s_tokens][: len(entries)].copy_(tokens_from[: len(entries)], non_blocking=True)
            graph.graph.replay()
            ops.launch_count += graph.num_kernels
            self.num_steps += 1
            self.num_graph_steps += 1
            return graph.logits[: len(entries)]
        pgraph = self._prefill_graph_for(entries, want)
        if pgraph is not None:
            pgraph.fill(self, entries[0])
            pgraph.graph.replay()
            ops.launch_count += pgraph.num_kernels
            self.num_steps += 1
            self.num_graph_steps += 1
            return None if want is not None and not list(want[0]) else pgraph.logits
        ctx, rows, r = self.build_context(entries, want)
        if self.tune_launch_overlap and self.device.type == "cuda":
            ops.use_pdl_mask(ops.PREFILL_PDL_MASK if ctx.num_prefill else ops.decode_pdl_mask(ctx.num_tokens))
        with ops.stream_scope():
            logits = self.model.forward(ctx, self.cache.entries, rows, r)
        self.num_steps += 1
        return logits
