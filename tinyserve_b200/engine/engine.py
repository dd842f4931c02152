"""The serving loop: the scheduler above the step function, one step at a time.

    engine = Engine(model, cache)
    ids = [engine.add_request(p, max_new_tokens=64) for p in prompts]
    while engine.has_work():
        engine.step()              # requests may be added between steps

Each step: the scheduler picks the requests and reserves cache room, the step function runs all
their tokens as one batch and returns logits for the requests that ran their last pending
token, the sampler picks one token for each, and the scheduler records them and retires what is
done. Names and meanings of the constructor arguments and methods follow upstream
src/tinyserve/engine.py:86-269 (``add_request``, ``step``, ``has_work``, ``abort``,
``release``, ``generate``, per-request ``times`` with ``ttft``/``tpot``, ``trace_steps``).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch

from ..cache.manager import CacheManager
from ..model import DecoderModel
from ..sampling.params import SamplingParams
from ..sampling.sampler import SampleTicket, Sampler, TokenLogprobs, derive_seed, token_logprobs
from .request import Request, Status
from .scheduler import Scheduler
from .step import ModelRunner, StepEntry


@dataclass
class RequestTimes:
    arrival: float
    tokens: list[float] = field(default_factory=list)    # when each output token came out

    @property
    def ttft(self) -> float:
        return self.tokens[0] - self.arrival

    @property
    def tpot(self) -> float | None:
        if len(self.tokens) < 2:
            return None
        return (self.tokens[-1] - self.tokens[0]) / (len(self.tokens) - 1)


@dataclass(frozen=True)
class StepRecord:
    num_seqs: int
    num_prefill_seqs: int
    num_tokens: int
    context_tokens: int
    schedule_ms: float
    forward_ms: float      # building the batch, the model, until the device has finished
    sample_ms: float       # sampling and the copy of the tokens to the host
    update_ms: float

    @property
    def total_ms(self) -> float:
        return self.schedule_ms + self.forward_ms + self.sample_ms + self.update_ms


@dataclass
class _StepInFlight:
    """A step that has been launched and whose tokens have not been read yet."""

    reqs: list[Request]                  # the step's requests, in the order of its entries
    sampled: list[Request]               # those of them that draw a token
    ticket: SampleTicket | None          # their tokens, on the way to the host
    logits: torch.Tensor | None
    entries: list[StepEntry]
    context: int
    replayed: bool                       # it ran as a recorded decode step
    marks: list[float]


class Engine:
    def __init__(self, model: DecoderModel, cache: CacheManager, max_num_seqs: int = 64,
                 max_batch_tokens: int = 2048, clock: Callable[[], float] = time.perf_counter,
                 seed: int = 0, trace_steps: bool = False, chunked_prefill: bool = False,
                 runner: ModelRunner | None = None, decode_graphs: bool = False,
                 graph_max_context: int | None = None, run_ahead: bool = True, prefill_graph: bool = True,
                 record_logits: bool = False) -> None:
        """``decode_graphs``: record the decode step once per batch-size bucket (CUDA graphs)
        and replay it whenever every scheduled request brings one token (upstream passes a
        ``DecodeGraphs`` object for this, src/tinyserve/engine.py:96,188-196). A model with a
        mixer that does not allow it (``Mixer.recordable``) runs kernel by kernel instead.

        ``prefill_graph`` (with ``decode_graphs`` and ``chunked_prefill``): the step of one request
        that brings a full portion of ``max_batch_tokens`` prompt tokens is recorded too.

        ``run_ahead``: while a recorded decode step runs, the next one is launched before its
        tokens are read, fed on the device with the tokens it is about to draw, so the host's
        work between two steps (reading tokens, bookkeeping, packing the next step) no longer
        leaves the device idle. It happens only when nothing about the next step depends on
        those tokens (see ``Scheduler.schedule_ahead``) except a possible end token: a request
        that draws one has then run one token too many, which is dropped. ``step()`` still
        returns one step's finished requests per call, in order.

        ``record_logits`` (tests, debugging): every step's logits rows are copied on the device as
        the step is launched and kept in ``logits_log`` as ``(request id, position, row)``: the
        float32 logits that predict the token after ``position`` of that request's tokens."""
        self.model = model
        self.cache = cache
        self.runner = runner if runner is not None else ModelRunner(model, cache)
        if decode_graphs and not self.runner.graphs:
            limit = min(model.spec.max_position_embeddings, cache.capacity_tokens)
            if model.parts.recordable("decode"):
                self.runner.record_decode_graphs(max_num_seqs, graph_max_context or limit)
            if (prefill_graph and chunked_prefill and max_batch_tokens <= (graph_max_context or limit)
                    and model.parts.recordable("prefill")):
                self.runner.record_prefill_graph(max_batch_tokens, graph_max_context or limit)
        self.scheduler = Scheduler(cache, max_num_seqs, max_batch_tokens, chunked_prefill=chunked_prefill)
        self.sampler = Sampler(model.device, max_rows=max(max_num_seqs, 1))
        self.clock = clock
        self.seed = seed
        self.requests: dict[int, Request] = {}
        self.times: dict[int, RequestTimes] = {}
        self.logprobs: dict[int, list[TokenLogprobs]] = {}
        self.num_steps = 0
        self.kv_utilization: list[float] = []
        self.step_records: list[StepRecord] | None = [] if trace_steps else None
        self._next_id = 0
        self._seeds: dict[int, int] = {}
        self.run_ahead = run_ahead and trace_steps is False
        self.num_steps_ahead = 0
        self._inflight: _StepInFlight | None = None
        self.logits_log: list[tuple[int, int, torch.Tensor]] | None = [] if record_logits else None

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], max_new_tokens: int,
                    eos_ids: frozenset[int] = frozenset(), sampling: SamplingParams | None = None) -> int:
        prompt = [int(t) for t in prompt]
        vocab = self.model.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"prompt has a token id outside 0..{vocab - 1}")
        rid = self._next_id
        params = sampling or SamplingParams()
        req = Request(rid, prompt, max_new_tokens, frozenset(eos_ids), params)
        self.scheduler.add(req)
        self._next_id += 1
        self.requests[rid] = req
        self.times[rid] = RequestTimes(arrival=self.clock())
        self._seeds[rid] = params.seed if params.seed is not None else derive_seed(self.seed, rid)
        if params.logprobs is not None:
            self.logprobs[rid] = []
        return rid

    def has_work(self) -> bool:
        return self._inflight is not None or self.scheduler.has_work()

    def abort(self, request_id: int) -> None:
        self.scheduler.abort(self.requests[request_id])
        cur = self._inflight
        if cur is not None and not any(r.status is Status.RUNNING for r in cur.reqs):
            # the step under way served nobody else: its tokens are read and dropped
            self._inflight = None
            if cur.ticket is not None:
                cur.ticket.wait()

    def release(self, request_id: int) -> None:
        """Forget a finished request's records."""
        if self.requests[request_id].status is not Status.FINISHED:
            raise ValueError(f"request {request_id} has not finished; abort it first")
        del self.requests[request_id], self.times[request_id]
        self._seeds.pop(request_id, None)
        self.logprobs.pop(request_id, None)

    # ---------------------------------------------------------------------- step
    def _mark(self, marks: list[float]) -> None:
        if self.step_records is None:
            return
        if self.model.device.type == "cuda":
            torch.cuda.synchronize(self.model.device)
        marks.append(self.clock())

    def _launch(self, reqs: list[Request], marks: list[float], ahead: _StepInFlight | None) -> _StepInFlight:
        """Launch the step of ``reqs`` (already scheduled) and the draw of its tokens. ``ahead``:
        the step before, still unread; this one takes its tokens on the device."""
        self.kv_utilization.append(self.cache.utilization)
        entries, want = [], []
        for r in reqs:
            end = r.cache.num_tokens
            # the token of a step launched ahead is not known here: a stand-in that the device overwrites
            toks = [0] if ahead is not None else r.token_slice(end - r.num_scheduled, end)
            entries.append(StepEntry(r.cache, toks))
            want.append([len(toks) - 1] if ahead is not None or not r.in_prefill() else [])
        context = sum(r.cache.num_tokens for r in reqs)
        self._mark(marks)
        replayed = self.runner.replays(entries, want)
        if ahead is not None:
            logits = self.runner.step(entries, want, tokens_from=ahead.ticket.device_tokens)
        else:
            logits = self.runner.step(entries, want)
        self._mark(marks)
        sampled = reqs if ahead is not None else [r for r in reqs if not r.in_prefill()]
        if self.logits_log is not None and sampled:
            rows = logits[: len(sampled)].clone()      # a step launched ahead reuses the buffer before this one is read
            self.logits_log.extend((r.request_id, r.cache.num_tokens - 1, rows[j]) for j, r in enumerate(sampled))
        ticket = None
        if sampled:
            drawn = 1 if ahead is not None else 0        # the token under way counts as drawn
            ticket = self.sampler.launch(
                logits, [r.sampling for r in sampled], [self._seeds[r.request_id] for r in sampled],
                [len(r.output) + drawn for r in sampled])
        return _StepInFlight(reqs, sampled, ticket, logits, entries, context, replayed, marks)

    def _launch_ahead(self, cur: _StepInFlight) -> _StepInFlight | None:
        """The step after ``cur``, launched before ``cur``'s tokens are read, if that is safe."""
        if not (self.run_ahead and cur.replayed and cur.ticket is not None and len(cur.sampled) == len(cur.reqs)):
            return None
        if any(r.sampling.logprobs is not None or r.status is not Status.RUNNING for r in cur.reqs):
            return None
        if self.scheduler.running != cur.reqs:           # the same requests, row for row
            return None
        if any(r.cache.num_tokens + 1 > self.runner.graph_max_context for r in cur.reqs):
            return None                                   # beyond what the recorded steps take
        reqs = self.scheduler.schedule_ahead()
        if reqs is None:
            return None
        self.num_steps_ahead += 1
        return self._launch(reqs, [], cur)

    def _collect(self, cur: _StepInFlight) -> list[Request]:
        """Read a launched step's tokens and record them; returns the requests it finished."""
        marks = cur.marks
        # a request that ended (end token, abort) while this step was already under way is skipped
        live = [j for j, r in enumerate(cur.sampled) if r.status is Status.RUNNING]
        sampled = [cur.sampled[j] for j in live]
        next_tokens: list[int] = []
        if cur.ticket is not None:
            drawn = cur.ticket.wait()
            next_tokens = [drawn[j] for j in live]
            params = [r.sampling for r in sampled]
            rows = [j for j, p in zip(live, params) if p.logprobs is not None]
            if rows:
                idx = torch.tensor(rows, device=cur.logits.device)
                lps = token_logprobs(cur.logits[idx], [drawn[j] for j in rows],
                                     [cur.sampled[j].sampling.logprobs or 0 for j in rows])
                for j, lp in zip(rows, lps):
                    self.logprobs[cur.sampled[j].request_id].append(lp)
        self._mark(marks)
        now = self.clock()
        for r in sampled:
            self.times[r.request_id].tokens.append(now)
        self.num_steps += 1
        finished = self.scheduler.update(sampled, next_tokens)
        if self.step_records is not None:
            self._mark(marks)
            ms = [(b - a) * 1e3 for a, b in zip(marks, marks[1:])]
            self.step_records.append(StepRecord(
                num_seqs=len(cur.reqs), num_prefill_seqs=sum(len(e.tokens) > 1 for e in cur.entries),
                num_tokens=sum(len(e.tokens) for e in cur.entries), context_tokens=cur.context,
                schedule_ms=ms[0], forward_ms=ms[1], sample_ms=ms[2], update_ms=ms[3]))
        return finished

    def step(self) -> list[Request]:
        """Run one step. Returns the requests that finished in it."""
        cur = self._inflight
        if cur is None:
            marks: list[float] = []
            self._mark(marks)
            self.scheduler.schedule()
            reqs = self.scheduler.scheduled()
            if not reqs:
                raise RuntimeError("the scheduler made no progress with requests still queued")
            cur = self._launch(reqs, marks, None)
        self._inflight = self._launch_ahead(cur)       # keeps the device busy while the host reads cur
        return self._collect(cur)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 eos_ids: frozenset[int] = frozenset(), sampling: SamplingParams | None = None) -> list[list[int]]:
        """Run all prompts to completion together; outputs in the order of ``prompts``."""
        ids = [self.add_request(p, max_new_tokens, eos_ids, sampling) for p in prompts]
        while self.has_work():
            self.step()
        return [self.requests[i].output for i in ids]
