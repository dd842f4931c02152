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
from ..sampling.sampler import Sampler, TokenLogprobs, derive_seed, token_logprobs
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


class Engine:
    def __init__(self, model: DecoderModel, cache: CacheManager, max_num_seqs: int = 64,
                 max_batch_tokens: int = 2048, clock: Callable[[], float] = time.perf_counter,
                 seed: int = 0, trace_steps: bool = False, chunked_prefill: bool = False,
                 runner: ModelRunner | None = None, decode_graphs: bool = False,
                 graph_max_context: int | None = None) -> None:
        """``decode_graphs``: record the decode step once per batch-size bucket (CUDA graphs)
        and replay it whenever every scheduled request brings one token (upstream passes a
        ``DecodeGraphs`` object for this, src/tinyserve/engine.py:96,188-196)."""
        self.model = model
        self.cache = cache
        self.runner = runner if runner is not None else ModelRunner(model, cache)
        if decode_graphs and not self.runner.graphs:
            limit = min(model.spec.max_position_embeddings, cache.num_pages * cache.page_size)
            self.runner.record_decode_graphs(max_num_seqs, graph_max_context or limit)
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
        return self.scheduler.has_work()

    def abort(self, request_id: int) -> None:
        self.scheduler.abort(self.requests[request_id])

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

    def step(self) -> list[Request]:
        """Run one step. Returns the requests that finished in it."""
        s = self.scheduler
        marks: list[float] = []
        self._mark(marks)
        s.schedule()
        reqs = s.scheduled()
        if not reqs:
            raise RuntimeError("the scheduler made no progress with requests still queued")
        self.kv_utilization.append(self.cache.utilization)
        entries, want = [], []
        for r in reqs:
            end = r.cache.num_tokens
            toks = r.token_slice(end - r.num_scheduled, end)
            entries.append(StepEntry(r.cache, toks))
            want.append([] if r.in_prefill() else [len(toks) - 1])
        context = sum(r.cache.num_tokens for r in reqs)
        self._mark(marks)
        logits = self.runner.step(entries, want)
        self._mark(marks)
        sampled = [r for r in reqs if not r.in_prefill()]
        next_tokens: list[int] = []
        if sampled:
            params = [r.sampling for r in sampled]
            next_tokens = self.sampler.sample(
                logits, params, [self._seeds[r.request_id] for r in sampled], [len(r.output) for r in sampled])
            rows = [j for j, p in enumerate(params) if p.logprobs is not None]
            if rows:
                idx = torch.tensor(rows, device=logits.device)
                lps = token_logprobs(logits[idx], [next_tokens[j] for j in rows], [params[j].logprobs or 0 for j in rows])
                for j, lp in zip(rows, lps):
                    self.logprobs[sampled[j].request_id].append(lp)
        self._mark(marks)
        now = self.clock()
        for r in sampled:
            self.times[r.request_id].tokens.append(now)
        self.num_steps += 1
        finished = s.update(sampled, next_tokens)
        if self.step_records is not None:
            self._mark(marks)
            ms = [(b - a) * 1e3 for a, b in zip(marks, marks[1:])]
            self.step_records.append(StepRecord(
                num_seqs=len(reqs), num_prefill_seqs=sum(len(e.tokens) > 1 for e in entries),
                num_tokens=sum(len(e.tokens) for e in entries), context_tokens=context,
                schedule_ms=ms[0], forward_ms=ms[1], sample_ms=ms[2], update_ms=ms[3]))
        return finished

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 eos_ids: frozenset[int] = frozenset(), sampling: SamplingParams | None = None) -> list[list[int]]:
        """Run all prompts to completion together; outputs in the order of ``prompts``."""
        ids = [self.add_request(p, max_new_tokens, eos_ids, sampling) for p in prompts]
        while self.has_work():
            self.step()
        return [self.requests[i].output for i in ids]
