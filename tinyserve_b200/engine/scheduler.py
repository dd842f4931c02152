"""Continuous-batching scheduler: which requests run in the next step and with how many tokens.

Policy, after upstream src/tinyserve/scheduler.py:127-273:

1. Running requests first, oldest first. A decoding request gets one token. With chunked
   prefill a request still in its prompt gets the next portion of it, as large as the token
   budget allows after one token for every decoding request.
2. Then waiting requests are admitted in arrival order while they fit: fewer than
   ``max_num_seqs`` running, tokens within the step's budget (with chunked prefill the prompt
   is cut to the budget), enough free pages (and a free state slot if the model keeps state).
   Admission stops at the first request that does not fit; nobody overtakes.

When pages run out for a running request, the NEWEST running request is preempted: its pages
and state are given back and it returns to the FRONT of the waiting queue; once re-admitted,
its prompt and output are recomputed. If nothing newer is left, the request preempts itself.
The oldest request therefore always makes progress. Requests that could never fit (longer
than the whole cache, or than the step budget when prompts are not chunked) are refused when
they are added.
"""

from __future__ import annotations

from collections import deque

from ..cache.manager import CacheManager
from .request import Request, Status


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int = 64, max_batch_tokens: int = 2048,
                 chunked_prefill: bool = False) -> None:
        if max_num_seqs <= 0 or max_batch_tokens <= 0:
            raise ValueError("max_num_seqs and max_batch_tokens must be positive")
        if chunked_prefill and max_batch_tokens < max_num_seqs:
            raise ValueError(f"chunked prefill needs max_batch_tokens ({max_batch_tokens}) >= "
                             f"max_num_seqs ({max_num_seqs}): every running request decodes one token")
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_batch_tokens = max_batch_tokens
        self.chunked_prefill = chunked_prefill
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []      # in admission order: oldest first
        self.num_preemptions = 0
        self.num_admitted_tokens = 0

    # ------------------------------------------------------------------ intake
    def add(self, req: Request) -> Request:
        if not self.chunked_prefill and req.max_cached_tokens > self.max_batch_tokens:
            raise ValueError(f"request needs up to {req.max_cached_tokens} tokens in one step, "
                             f"max_batch_tokens is {self.max_batch_tokens}")
        if not self.cache.can_ever_hold(req.max_cached_tokens, self.max_batch_tokens):
            raise ValueError(f"request needs up to {req.max_cached_tokens} cached tokens, the cache holds "
                             f"{self.cache.capacity_tokens}")
        req.status = Status.WAITING
        self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- one step
    def schedule(self) -> list[Request]:
        """Pick this step's requests and reserve cache room for their tokens. Each returned
        request runs the ``num_scheduled`` tokens that follow what its cache held before."""
        self._reserve_running()
        self._admit_waiting()
        return list(self.running)

    def schedule_ahead(self) -> list[Request] | None:
        """Reserve the NEXT decode step while the step just scheduled is still running and its
        tokens are unknown. Possible only when that needs no decision that depends on them:
        nobody waits, every running request has just run its last pending token and will not
        reach ``max_new_tokens`` with the token under way, and one more token fits for all of
        them without preempting anybody. Returns the requests (one token each) or None; in
        between, such a request has -1 pending tokens. A request that turns out to have ended
        (an end token) simply leaves as usual; the extra token it was given room for is never
        used."""
        if self.waiting or not self.running:
            return None
        for r in self.running:
            if r.num_scheduled != 1 or r.num_pending() != 0 or len(r.output) + 1 >= r.max_new_tokens:
                return None
        if self.cache.pages_short_for_all([r.cache for r in self.running], 1):
            return None
        for r in self.running:
            self.cache.append(r.cache, 1)
        return list(self.running)

    def _reserve_running(self) -> None:
        queue = deque(self.running)
        self.running = []
        budget = self.max_batch_tokens - sum(1 for r in queue if r.num_pending() == 1)
        while queue:
            req = queue.popleft()
            n = req.num_pending()
            mid_prompt = n > 1          # not counted among the one-token requests when the budget was formed
            if mid_prompt:
                n = min(n, max(budget, 0))
            fits = True
            while n > 0 and self.cache.pages_short(req.cache, n):
                if queue:
                    self._preempt(queue.pop())
                else:
                    self._preempt(req)
                    fits = False
                    break
            if not fits:
                continue
            if n == 0:
                # Mid-prompt with no budget left this step: keeps its place and its cache.
                req.num_scheduled = 0
                self.running.append(req)
                continue
            self.cache.append(req.cache, n)
            req.num_scheduled = n
            self.running.append(req)
            if mid_prompt:
                budget -= n             # also when the portion was cut down to a single token

    def _admit_waiting(self) -> None:
        budget = self.max_batch_tokens - sum(r.num_scheduled for r in self.running)
        while self.waiting:
            req = self.waiting[0]
            if len(self.running) >= self.max_num_seqs or not self.cache.can_admit():
                break
            n = req.num_pending()
            if self.chunked_prefill and budget > 0:
                n = min(n, budget)
            if n > budget:
                break
            if self.cache.pages_short(None, n):
                break
            self.waiting.popleft()
            req.cache = self.cache.new_request()
            self.cache.append(req.cache, n)
            req.num_scheduled = n
            req.status = Status.RUNNING
            self.running.append(req)
            budget -= n
            self.num_admitted_tokens += req.num_tokens

    def _preempt(self, req: Request) -> None:
        self.cache.free(req.cache)
        req.cache = None
        req.num_scheduled = 0
        req.status = Status.WAITING
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)

    def scheduled(self) -> list[Request]:
        """The running requests that take part in the step just scheduled."""
        return [r for r in self.running if r.num_scheduled > 0]

    def update(self, sampled: list[Request], next_tokens: list[int]) -> list[Request]:
        """Record each sampled request's new token, give back pages a window has passed, and
        retire the requests that are done. ``sampled`` are the step's requests that ran their
        last pending token; a request still in its prompt must not be among them."""
        if len(sampled) != len(next_tokens):
            raise ValueError(f"{len(sampled)} requests but {len(next_tokens)} tokens")
        finished: list[Request] = []
        for req, tok in zip(sampled, next_tokens):
            if req.in_prefill():
                raise ValueError(f"request {req.request_id} is still in its prompt and samples nothing")
            req.output.append(int(tok))
        for req in self.running:
            if req.cache is not None:
                self.cache.release_passed(req.cache)
        for req in sampled:
            if req.is_done():
                self.cache.free(req.cache)
                req.cache = None
                req.status = Status.FINISHED
                finished.append(req)
        self.running = [r for r in self.running if r.status is Status.RUNNING]
        return finished

    def abort(self, req: Request) -> None:
        """Drop a request between steps and give back what it holds."""
        if req.status is Status.FINISHED:
            return
        if req.status is Status.RUNNING:
            self.running.remove(req)
            self.cache.free(req.cache)
            req.cache = None
        else:
            self.waiting.remove(req)
        req.status = Status.FINISHED
