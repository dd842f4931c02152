"""One request's state as the scheduler moves it between its queues.

What a request is made of (prompt, output, a limit on new tokens, end tokens, its place in
the cache), the three states and the questions the scheduler asks of it (how many tokens are
pending, is it still in its prompt, is it done) are dictated by upstream's scheduling policy
(src/tinyserve/sequence.py:23-74), which this engine keeps; the record itself, the cache handle
of several page groups and a state slot, and the slice helper are this engine's own.

A request's tokens are its prompt followed by what it has generated. The cache holds the
first ``num_cached`` of them; the rest are pending and go into coming steps: the whole prompt
for a fresh request, one token while decoding, prompt plus output after a preemption (its
cache was given back, so everything is recomputed).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from ..cache.manager import RequestCache
from ..sampling.params import SamplingParams


class Status(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class Request:
    request_id: int
    prompt: list[int]
    max_new_tokens: int
    eos_ids: frozenset[int] = frozenset()
    sampling: SamplingParams = field(default_factory=SamplingParams)
    output: list[int] = field(default_factory=list)
    status: Status = Status.WAITING
    cache: RequestCache | None = None
    num_scheduled: int = 0        # tokens given to the last scheduled step
    num_preemptions: int = 0

    def __post_init__(self) -> None:
        if len(self.prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        if self.max_new_tokens < 1:
            raise ValueError(f"max_new_tokens={self.max_new_tokens}: a request generates at least one token")

    @property
    def tokens(self) -> list[int]:
        return [*self.prompt, *self.output]

    def token_slice(self, start: int, end: int) -> list[int]:
        """``tokens[start:end]`` without building the whole list (a decode step needs one token)."""
        n = len(self.prompt)
        if end <= n:
            return self.prompt[start:end]
        if start >= n:
            return self.output[start - n: end - n]
        return self.prompt[start:] + self.output[: end - n]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def num_cached(self) -> int:
        return 0 if self.cache is None else self.cache.num_tokens

    @property
    def max_cached_tokens(self) -> int:
        """The longest the request's cache can grow: every token except the last one it
        generates, which is handed out and never run."""
        return self.num_tokens - len(self.output) + self.max_new_tokens - 1

    def num_pending(self) -> int:
        return self.num_tokens - self.num_cached

    def in_prefill(self) -> bool:
        """Asked after scheduling: does the request still hold tokens back for later steps? Then
        this step's logits predict a token it already has, and it samples nothing."""
        return self.num_pending() > 0

    def is_done(self) -> bool:
        """The limit is reached, or the newest token is one of the request's end tokens."""
        n = len(self.output)
        return n >= self.max_new_tokens or (n > 0 and self.output[-1] in self.eos_ids)
