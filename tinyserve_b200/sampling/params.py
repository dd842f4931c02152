"""Per-request sampling options; names and meanings follow upstream
src/tinyserve/sampling.py:37-53."""

from __future__ import annotations

import math
from dataclasses import dataclass

MAX_LOGPROBS = 20


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0      # 0 = greedy (argmax of the raw logits)
    top_p: float = 1.0            # nucleus mass; 1 = the whole vocabulary
    seed: int | None = None       # a request with a seed draws the same tokens whatever its batch
    logprobs: int | None = None   # k: report the drawn token's log-probability and the top k

    def __post_init__(self) -> None:
        if not (math.isfinite(self.temperature) and self.temperature >= 0):
            raise ValueError(f"temperature must be finite and >= 0, got {self.temperature}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.logprobs is not None and not 0 <= self.logprobs <= MAX_LOGPROBS:
            raise ValueError(f"logprobs must be in [0, {MAX_LOGPROBS}], got {self.logprobs}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0
