"""Per-request sampling options.

The option names, their defaults and their legal ranges are upstream's schema
(src/tinyserve/sampling.py:37-53: ``temperature`` 0 = greedy, ``top_p`` in (0, 1], an optional
``seed``, ``logprobs`` up to 20), so that a caller of upstream's engine can pass the same
arguments here. How the options are used is this engine's own (``sampling/sampler.py``,
``csrc/sampling.cu``).
"""

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
        problems = []
        if not math.isfinite(self.temperature) or self.temperature < 0:
            problems.append(f"temperature={self.temperature!r} (a finite number, 0 or more)")
        if not (self.top_p > 0 and self.top_p <= 1):
            problems.append(f"top_p={self.top_p!r} (above 0, at most 1)")
        if self.logprobs is not None and self.logprobs not in range(MAX_LOGPROBS + 1):
            problems.append(f"logprobs={self.logprobs!r} (None or 0..{MAX_LOGPROBS})")
        if self.seed is not None and not isinstance(self.seed, int):
            problems.append(f"seed={self.seed!r} (None or an integer)")
        if problems:
            raise ValueError("sampling options out of range: " + "; ".join(problems))

    @property
    def greedy(self) -> bool:
        return self.temperature == 0
