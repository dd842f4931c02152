"""Trace replay: feed given token ids through the model step by step and hand back logits.

It samples nothing and schedules nothing; it drives the same model, step function, cache
manager and kernels that generation uses. ``bin/trace_run`` is a thin command line around
``Replayer``. Upstream has no such program; its nearest relatives are the chunk-feeding tests
(tests/test_batched_forward.py:176-199) and ``greedy_generate_paged`` (src/tinyserve/model.py:379-413).
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from ..cache.manager import CacheManager, RequestCache
from ..model import DecoderModel
from ..kernels import ops
from .step import ModelRunner, StepEntry

DEFAULT_PAGE_SIZE = 16


class Replayer:
    def __init__(self, model: DecoderModel, max_tokens: int, page_size: int = DEFAULT_PAGE_SIZE,
                 max_live: int = 64) -> None:
        """``max_tokens``: the most tokens live requests hold at any time, each request's count
        rounded up to a multiple of 64 (so to whole pages, for any page size that divides 64).
        The page pool is made for exactly this many."""
        if 64 % page_size:
            raise ValueError(f"page_size={page_size} must divide 64")
        self.model = model
        num_pages = max(1, -(-max_tokens // page_size))
        self.cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=num_pages,
                                  max_requests=max_live, dtype=model.dtype, device=model.device)
        self.runner = ModelRunner(model, self.cache)
        self.live: dict[str, RequestCache] = {}

    @classmethod
    def from_folder(cls, model_dir: str | Path, dtype: torch.dtype, max_tokens: int,
                    page_size: int = DEFAULT_PAGE_SIZE, device: str = "cuda") -> "Replayer":
        return cls(DecoderModel.from_folder(model_dir, dtype, device), max_tokens, page_size)

    def run_step(self, entries: Sequence[tuple[str, Sequence[int], Sequence[int]]],
                 end: Sequence[str] = ()) -> torch.Tensor | None:
        """``entries``: (request id, its next tokens, wanted places among them). Returns
        float32 logits ``[wanted, vocab]`` in the order of the entries and their places, or
        ``None``. Requests named in ``end`` give back what they hold after the step."""
        step_entries: list[StepEntry] = []
        want: list[Sequence[int]] = []
        vocab = self.model.vocab_size
        for rid, tokens, places in entries:
            if not tokens:
                raise ValueError(f"request {rid!r} brings no tokens")
            if min(tokens) < 0 or max(tokens) >= vocab:
                raise ValueError(f"request {rid!r} has a token id outside 0..{vocab - 1}")
            req = self.live.get(rid)
            if req is None:
                req = self.live[rid] = self.cache.new_request()
            self.cache.append(req, len(tokens))
            step_entries.append(StepEntry(req, list(tokens)))
            want.append(list(places))
        logits = self.runner.step(step_entries, want) if step_entries else None
        if self.model.device.type == "cuda":
            ops.check_device_errors()      # a kernel that gave up on a bounded wait: raise, never hand back its logits
        for req in {id(e.cache): e.cache for e in step_entries}.values():
            self.cache.release_passed(req)
        for rid in end:
            req = self.live.pop(rid, None)
            if req is not None:
                self.cache.free(req)
        return logits
