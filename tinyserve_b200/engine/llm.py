"""Convenience entry point: from a model folder (or a configuration and a seed) to an engine
with a cache sized for the job.

    llm = LLM.from_folder("path/to/model", dtype="bfloat16")
    outputs = llm.generate([[1, 2, 3]], max_new_tokens=16)
"""

from __future__ import annotations

from pathlib import Path
from typing import Sequence

import torch

from .. import architectures as _architectures  # noqa: F401  (registers the architectures)
from ..cache.manager import CacheManager
from ..config.base import ModelConfig
from ..model import DecoderModel
from ..sampling.params import SamplingParams
from .engine import Engine

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}")
    return _DTYPES[dtype]


class LLM:
    def __init__(self, model: DecoderModel, *, page_size: int = 16, num_pages: int | None = None,
                 kv_fraction: float = 0.85, max_num_seqs: int = 64, max_batch_tokens: int = 2048,
                 chunked_prefill: bool = False, seed: int = 0, trace_steps: bool = False,
                 decode_graphs: bool = True, graph_max_context: int | None = None, run_ahead: bool = True,
                 prefill_graph: bool = True, record_logits: bool = False) -> None:
        """``num_pages``: size of every page pool; by default the pools together take
        ``kv_fraction`` of the device memory that is free once the weights are loaded."""
        self.model = model
        needs = model.cache_needs()
        if num_pages is None:
            elem = torch.empty(0, dtype=model.dtype).element_size()
            per_page = CacheManager.bytes_per_token(needs, elem) * page_size
            if model.device.type == "cuda":
                free, _ = torch.cuda.mem_get_info(model.device)
            else:
                free = 1 << 30
            num_pages = max(1, int(free * kv_fraction) // max(per_page, 1))
            # No request can use more than the model's longest context times the batch.
            most = -(-model.spec.max_position_embeddings // page_size) * max_num_seqs
            num_pages = min(num_pages, most)
        self.cache = CacheManager(needs, page_size=page_size, num_pages=num_pages, max_requests=max_num_seqs,
                                  dtype=model.dtype, device=model.device, max_step_tokens=max_batch_tokens)
        self.engine = Engine(model, self.cache, max_num_seqs=max_num_seqs, max_batch_tokens=max_batch_tokens,
                             chunked_prefill=chunked_prefill, seed=seed, trace_steps=trace_steps,
                             decode_graphs=decode_graphs and model.device.type == "cuda",
                             graph_max_context=graph_max_context, run_ahead=run_ahead, prefill_graph=prefill_graph,
                             record_logits=record_logits)

    @classmethod
    def from_folder(cls, model_dir: str | Path, dtype: str | torch.dtype = "bfloat16", device: str = "cuda",
                    **kwargs) -> "LLM":
        return cls(DecoderModel.from_folder(model_dir, _dtype(dtype), device), **kwargs)

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int = 0, dtype: str | torch.dtype = "bfloat16",
                    device: str = "cuda", **kwargs) -> "LLM":
        """Random weights made on the device from ``config`` and ``seed``."""
        return cls(DecoderModel.from_config(config, seed, _dtype(dtype), device), **kwargs)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 eos_ids: frozenset[int] = frozenset(), sampling: SamplingParams | None = None) -> list[list[int]]:
        return self.engine.generate(prompts, max_new_tokens, eos_ids, sampling)
