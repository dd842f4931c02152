"""The reference arm of ``bench.py``: the same metric on the same configuration, run by the UNMODIFIED
upstream engine from ``baseline/_ref`` through its own public API and its stock fast path.

Nothing of ``tinyserve_b200`` is imported here. What runs is upstream's ``Engine`` with everything
its own benchmark switches on (upstream scripts/benchmark.py:81-92, :128-138): the Triton split-K
decode attention, the Triton varlen prefill attention, the fused norm / rotation / cache-write
kernels, chunked prefill and ``DecodeGraphs``. Weights are drawn for upstream's own
``expected_shapes`` with the law this repository's random-weights mode uses (N(0, 0.02); norm
weights 1 + N(0, 0.02)); the batch, prompt length, steps and warm-up are the caller's. Upstream's
engine reads the sampled tokens back to the host in every step, so its device-timed ``value`` and
its end-to-end ``e2e`` are the same run timed twice (CUDA events and the wall clock).
"""

from __future__ import annotations

import importlib
import json
import statistics
import sys
import time
from pathlib import Path
from typing import Any, Callable

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def run(args: Any, cfg_dict: dict[str, Any], full_layers: int, clock_sampler: Callable[[], Any],
        peaks: dict[str, float], peaks_source: str) -> int:
    if not (REF / "tinyserve" / "engine.py").is_file():
        return unavailable("baseline/_ref does not hold the upstream package; run "
                           "python baseline/install_reference.py <upstream checkout>")
    # upstream first on the path, and this repository's package nowhere on it
    sys.path[:] = [str(REF)] + [p for p in sys.path if Path(p or ".").resolve() != HERE.parent]
    for name in list(sys.modules):
        if name == "tinyserve_b200" or name.startswith("tinyserve_b200."):
            return unavailable("this repository's package was imported before the reference arm ran")
    try:
        import torch

        ts = importlib.import_module("tinyserve")
        if Path(ts.__file__).resolve().parent != (REF / "tinyserve").resolve():
            return unavailable(f"'tinyserve' resolved to {ts.__file__}, not to baseline/_ref")
        from tinyserve.config import ModelConfig
        from tinyserve.cuda_graphs import DecodeGraphs
        from tinyserve.engine import Engine
        from tinyserve.kv_cache import KVCache
        from tinyserve.model import Qwen3
        from tinyserve.weights import expected_shapes
    except Exception as exc:  # noqa: BLE001  (any import failure is the answer)
        return unavailable(f"upstream does not import here: {type(exc).__name__}: {exc}")

    if not torch.cuda.is_available():
        return unavailable("no CUDA device here; the reference arm runs upstream's Triton kernels on a GPU")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    dtype = torch.bfloat16
    cfg = ModelConfig.from_dict(cfg_dict)
    gen = torch.Generator(device=dev).manual_seed(0)
    weights: dict[str, torch.Tensor] = {}
    for name, shape in expected_shapes(cfg).items():
        w = torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, 0.02, generator=gen)
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            w += 1.0
        weights[name] = w.to(dtype)
    page = 16
    g = torch.Generator().manual_seed(0)

    def prompts(n: int, length: int) -> list[list[int]]:
        return torch.randint(0, min(cfg.vocab_size, 150_000), (n, length), generator=g).tolist()

    try:
        model = Qwen3(cfg, weights, decode_attention="triton_split", prefill_attention="triton", fused_kernels=True)

        def prefilled(batch: int, steps: int) -> Any:
            margin = -(-batch * args.prompt_len // 2048) + 8
            per_seq = -(-(args.prompt_len + steps + margin) // page) + 1
            blocks = max(batch * per_seq, cfg.max_position_embeddings // page)
            cache = KVCache(cfg, blocks, page, dtype, dev)
            graphs = DecodeGraphs(model, cache, max_batch=batch)
            e = Engine(model, cache, batch, max(2048, batch), decode_graphs=graphs, chunked_prefill=True)
            for p in prompts(batch, args.prompt_len):
                e.add_request(p, max_new_tokens=steps + margin)
            while e.scheduler.waiting or any(len(s.pending()) > 1 for s in e.scheduler.running):
                e.step()
            return e

        def decode(batch: int, warmup: int, steps: int) -> tuple[float, float, float]:
            """ms per step by CUDA events, ms per step by the wall clock, mean context length."""
            e = prefilled(batch, warmup + steps)
            for _ in range(warmup):
                e.step()
            torch.cuda.synchronize()
            ctx = 0
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            for _ in range(steps):
                ctx += sum(s.table.num_tokens + 1 for s in e.scheduler.running)
                e.step()
            end.record()
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) * 1e3 / steps
            return start.elapsed_time(end) / steps, wall, ctx / (steps * batch)

        sampler = clock_sampler()
        sampler.start()
        ms, wall_ms, ctx = decode(args.batch, args.warmup, args.steps)
        clocks = sampler.stop()
        storages = {t.untyped_storage().data_ptr(): t.untyped_storage().nbytes() for t in model.w.values()}
        weight_bytes = sum(storages.values())       # merged matrices and their row views count once
        kv_per_token = 2 * cfg.num_layers * cfg.kv_size * 2
        achieved = (weight_bytes + args.batch * ctx * kv_per_token) / (ms * 1e-3) / 1e9
        width = -(-(args.prompt_len + args.warmup + args.steps) // page)
        result = {
            "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.model.upper()} sizes, bf16, "
                      f"{args.prompt_len:,}-token prompts)",
            "value": round(args.batch * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
            "impl": "reference",
            "config": {
                "model": f"Qwen3-{args.model.upper()} sizes", "layers": cfg.num_layers,
                "layers_of_configuration": full_layers, "hidden": cfg.hidden_size, "q_heads": cfg.num_heads,
                "kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
                "vocab": cfg.vocab_size, "tied_embeddings": cfg.tie_word_embeddings, "global_batch": args.batch,
                "seq_len": args.prompt_len, "context_limit": cfg.max_position_embeddings,
                "mean_context": round(ctx, 1), "page_size": page, "parallelism": "single GPU",
                "path": "upstream Engine.step: triton_split decode, triton prefill, fused kernels, DecodeGraphs",
                "l2": f"inputs larger than L2 (weights {weight_bytes / 1e9:.2f} GB read every step)",
                "peaks": peaks_source,
            },
            "e2e": {"value": round(args.batch * 1e3 / wall_ms, 1), "unit": "tokens/s", "ms_per_step": round(wall_ms, 4),
                    "h2d_bytes_per_step": args.batch * (3 * 8 + 4 + 4 * width), "d2h_bytes_per_step": 8 * args.batch},
            "gpu_launches": None,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks_source},
        }
        if not args.skip_points:
            points = {}
            for b in (1, 64):
                pms, _, _ = decode(b, 3, max(16, args.steps // 4))
                points[f"decode_b{b}"] = round(b * 1e3 / pms, 1)
            result["points"] = points
            t_pre = 2048
            cache = KVCache(cfg, cfg.max_position_embeddings // page, page, dtype, dev)
            times = []
            toks = prompts(1, t_pre)[0]
            for it in range(3 + 5):
                e = Engine(model, cache, 1, t_pre, chunked_prefill=True)
                e.add_request(toks, max_new_tokens=1)
                torch.cuda.synchronize()
                s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s_.record()
                e.step()
                e_.record()
                torch.cuda.synchronize()
                if it >= 3:
                    times.append(s_.elapsed_time(e_))
            pre_ms = statistics.median(times)
            result["prefill"] = {"value": round(t_pre * 1e3 / pre_ms, 1), "tokens": t_pre, "ms": round(pre_ms, 3)}
    except Exception as exc:  # noqa: BLE001  (a compiler or launch failure of upstream's kernels is the answer)
        return unavailable(f"upstream's stock path failed on this GPU: {type(exc).__name__}: {exc}")
    print(json.dumps(result))
    return 0
