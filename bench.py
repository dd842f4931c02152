"""Headline benchmark: decode tokens/s at batch 8 (and 1, 64) and prefill tokens/s at 2,048
tokens for the Qwen3-0.6B layer sizes with random weights in bfloat16, on ONE B200; beside it
the two larger configurations: 64 mixed requests through the scheduler at the Qwen3-8B sizes
and decode at batch 1 / 8 / 64 at the Qwen3-32B sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--model 0.6b|8b|32b] [--workload decode|mixed] [--kernels]

Prints ONE JSON line. ``value`` is decoded tokens per second timed on the device with CUDA
events around K decode steps (step function + sampling kernel, no host read-back between
steps); ``e2e`` is the same through the Python entry point (``Engine.step``): host token lists
in, pinned-memory copy of each step's inputs, sampled tokens read back to the host every step.
``prefill`` times one 2,048-token prompt; ``roofline`` relates the decode step to the bytes it
must read (every weight once + the cache of the live requests) and the measured HBM bandwidth.
Before anything is timed, the first replayed decode step of every batch size is compared with the
same step launched kernel by kernel (``checked``). ``points`` adds decode at batch 1 and 64, the
mixed workload at the 8B sizes (``mixed_8b``: output tokens per second of 64 requests with prompt
lengths U[16, 2,048], 128 tokens each, chunked prefill 512, through ``Engine.add_request`` /
``Engine.step``) and decode at the 32B sizes (``decode_32b_b1/8/64``: 2,048-token prompts, all 64
layers, pages sized to the memory that is left); ``large`` says more about those runs.
``--kernels`` adds a table of the decode step's kernel classes (ms, GB/s, share of the measured
peak) timed with CUDA events inside a step launched kernel by kernel.
This engine serves one GPU: for ``--gpus`` above 1 it says so and exits with 2.
"""

from __future__ import annotations

import argparse
import gc
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# The headline configuration: the Qwen3-0.6B layer sizes.
QWEN3_0_6B = {
    "architectures": ["Qwen3ForCausalLM"], "vocab_size": 151936, "hidden_size": 1024,
    "intermediate_size": 3072, "num_hidden_layers": 28, "num_attention_heads": 16,
    "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
    "max_position_embeddings": 4096, "tie_word_embeddings": True, "hidden_act": "silu",
}
# Two larger configurations: the Qwen3-8B and Qwen3-32B layer sizes (untied heads).
QWEN3_8B = {**QWEN3_0_6B, "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 36,
            "num_attention_heads": 32, "num_key_value_heads": 8, "tie_word_embeddings": False}
QWEN3_32B = {**QWEN3_0_6B, "hidden_size": 5120, "intermediate_size": 25600, "num_hidden_layers": 64,
             "num_attention_heads": 64, "num_key_value_heads": 8, "tie_word_embeddings": False}
MODELS = {"0.6b": QWEN3_0_6B, "8b": QWEN3_8B, "32b": QWEN3_32B}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PAGE = 16
CHECK_REL = 2e-2          # replayed against eager logits: rounding, as a share of the logits' size


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            d = json.loads(path.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}, "measured"
        except (ValueError, KeyError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.rows: list[list[str]] = []
        self._proc: subprocess.Popen | None = None
        self._thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                           "--format=csv,noheader,nounits", "-lms", "100"],
                                          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self) -> None:
        assert self._proc is not None and self._proc.stdout is not None
        for line in self._proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        rows = [r for r in self.rows if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower() == "active" for r in rows)]
        return {"sm_mhz": int(statistics.median(int(r[0]) for r in rows)), "sm_max_mhz": int(rows[0][1]),
                "reasons": reasons, "samples": len(rows)}


def reference_arm(args: argparse.Namespace) -> int:
    """The same metric by the unmodified upstream engine (``baseline/reference_arm.py``); nothing of
    this repository's package is imported on that path."""
    sys.path.insert(0, str(ROOT / "baseline"))
    import reference_arm as arm

    cfg_dict = dict(MODELS[args.model])
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    pk, pk_src = peaks()
    args.warmup = max(args.warmup, 3)
    return arm.run(args, cfg_dict, full_layers, ClockSampler, pk, pk_src)


def percentile(values: list[float], p: float) -> float:
    xs = sorted(values)
    rank = (len(xs) - 1) * p / 100
    lo = int(rank)
    hi = min(lo + 1, len(xs) - 1)
    return xs[lo] + (xs[hi] - xs[lo]) * (rank - lo)


class Bench:
    """One model on the device and the measurements that can be made of it."""

    def __init__(self, name: str, layers: int | None, graphs: bool = True) -> None:
        import torch

        from tinyserve_b200.config import config_from_dict
        from tinyserve_b200.model import DecoderModel

        self.torch = torch
        self.name = name
        cfg_dict = dict(MODELS[name])
        self.full_layers = cfg_dict["num_hidden_layers"]
        if layers:
            cfg_dict["num_hidden_layers"] = layers
        self.cfg = config_from_dict(cfg_dict)
        self.dev = torch.device("cuda:0")
        torch.cuda.set_device(self.dev)
        self.model = DecoderModel.from_config(self.cfg, seed=0, dtype=torch.bfloat16, device=self.dev)
        self.graphs = graphs
        self.gen = torch.Generator().manual_seed(0)
        self.check_rel = 0.0          # worst replayed-against-eager difference seen by the checks
        self.checks = 0

    def close(self) -> None:
        self.model = None
        gc.collect()
        self.torch.cuda.empty_cache()

    # ---------------------------------------------------------------- pieces
    def prompts(self, lengths: list[int]) -> list[list[int]]:
        high = min(self.cfg.vocab_size, 150_000)
        return [self.torch.randint(0, high, (n,), generator=self.gen).tolist() for n in lengths]

    def kv_bytes_per_token(self) -> int:
        from tinyserve_b200.cache import CacheManager

        return CacheManager.bytes_per_token(self.model.cache_needs(), 2)

    def pages_that_fit(self, fraction: float = 0.85) -> int:
        """Pages for the memory that is left once the weights are on the device."""
        free, _ = self.torch.cuda.mem_get_info(self.dev)
        return int(free * fraction) // (self.kv_bytes_per_token() * PAGE)

    def new_cache(self, pages: int, max_requests: int):
        from tinyserve_b200.cache import CacheManager

        return CacheManager(self.model.cache_needs(), page_size=PAGE, num_pages=pages, max_requests=max_requests,
                            dtype=self.torch.bfloat16, device=self.dev)

    def new_engine(self, batch: int, tokens_per_seq: int, cache=None, budget: int = 2048, run_ahead: bool = True):
        from tinyserve_b200.engine import Engine
        from tinyserve_b200.engine.step import ModelRunner

        if cache is None:
            pages = max(batch * (-(-tokens_per_seq // PAGE) + 1), self.cfg.max_position_embeddings // PAGE)
            cache = self.new_cache(pages, batch)
        return Engine(self.model, cache, max_num_seqs=batch, max_batch_tokens=max(budget, batch), chunked_prefill=True,
                      decode_graphs=self.graphs, graph_max_context=self.cfg.max_position_embeddings,
                      runner=ModelRunner(self.model, cache), run_ahead=run_ahead)

    def decode_bytes(self, batch: int, ctx: float) -> float:
        return self.model.weight_bytes() + batch * ctx * self.kv_bytes_per_token()

    def prefilled(self, batch: int, prompt_len: int, steps: int, cache=None, run_ahead: bool = True):
        """An engine whose ``batch`` requests have their prompts in the cache. ``run_ahead`` False for
        callers that step the runner themselves afterwards (no step is then left unread)."""
        # While later prompts are still being prefilled, earlier requests already decode.
        margin = -(-batch * prompt_len // 2048) + 8
        e = self.new_engine(batch, prompt_len + steps + margin, cache, run_ahead=run_ahead)
        for p in self.prompts([prompt_len] * batch):
            e.add_request(p, max_new_tokens=steps + margin)
        while any(r.num_pending() > 1 or r.cache is None for r in e.requests.values()):
            e.step()
        return e

    def check_replay(self, e, reqs) -> None:
        """The next decode step replayed from its recording against the same step launched kernel by
        kernel (it rewrites the same cache rows, so running it twice harms nothing)."""
        from tinyserve_b200.engine.step import StepEntry
        from tinyserve_b200.kernels import ops

        runner = e.runner
        entries = []
        for r in reqs:
            e.cache.append(r.cache, 1)
            entries.append(StepEntry(r.cache, [r.output[-1]]))
        if not runner.replays(entries):
            return
        got = runner.step(entries).float().clone()
        saved, runner.graphs = runner.graphs, {}
        try:
            eager = runner.step(entries).float().clone()
        finally:
            runner.graphs = saved
        ops.check_device_errors()
        rel = float((got - eager).pow(2).mean().sqrt() / eager.pow(2).mean().sqrt())
        self.check_rel = max(self.check_rel, rel if rel == rel else float("inf"))
        self.checks += 1

    def device_decode(self, batch: int, prompt_len: int, warmup: int, steps: int, cache=None, check: bool = True):
        """K decode steps timed on the device: step function + sampling kernel, tokens stay on
        the device. Returns (ms per step, mean context length, kernels launched)."""
        from tinyserve_b200.engine.step import StepEntry
        from tinyserve_b200.kernels import ops

        torch = self.torch
        e = self.prefilled(batch, prompt_len, warmup + steps + 1, cache, run_ahead=False)
        reqs = list(e.requests.values())
        if check and self.graphs:
            self.check_replay(e, reqs)
        out = torch.empty(batch, dtype=torch.int32, device=self.dev)
        ctx_sum = 0

        def one() -> None:
            nonlocal ctx_sum
            entries = []
            for r in reqs:
                e.cache.append(r.cache, 1)
                entries.append(StepEntry(r.cache, [r.output[-1]]))
                ctx_sum += r.cache.num_tokens
            ops.sample(e.runner.step(entries), out)

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        ctx_sum = 0
        before = ops.launch_count
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            one()
        end.record()
        torch.cuda.synchronize()
        ops.check_device_errors()
        for r in reqs:
            e.cache.free(r.cache)
        return start.elapsed_time(end) / steps, ctx_sum / (steps * batch), ops.launch_count - before

    def e2e_decode(self, batch: int, prompt_len: int, warmup: int, steps: int):
        torch = self.torch
        e = self.prefilled(batch, prompt_len, warmup + steps)
        for _ in range(warmup):
            e.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            e.step()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3 / steps
        # per step: the packed int32 inputs (token, position, slot, lengths, block table) and the
        # status word with the tokens back
        width = -(-(prompt_len + warmup + steps) // PAGE)
        return ms, 4 * (batch * (8 + width) + 16), 4 * (batch + 1)

    def prefill(self, tokens: int = 2048) -> tuple[float, float]:
        """One prompt of ``tokens`` tokens in one step: (ms, flops of the step)."""
        from tinyserve_b200.engine.step import StepEntry
        from tinyserve_b200.kernels import ops

        torch, cfg = self.torch, self.cfg
        e = self.new_engine(1, tokens + 8)
        toks = self.prompts([tokens])[0]
        times = []
        for it in range(3 + 5):
            req = e.cache.new_request()
            e.cache.append(req, tokens)
            torch.cuda.synchronize()
            s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_.record()
            e.runner.step([StepEntry(req, toks)])
            e_.record()
            torch.cuda.synchronize()
            e.cache.free(req)
            if it >= 3:
                times.append(s_.elapsed_time(e_))
        ops.check_device_errors()
        table = cfg.vocab_size * cfg.hidden_size
        matmul_params = self.model.weight_bytes() // 2 - table * (1 if cfg.tie_word_embeddings else 2)
        flops = 2.0 * tokens * matmul_params + 2.0 * table                                 # the head on one row
        flops += cfg.num_layers * 4.0 * cfg.num_heads * cfg.head_dim * (tokens * (tokens + 1) / 2)
        return statistics.median(times), flops

    def mixed(self, num_requests: int = 64, out_tokens: int = 128, chunk: int = 512) -> dict:
        """The closed loop of upstream src/tinyserve/bench.py:101-117 with everybody in flight at
        once: ``num_requests`` requests with prompt lengths U[16, 2,048] (seeded), ``out_tokens``
        greedy tokens each, chunked prefill ``chunk``, through ``Engine.add_request`` / ``step``."""
        from tinyserve_b200.kernels import ops

        torch = self.torch
        g = torch.Generator().manual_seed(1)
        lengths = torch.randint(16, 2049, (num_requests,), generator=g).tolist()
        need = sum(-(-(n + out_tokens) // PAGE) + 1 for n in lengths)
        pages = min(self.pages_that_fit(), max(need, self.cfg.max_position_embeddings // PAGE))
        cache = self.new_cache(pages, num_requests)
        e = self.new_engine(num_requests, 0, cache, budget=chunk)
        for p in self.prompts([40, 700]):              # warm-up, not reported (upstream scripts/benchmark.py:140)
            e.add_request(p, 4)
        while e.has_work():
            e.step()
        torch.cuda.synchronize()
        steps0, ahead0, graph0 = e.num_steps, e.num_steps_ahead, e.runner.num_graph_steps
        prompts = self.prompts(lengths)
        start = e.clock()
        ids = [e.add_request(p, out_tokens) for p in prompts]
        while e.has_work():
            e.step()
        torch.cuda.synchronize()
        seconds = e.clock() - start
        ops.check_device_errors()
        times = [e.times[i] for i in ids]
        outs = sum(len(e.requests[i].output) for i in ids)
        return {
            "value": round(outs / seconds, 1), "unit": "output tokens/s", "requests": num_requests,
            "prompt_tokens": sum(lengths), "output_tokens": outs, "seconds": round(seconds, 3),
            "chunked_prefill": chunk, "steps": e.num_steps - steps0, "steps_replayed": e.runner.num_graph_steps - graph0,
            "steps_ahead": e.num_steps_ahead - ahead0, "preemptions": e.scheduler.num_preemptions,
            "ttft_p50_ms": round(percentile([t.ttft * 1e3 for t in times], 50), 2),
            "ttft_p99_ms": round(percentile([t.ttft * 1e3 for t in times], 99), 2),
            "tpot_p50_ms": round(percentile([t.tpot * 1e3 for t in times if t.tpot is not None], 50), 3),
            "kv_util_max": round(max(e.kv_utilization), 3), "pages": pages, "layers": self.cfg.num_layers,
            "layers_of_configuration": self.full_layers,
        }

    def kernel_table(self, batch: int, prompt_len: int, pk: dict, prefill_tokens: int = 0) -> dict:
        """Where a step's device time goes, by kernel class: the step is launched kernel by
        kernel with a pair of CUDA events around every call of ``ops`` (no recording, no launch
        overlap; the step is queued behind a spin kernel so that the host's launch time is not in
        it), and the median of three steps is summed per class. ``gb_s`` relates the bytes a call
        must move (its weights, its rows, the cache of the live requests), from its arguments, to
        its time; ``tflops`` its multiply-adds (products and attention). The step is a decode step
        of ``batch`` requests, or, with ``prefill_tokens``, one prompt of that many tokens."""
        from tinyserve_b200.engine.step import StepEntry
        from tinyserve_b200.kernels import ops

        torch = self.torch
        saved_graphs, self.graphs = self.graphs, False
        if prefill_tokens:
            e = self.new_engine(1, prefill_tokens + 8, run_ahead=False)
            prompt = self.prompts([prefill_tokens])[0]
            reqs = []
        else:
            e = self.prefilled(batch, prompt_len, 16, run_ahead=False)
            reqs = list(e.requests.values())
        self.graphs = saved_graphs
        e.runner.tune_launch_overlap = False
        ops.set_programmatic_launch(0)
        records: list[tuple[str, object, object, float, float]] = []

        def flops(name: str, a: tuple) -> float:
            if name == "gemm":
                return 2.0 * a[0].shape[0] * a[1].shape[0] * a[1].shape[1]
            if name == "gemm_swiglu":
                return 2.0 * a[0].shape[0] * a[1].shape[0] * a[1].shape[1]
            if name == "gemm_to_stream":
                return 2.0 * a[0].shape[0] * a[1].shape[0] * a[1].shape[1]
            if name == "gemm_normed":
                return 2.0 * a[0].shape[0] * a[4].shape[0] * a[4].shape[1]
            if name in ("paged_attention", "decode_attention_fused"):
                ctx = a[5] if name == "paged_attention" else a[11]
                heads, d = (a[0].shape[1], a[0].shape[2]) if name == "paged_attention" else (a[14], a[7].shape[3])
                pairs = sum(n * (c - n) + n * (n + 1) / 2 for n, c in zip(ctx.query_lens, ctx.context_lens))
                return 4.0 * heads * d * pairs
            return 0.0

        def nbytes(*ts) -> float:
            return float(sum(t.numel() * t.element_size() for t in ts if isinstance(t, torch.Tensor)))

        def work(name: str, a: tuple) -> float:
            if name in ("gemm", "gemm_swiglu"):
                return nbytes(a[0], a[1], a[2])
            if name == "qk_norm_rope_write":      # the rows it reads and writes, not the cache tensors
                return 2.0 * nbytes(a[0])
            if name == "embed":                   # the rows it gathers, not the table
                return nbytes(a[0], a[2]) + a[0].numel() * a[1].shape[1] * a[1].element_size()
            if name == "gemm_to_stream":
                return nbytes(a[0], a[1], a[2], a[2])
            if name == "gemm_normed":
                return nbytes(a[0], a[4], a[5])
            if name in ("paged_attention", "decode_attention_fused"):
                kc = a[1] if name == "paged_attention" else a[7]
                ctx = a[5] if name == "paged_attention" else a[11]
                return float(sum(ctx.context_lens)) * 2.0 * kc.shape[1] * kc.shape[3] * kc.element_size()
            return nbytes(*a)

        names = ["embed", "add_rms_norm", "rope_tables", "silu_mul", "qk_norm_rope_write", "paged_attention",
                 "decode_attention_fused", "gemm", "gemm_swiglu", "gemm_to_stream", "gemm_normed", "sample"]
        originals = {n: getattr(ops, n) for n in names}
        depth = [0]

        def wrap(name: str):
            fn = originals[name]

            def timed(*a, **k):
                if depth[0]:                      # a product inside gemm_swiglu's fallback: counted with its caller
                    return fn(*a, **k)
                s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s_.record()
                depth[0] += 1
                try:
                    r = fn(*a, **k)
                finally:
                    depth[0] -= 1
                e_.record()
                records.append((name, s_, e_, work(name, a), flops(name, a)))
                return r
            return timed

        for n in names:
            setattr(ops, n, wrap(n))
        out = torch.empty(batch, dtype=torch.int32, device=self.dev)
        rounds: list[dict[str, list[float]]] = []
        try:
            for it in range(5):
                records.clear()
                entries = []
                if prefill_tokens:
                    req = e.cache.new_request()
                    e.cache.append(req, prefill_tokens)
                    entries.append(StepEntry(req, prompt))
                for r in reqs:
                    e.cache.append(r.cache, 1)
                    entries.append(StepEntry(r.cache, [r.output[-1]]))
                # the device idles behind a spin kernel while the host queues the whole step, so that
                # the kernels then run back to back and an event pair brackets device time only
                torch.cuda._sleep(40_000_000 if not prefill_tokens else 100_000_000)
                ops.sample(e.runner.step(entries), out[: len(entries)])
                torch.cuda.synchronize()
                if prefill_tokens:
                    e.cache.free(req)
                if it >= 2:
                    acc: dict[str, list[float]] = {}
                    for name, s_, e_, by, fl in records:
                        a = acc.setdefault(name, [0.0, 0.0, 0.0, 0.0])
                        a[0] += s_.elapsed_time(e_)
                        a[1] += by
                        a[2] += 1
                        a[3] += fl
                    rounds.append(acc)
        finally:
            for n in names:
                setattr(ops, n, originals[n])
            ops.set_programmatic_launch(ops.DEFAULT_PDL_MASK)
        table = {}
        for name in rounds[0]:
            ms = statistics.median(r[name][0] for r in rounds)
            _, by, calls, fl = rounds[0][name]
            table[name] = {"calls": int(calls), "ms": round(ms, 4), "gb_s": round(by / (ms * 1e-3) / 1e9, 1),
                           "hbm_frac": round(by / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 3)}
            if fl:
                table[name]["tflops"] = round(fl / (ms * 1e-3) / 1e12, 1)
                table[name]["tensor_frac"] = round(fl / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 3)
        return table


def gemm_table() -> int:
    """The tcgen05 product of this engine against the vendor library's at the four layer shapes of the
    three model sizes, 512 and 2,048 rows, kernel by kernel with CUDA events (20 launches after 3)."""
    import torch

    from tinyserve_b200.kernels import ops

    dev, bf = torch.device("cuda:0"), torch.bfloat16

    def timed(fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record()
        for _ in range(20):
            fn()
        e_.record()
        torch.cuda.synchronize()
        return s_.elapsed_time(e_) / 20 * 1e3

    print(f"{'rows':>5} {'shape':<14} {'N':>6} {'K':>6} {'library us':>10} {'TFLOP/s':>8} {'tcgen05 us':>10} {'TFLOP/s':>8} "
          f"{'by pairs us':>11} {'TFLOP/s':>8}")
    for m in (512, 2048, 8192):
        for name, d in MODELS.items():
            h, inter = d["hidden_size"], d["intermediate_size"]
            q, kv = d["num_attention_heads"] * d["head_dim"], d["num_key_value_heads"] * d["head_dim"]
            for what, n, k in (("qkv", q + 2 * kv, h), ("o", h, q), ("gate_up", 2 * inter, h), ("down", h, inter)):
                w = (torch.randn(n, k, device=dev) * 0.02).to(bf)
                x = torch.randn(m, k, device=dev).to(bf)
                out = torch.empty(m, n, device=dev, dtype=bf)
                lib = timed(lambda: torch.mm(x, w.t(), out=out))
                own = timed(lambda: ops.gemm_tcgen05(x, w, out, 256))
                pair = timed(lambda: ops.gemm_tcgen05(x, w, out, ops.TCGEN05_PAIR_TILE))
                fl = 2.0 * m * n * k
                print(f"{m:>5} {name + ' ' + what:<14} {n:>6} {k:>6} {lib:>10.1f} {fl / lib / 1e6:>8.0f} {own:>10.1f} {fl / own / 1e6:>8.0f} "
                      f"{pair:>11.1f} {fl / pair / 1e6:>8.0f}")
                del w, x, out
    ops.check_device_errors()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=sorted(MODELS), default="0.6b",
                    help="layer sizes of the headline run: 0.6b (the headline configuration) or one of the larger ones")
    ap.add_argument("--workload", choices=["decode", "mixed"], default="decode",
                    help="decode: uniform batches that were prefilled first (the headline); mixed: the closed loop of "
                         "64 requests through the scheduler, alone")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--kernels", action="store_true", help="add the per-kernel-class table of the decode step")
    ap.add_argument("--profile", choices=["decode", "prefill", "timeline", "gemm"], default=None,
                    help="decode / prefill: run a small case kernel by kernel between cudaProfilerStart/Stop and exit "
                         "(for ncu --profile-from-start off); timeline: when every kernel of a recorded decode step "
                         "started (needs the timeline build); gemm: this engine's tcgen05 product against the "
                         "library's at the layer shapes of the three model sizes; combine with --layers, --batch")
    ap.add_argument("--skip-points", action="store_true",
                    help="skip the batch 1 / 64 points, the prefill and the larger models")
    ap.add_argument("--skip-large", action="store_true", help="skip the points of the 8B and 32B sizes")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU only; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch

    from tinyserve_b200.engine.step import StepEntry
    from tinyserve_b200.kernels import ops

    pk, pk_src = peaks()
    if args.profile == "gemm":
        return gemm_table()
    b = Bench(args.model, args.layers, graphs=not args.no_graphs)
    cfg, dev = b.cfg, b.dev

    if args.workload == "mixed":
        result = b.mixed()
        print(json.dumps({"metric": f"output tok/s, 64 mixed requests through the scheduler (Qwen3-{args.model.upper()} "
                                    f"sizes, bf16)", **result, "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
                          "impl": "ours", "data": "synthetic token ids, random-init weights"}))
        return 0
    if args.profile == "timeline":
        # When each kernel of one recorded decode step started and when its wait for the kernels
        # before it returned, from the device clock. Needs the library built with the notes in
        # (TINYSERVE_B200_TIMELINE=1 in the environment); no JSON line, no timing claim.
        if not ops.build.TIMELINE:
            print("--profile timeline needs TINYSERVE_B200_TIMELINE=1 in the environment")
            return 2
        e = b.prefilled(args.batch, args.prompt_len, 16, run_ahead=False)
        reqs = list(e.requests.values())
        out = torch.empty(args.batch, dtype=torch.int32, device=dev)
        for it in range(12):
            if it == 11:
                ops.timeline()
            entries = []
            for r in reqs:
                e.cache.append(r.cache, 1)
                entries.append(StepEntry(r.cache, [r.output[-1]]))
            ops.sample(e.runner.step(entries), out)
        records = ops.timeline()
        t0 = records[0]["start"]
        print(f"one decode step, batch {args.batch}, layers {cfg.num_layers}: us from the first kernel's start")
        print(f"{'#':>4} {'class':<12} {'grid':<12} {'block':>5} {'started':>9} {'wait over':>9} {'to next wait':>12}")
        for i, r in enumerate(records):
            w = r["waited"] or r["start"]
            nxt = (records[i + 1]["waited"] or records[i + 1]["start"]) if i + 1 < len(records) else w
            print(f"{i:>4} {r['class']:<12} {str(r['grid']):<12} {r['block']:>5} {(r['start'] - t0) / 1e3:>9.2f} "
                  f"{(w - t0) / 1e3:>9.2f} {(nxt - w) / 1e3:>12.2f}")
        return 0
    if args.profile:
        # A small, eager case for a profiler: nothing is timed and no JSON line is printed.
        b.graphs = False
        if args.profile == "decode":
            e = b.prefilled(args.batch, args.prompt_len, 8)
            for _ in range(2):
                e.step()
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            for _ in range(2):
                e.step()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        else:
            e = b.new_engine(1, 2048 + 8)
            toks = b.prompts([2048])[0]
            for it in range(3):
                req = e.cache.new_request()
                e.cache.append(req, 2048)
                if it == 2:
                    torch.cuda.profiler.start()
                e.runner.step([StepEntry(req, toks)])
                torch.cuda.synchronize()
                e.cache.free(req)
            torch.cuda.profiler.stop()
        print(f"profiled {args.profile}: batch {args.batch}, layers {cfg.num_layers}")
        return 0

    sampler = ClockSampler()
    sampler.start()
    ms, ctx, launches = b.device_decode(args.batch, args.prompt_len, args.warmup, args.steps)
    clocks = sampler.stop()
    value = args.batch * 1e3 / ms
    e2e_ms, h2d, d2h = b.e2e_decode(args.batch, args.prompt_len, args.warmup, args.steps)
    achieved = b.decode_bytes(args.batch, ctx) / (ms * 1e-3) / 1e9

    result = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.model.upper()} sizes, bf16, "
                  f"{args.prompt_len:,}-token prompts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights", "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.model.upper()} sizes", "layers": cfg.num_layers, "layers_of_configuration": b.full_layers,
            "hidden": cfg.hidden_size, "q_heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "tied_embeddings": cfg.tie_word_embeddings, "global_batch": args.batch, "seq_len": args.prompt_len,
            "context_limit": cfg.max_position_embeddings, "mean_context": round(ctx, 1), "page_size": PAGE,
            "parallelism": "single GPU",
            "l2": f"inputs larger than L2 (weights {b.model.weight_bytes() / 1e9:.2f} GB read every step)",
            "peaks": pk_src,
        },
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_src},
    }
    if args.kernels:
        result["kernels"] = b.kernel_table(args.batch, args.prompt_len, pk)
        b.graphs = False
        eager_ms, _, _ = b.device_decode(args.batch, args.prompt_len, 3, max(16, args.steps // 4), check=False)
        b.graphs = not args.no_graphs
        result["step_ms"] = {"recorded": round(ms, 4), "kernel_by_kernel": round(eager_ms, 4),
                             "sum_of_kernel_classes": round(sum(r["ms"] for r in result["kernels"].values()), 4)}
        result["prefill_kernels"] = b.kernel_table(1, 0, pk, prefill_tokens=2048)
        for title, table in ((f"decode step, batch {args.batch}", result["kernels"]),
                             ("one prompt of 2,048 tokens", result["prefill_kernels"])):
            width = max(len(n) for n in table)
            print(f"{title}\n{'kernel class':<{width}} {'calls':>5} {'ms':>8} {'GB/s':>8} {'of HBM peak':>11} {'TFLOP/s':>8} "
                  f"{'of bf16 peak':>12}", file=sys.stderr)
            for name, r in sorted(table.items(), key=lambda kv: -kv[1]["ms"]):
                print(f"{name:<{width}} {r['calls']:>5} {r['ms']:>8.4f} {r['gb_s']:>8.1f} {r['hbm_frac']:>11.1%} "
                      f"{r.get('tflops', 0):>8.1f} {r.get('tensor_frac', 0):>12.1%}", file=sys.stderr)
    check_rel, checks = b.check_rel, b.checks
    if not args.skip_points:
        points: dict[str, float] = {}
        roofs: dict[str, float] = {}
        for n in (1, 64):
            pms, pctx, _ = b.device_decode(n, args.prompt_len, 3, max(16, args.steps // 4))
            points[f"decode_b{n}"] = round(n * 1e3 / pms, 1)
            roofs[f"decode_b{n}"] = round(b.decode_bytes(n, pctx) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        result["points"] = points
        result["points_hbm_frac"] = roofs
        pre_ms, flops = b.prefill(2048)
        result["prefill"] = {"value": round(2048 * 1e3 / pre_ms, 1), "tokens": 2048, "ms": round(pre_ms, 3),
                             "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk_src}
        check_rel, checks = b.check_rel, b.checks
        if not args.skip_large and args.model == "0.6b" and not args.layers:
            b.close()
            large: dict[str, dict] = {}
            # ---- 64 mixed requests through the scheduler at the Qwen3-8B sizes
            big = Bench("8b", None, graphs=not args.no_graphs)
            large["mixed_8b"] = big.mixed()
            points["mixed_8b"] = large["mixed_8b"]["value"]
            big.close()
            # ---- decode at the Qwen3-32B sizes, all layers, pages sized to the memory that is left
            big = Bench("32b", None, graphs=not args.no_graphs)
            want_pages = 64 * (-(-(2048 + 128 + 80) // PAGE) + 1)
            pages = min(big.pages_that_fit(), want_pages)
            cache = big.new_cache(pages, 64)
            info = {"layers": big.cfg.num_layers, "layers_of_configuration": big.full_layers, "prompt_len": 2048,
                    "pages": pages, "weights_gb": round(big.model.weight_bytes() / 1e9, 1),
                    "cache_gb": round(cache.memory_bytes() / 1e9, 1)}
            for n in (1, 8, 64):
                pms, pctx, _ = big.device_decode(n, 2048, 3, 32 if n < 64 else 24, cache=cache)
                points[f"decode_32b_b{n}"] = round(n * 1e3 / pms, 1)
                info[f"b{n}"] = {"ms_per_step": round(pms, 3), "mean_context": round(pctx, 1),
                                 "hbm_frac": round(big.decode_bytes(n, pctx) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}
            large["decode_32b"] = info
            check_rel, checks = max(check_rel, big.check_rel), checks + big.checks
            big.close()
            result["large"] = large
    result["checked"] = checks > 0 and check_rel <= CHECK_REL
    result["check"] = {"replayed_vs_eager_rel": float(f"{check_rel:.3g}"), "steps_compared": checks, "tolerance": CHECK_REL}
    if not result["checked"] and not args.no_graphs:
        print(f"bench.py: replayed and eager logits differ by {check_rel:.3g} of their size (tolerance {CHECK_REL})",
              file=sys.stderr)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
