"""Headline benchmark: decode tokens/s at batch 8 (and 1, 64) and prefill tokens/s at 2,048
tokens for the Qwen3-0.6B layer sizes with random weights in bfloat16, on ONE B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line. ``value`` is decoded tokens per second timed on the device with CUDA
events around K decode steps (step function + sampling kernel, no host read-back between
steps); ``e2e`` is the same through the Python entry point (``Engine.step``): host token lists
in, pinned-memory copy of each step's inputs, sampled tokens read back to the host every step.
``prefill`` times one 2,048-token prompt; ``roofline`` relates the decode step to the bytes it
must read (every weight once + the cache of the live requests) and the measured HBM bandwidth.
This engine serves one GPU: for ``--gpus`` above 1 it says so and exits with 2.
"""

from __future__ import annotations

import argparse
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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=sorted(MODELS), default="0.6b",
                    help="layer sizes: the headline configuration (0.6b) or the two larger ones")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--pdl", type=int, default=None,
                    help="mask of kernel classes launched with programmatic dependent launch (default: the engine's)")
    ap.add_argument("--no-pdl", action="store_true", help="no programmatic dependent launch between kernels")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--fused-decode-rows", type=int, default=None,
                    help="largest decode batch that takes the fused norm+rotation+attention kernel (0: never)")
    ap.add_argument("--max-splits", type=int, default=None, help="most key ranges per request in decode attention")
    ap.add_argument("--no-cluster-merge", action="store_true",
                    help="decode attention merges its key ranges through global memory, not inside a cluster")
    ap.add_argument("--separate-norms", action="store_true",
                    help="decode steps run every RMSNorm as a kernel of its own (default: folded into the products "
                         "around it for up to 8 rows)")
    ap.add_argument("--profile", choices=["decode", "prefill", "timeline"], default=None,
                    help="run a small case kernel by kernel between cudaProfilerStart/Stop and exit "
                         "(for ncu --profile-from-start off); combine with --layers, --batch")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU only; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch

    from tinyserve_b200 import LLM
    from tinyserve_b200.cache import CacheManager
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.engine import Engine
    from tinyserve_b200.engine.step import ModelRunner, StepEntry
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    if args.separate_norms:
        ops.FUSE_STREAM_NORM = False
    if args.max_splits is not None:
        ops.MAX_SPLITS = args.max_splits
    if args.no_cluster_merge:
        ops.set_decode_cluster_merge(False)
    if args.fused_decode_rows is not None:
        ops.FUSED_DECODE_MAX_ROWS = args.fused_decode_rows
    fixed_pdl = args.no_pdl or args.pdl is not None
    if fixed_pdl:
        ops.set_programmatic_launch(0 if args.no_pdl else args.pdl)
    cfg_dict = dict(MODELS[args.model])
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = config_from_dict(cfg_dict)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    model = DecoderModel.from_config(cfg, seed=0, dtype=torch.bfloat16, device=dev)
    pk, pk_src = peaks()
    page = 16
    vocab = cfg.vocab_size
    g = torch.Generator().manual_seed(0)

    def prompts(n: int, length: int) -> list[list[int]]:
        return torch.randint(0, min(vocab, 150_000), (n, length), generator=g).tolist()

    def new_engine(batch: int, tokens_per_seq: int) -> Engine:
        pages = max(batch * (-(-tokens_per_seq // page) + 1), cfg.max_position_embeddings // page)
        cache = CacheManager(model.cache_needs(), page_size=page, num_pages=pages, max_requests=batch,
                             dtype=torch.bfloat16, device=dev)
        runner = ModelRunner(model, cache)
        runner.tune_launch_overlap = not fixed_pdl
        return Engine(model, cache, max_num_seqs=batch, max_batch_tokens=max(2048, batch), chunked_prefill=True,
                      decode_graphs=not args.no_graphs, graph_max_context=cfg.max_position_embeddings, runner=runner)

    def decode_bytes(batch: int, ctx: float) -> float:
        kv = CacheManager.bytes_per_token(model.cache_needs(), 2)
        return model.weight_bytes() + batch * ctx * kv

    def prefilled(batch: int, steps: int) -> Engine:
        # While later prompts are still being prefilled, earlier requests already decode.
        margin = -(-batch * args.prompt_len // 2048) + 8
        e = new_engine(batch, args.prompt_len + steps + margin)
        for p in prompts(batch, args.prompt_len):
            e.add_request(p, max_new_tokens=steps + margin)
        while any(r.num_pending() > 1 or r.cache is None for r in e.requests.values()):
            e.step()
        return e

    def device_decode(batch: int, warmup: int, steps: int) -> tuple[float, float, int]:
        """K decode steps timed on the device: step function + sampling kernel, tokens stay on
        the device. Returns (ms per step, mean context length, kernels launched)."""
        e = prefilled(batch, warmup + steps)
        reqs = list(e.requests.values())
        out = torch.empty(batch, dtype=torch.int32, device=dev)
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
        return start.elapsed_time(end) / steps, ctx_sum / (steps * batch), ops.launch_count - before

    def e2e_decode(batch: int, warmup: int, steps: int) -> tuple[float, int, int]:
        e = prefilled(batch, warmup + steps)
        for _ in range(warmup):
            e.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            e.step()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3 / steps
        # per step: the packed int32 inputs (token, position, slot, lengths, block table) and the tokens back
        width = -(-(args.prompt_len + warmup + steps) // page)
        h2d = 4 * (batch * (8 + width) + 16)
        return ms, h2d, 4 * batch

    if args.profile == "timeline":
        # When each kernel of one recorded decode step started and when its wait for the kernels
        # before it returned, from the device clock. Needs the library built with the notes in
        # (TINYSERVE_B200_TIMELINE=1 in the environment); no JSON line, no timing claim.
        if not ops.build.TIMELINE:
            print("--profile timeline needs TINYSERVE_B200_TIMELINE=1 in the environment")
            return 2
        e = prefilled(args.batch, 16)
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
        args.no_graphs = True
        if args.profile == "decode":
            e = prefilled(args.batch, 8)
            for _ in range(2):
                e.step()
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            for _ in range(2):
                e.step()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        else:
            e = new_engine(1, 2048 + 8)
            toks = prompts(1, 2048)[0]
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
    ms, ctx, launches = device_decode(args.batch, args.warmup, args.steps)
    clocks = sampler.stop()
    value = args.batch * 1e3 / ms
    e2e_ms, h2d, d2h = e2e_decode(args.batch, args.warmup, args.steps)
    achieved = decode_bytes(args.batch, ctx) / (ms * 1e-3) / 1e9

    result = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.model.upper()} sizes, bf16, "
                  f"{args.prompt_len:,}-token prompts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights", "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.model.upper()} sizes", "layers": cfg.num_layers, "layers_of_configuration": full_layers,
            "hidden": cfg.hidden_size, "q_heads": cfg.num_heads, "kv_heads": cfg.num_kv_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "tied_embeddings": cfg.tie_word_embeddings, "global_batch": args.batch, "seq_len": args.prompt_len,
            "context_limit": cfg.max_position_embeddings, "mean_context": round(ctx, 1), "page_size": page,
            "parallelism": "single GPU", "l2": f"inputs larger than L2 (weights {model.weight_bytes() / 1e9:.2f} GB read every step)",
            "peaks": pk_src,
        },
        "e2e": {"value": round(args.batch * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_src},
    }
    if not args.skip_points:
        points = {}
        for b in (1, 64):
            pms, _, _ = device_decode(b, 3, max(16, args.steps // 4))
            points[f"decode_b{b}"] = round(b * 1e3 / pms, 1)
        result["points"] = points
        # prefill: one 2,048-token prompt in one step
        t_pre = 2048
        e = new_engine(1, t_pre + 8)
        toks = prompts(1, t_pre)[0]
        times = []
        for it in range(3 + 5):
            req = e.cache.new_request()
            e.cache.append(req, t_pre)
            torch.cuda.synchronize()
            s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_.record()
            e.runner.step([StepEntry(req, toks)])
            e_.record()
            torch.cuda.synchronize()
            e.cache.free(req)
            if it >= 3:
                times.append(s_.elapsed_time(e_))
        pre_ms = statistics.median(times)
        matmul_params = (model.weight_bytes() // 2) - cfg.vocab_size * cfg.hidden_size   # all but the table
        flops = 2.0 * t_pre * matmul_params + 2.0 * cfg.vocab_size * cfg.hidden_size     # head on one row
        flops += cfg.num_layers * 4.0 * cfg.num_heads * cfg.head_dim * (t_pre * (t_pre + 1) / 2)
        result["prefill"] = {"value": round(t_pre * 1e3 / pre_ms, 1), "tokens": t_pre, "ms": round(pre_ms, 3),
                             "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk_src}
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
