"""Command line: prompt in, generated tokens out, in the manner of upstream
scripts/generate.py:35-109 (same option names and meanings where upstream has them).

    python -m tinyserve_b200.generate --model-dir DIR --prompt "The capital of France is" --max-new-tokens 20
    python -m tinyserve_b200.generate --model-dir DIR --prompt-ids 1,2,3 --temperature 0.8 --top-p 0.95 \
        --num-samples 4 --seed 1

``--model-dir`` holds ``config.json`` and ``*.safetensors`` (and ``tokenizer.json`` if
``--prompt`` is text; ``generation_config.json`` supplies the EOS ids). Greedy with one sample
feeds the prompt once and then one token per step from the paged cache; ``--no-cache`` re-runs
the whole sequence for every token instead. ``--temperature > 0`` or ``--num-samples > 1`` runs
the samples as one batch, sample ``i`` with seed ``seed + i``. Options beyond upstream's:
``--dtype bfloat16``, ``--prompt-ids``, ``--random-weights`` (write a random model folder for
the ``config.json`` found in ``--model-dir`` first), ``--max-num-seqs``, ``--max-batch-tokens``,
``--chunked-prefill``, ``--num-blocks``, ``--no-cuda-graphs`` (decode steps are recorded once per
batch size and replayed, and launched ahead of their tokens, unless this is given). The engine
is set up before the clock starts, so the tokens/s line is about generation alone.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path


def eos_ids(model_dir: Path) -> frozenset[int]:
    path = model_dir / "generation_config.json"
    if not path.exists():
        return frozenset()
    eos = json.loads(path.read_text(encoding="utf-8")).get("eos_token_id", [])
    return frozenset(eos if isinstance(eos, list) else [eos])


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Generate with tinyserve_b200 (one B200, hand-written CUDA kernels).")
    p.add_argument("--model-dir", type=Path, default=Path("checkpoints/Qwen3-0.6B"))
    p.add_argument("--prompt", default="The capital of France is")
    p.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of --prompt")
    p.add_argument("--max-new-tokens", type=int, default=20)
    p.add_argument("--dtype", choices=["float32", "bfloat16"], default="float32")
    p.add_argument("--device", default="cuda")
    p.add_argument("--no-cache", action="store_true", help="re-run the whole sequence for every token")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--num-blocks", type=int, default=None, help="cache pages (default: just enough)")
    p.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=None, help="per-sample seeds start here")
    p.add_argument("--num-samples", type=int, default=1)
    p.add_argument("--max-num-seqs", type=int, default=None)
    p.add_argument("--max-batch-tokens", type=int, default=2048)
    p.add_argument("--chunked-prefill", action="store_true")
    p.add_argument("--no-cuda-graphs", action="store_true", help="launch every decode step kernel by kernel")
    p.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                   help="first write model.safetensors with random weights for --model-dir's config.json")
    return p


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    import torch

    from . import architectures  # noqa: F401
    from .config.registry import load_config
    from .engine.engine import Engine
    from .engine.llm import LLM
    from .model import DecoderModel
    from .sampling.params import SamplingParams
    from .weights.random_init import write_random_model

    if args.device != "cuda" or not torch.cuda.is_available():
        print("tinyserve_b200 runs on a CUDA device only (no CPU path)", file=sys.stderr)
        return 2
    dtype = getattr(torch, args.dtype)
    if args.random_weights is not None:
        write_random_model(args.model_dir, load_config(args.model_dir), args.random_weights, torch.bfloat16)
    model = DecoderModel.from_folder(args.model_dir, dtype, args.device)

    tok = None
    if args.prompt_ids is not None:
        prompt_ids = [int(x) for x in args.prompt_ids.split(",") if x.strip()]
    else:
        tok_path = args.model_dir / "tokenizer.json"
        if not tok_path.exists():
            print(f"no tokenizer.json in {args.model_dir}: pass --prompt-ids", file=sys.stderr)
            return 2
        from tokenizers import Tokenizer

        tok = Tokenizer.from_file(str(tok_path))
        prompt_ids = tok.encode(args.prompt).ids
    eos = eos_ids(args.model_dir)
    n = args.num_samples
    per_seq = -(-(len(prompt_ids) + args.max_new_tokens) // args.block_size)
    num_blocks = args.num_blocks or n * per_seq

    def make_engine(max_seqs: int) -> Engine:
        # the same sizing and switches as the Python entry point
        return LLM(model, page_size=args.block_size, num_pages=num_blocks, max_num_seqs=max_seqs,
                   max_batch_tokens=max(args.max_batch_tokens, max_seqs), chunked_prefill=args.chunked_prefill,
                   decode_graphs=not args.no_cuda_graphs).engine

    def show(ids: list[int]) -> str:
        return repr(tok.decode(ids)) if tok is not None else str(ids)

    sampled = args.temperature > 0 or n > 1
    if sampled:
        engine = make_engine(args.max_num_seqs or n)
        start = time.perf_counter()
        rids = []
        for i in range(n):
            seed = None if args.seed is None else args.seed + i
            rids.append(engine.add_request(prompt_ids, args.max_new_tokens, eos,
                                           SamplingParams(args.temperature, args.top_p, seed)))
        while engine.has_work():
            engine.step()
        secs = time.perf_counter() - start
        total = 0
        for i in rids:
            out = engine.requests[i].output
            total += len(out)
            print(f"[{i}] {show(prompt_ids)} -> {show(out)}")
        print(f"{n} samples, {total} tokens in {secs:.2f}s on {args.device} ({args.dtype}), temperature "
              f"{args.temperature}, top_p {args.top_p}, seed {args.seed}, {engine.num_steps} engine steps")
        return 0
    if args.no_cache:
        mode = "no cache between steps"
        new: list[int] = []
        ids = list(prompt_ids)
        args.no_cuda_graphs = True      # every token is a prompt step of a fresh engine: nothing to replay
        start = time.perf_counter()
        for _ in range(args.max_new_tokens):
            engine = make_engine(1)     # nothing is kept from one token to the next
            nxt = engine.generate([ids], 1)[0][0]
            new.append(nxt)
            ids.append(nxt)
            if nxt in eos:
                break
    else:
        mode = f"paged cache, {num_blocks} blocks x {args.block_size} tokens"
        engine = make_engine(1)
        start = time.perf_counter()
        new = engine.generate([prompt_ids], args.max_new_tokens, eos)[0]
        if engine.runner.graphs:
            mode += f", {engine.runner.num_graph_steps} of {engine.num_steps} steps replayed from recordings"
    secs = time.perf_counter() - start
    print(f"prompt ids: {prompt_ids}")
    print(f"new ids:    {new}")
    if tok is not None:
        print(f"text: {args.prompt!r} -> {tok.decode(new)!r}")
    print(f"{len(new)} tokens in {secs:.2f}s ({len(new) / secs:.1f} tokens/s) on {args.device} ({args.dtype}), {mode}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
