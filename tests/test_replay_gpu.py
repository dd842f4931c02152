"""The engine on the GPU against the plain implementation, in float32 and bfloat16, under every
way of cutting the work: each request alone and whole; most of it in one step and the last 32
tokens one by one; portions of changing size down to two tokens; mixed, up to four live requests
with so few pages that they are used again. Also ``bin/trace_run`` itself as a subprocess."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_cases as cases
from tiny_configs import TINIES, random_prompt, write_tiny

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"A": [5, 17, 33, 70, 130], "B": [1, 9, 24, 40, 63, 97], "C": [3, 50, 31, 64]}


from closeness import FP32_TOL, close_enough  # noqa: E402,F401  (re-exported to the other GPU tests)


def run_steps(model, page: int, steps, max_tokens: int):
    from tinyserve_b200.engine.replay import Replayer

    rep = Replayer(model, max_tokens, page_size=page)
    # Pages nobody owns hold NaN: a read outside a request's own tokens shows in the logits.
    for g in rep.cache.groups:
        g.kv.fill_(float("nan"))
    got: dict[str, dict[int, torch.Tensor]] = {}
    fed: dict[str, int] = {}
    for entries, end in steps:
        logits = rep.run_step(entries, end)
        row = 0
        for rid, toks, places in entries:
            base = fed.get(rid, 0)
            for p in places:
                got.setdefault(rid, {})[base + p] = logits[row].float().cpu()
                row += 1
            fed[rid] = base + len(toks)
    rep.cache.check_invariant()
    assert all(g.allocator.num_used == 0 for g in rep.cache.groups), "pages leaked"
    return got


def check(got, want, reqs, dtype) -> None:
    want32, want16 = want
    for rid, toks in reqs.items():
        assert sorted(got[rid]) == list(range(len(toks)))
        rows = torch.stack([got[rid][p] for p in range(len(toks))])
        assert not rows.isnan().any(), f"{rid}: NaN in the logits (a read outside the request's pages?)"
        close_enough(rows, want32[rid], want16[rid], dtype)


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    out = {}
    for name, (cfg, page, seed) in TINIES.items():
        folder = write_tiny(tmp_path_factory.mktemp(f"tiny_{name}"), name, torch.bfloat16)
        reqs = {f"r{i}": random_prompt(n, cfg["vocab_size"], 10 * seed + i) for i, n in enumerate(LENGTHS[name])}
        pcfg = plain.read_config(folder)
        # The oracle is the plain implementation in 32-bit on the same (bf16-representable) weights.
        pw = plain.read_weights(folder, torch.float32)
        pw16 = plain.read_weights(folder, torch.bfloat16)
        want = ({rid: plain.forward(pcfg, pw, toks) for rid, toks in reqs.items()},
                {rid: plain.forward(pcfg, pw16, toks) for rid, toks in reqs.items()})
        out[name] = (folder, page, seed, reqs, want)
    return out


@pytest.fixture(scope="module")
def models(tiny):
    from tinyserve_b200.model import DecoderModel
    import tinyserve_b200.architectures  # noqa: F401

    return {(name, dt): DecoderModel.from_folder(tiny[name][0], dt, "cuda")
            for name in tiny for dt in (torch.float32, torch.bfloat16)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", sorted(TINIES))
def test_alone_and_whole(tiny, models, name, dtype) -> None:
    _, page, _, reqs, want = tiny[name]
    for rid, toks in reqs.items():
        steps = cases.whole(rid, toks)
        check(run_steps(models[name, dtype], page, steps, cases.max_live_tokens(steps)), want, {rid: toks}, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", sorted(TINIES))
def test_last_32_tokens_one_by_one(tiny, models, name, dtype) -> None:
    _, page, _, reqs, want = tiny[name]
    for rid, toks in reqs.items():
        steps = cases.tail_decoded(rid, toks, 32)
        check(run_steps(models[name, dtype], page, steps, cases.max_live_tokens(steps)), want, {rid: toks}, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", sorted(TINIES))
def test_portions_of_changing_size(tiny, models, name, dtype) -> None:
    _, page, seed, reqs, want = tiny[name]
    for rid, toks in reqs.items():
        steps = cases.portions(rid, toks, seed)
        check(run_steps(models[name, dtype], page, steps, cases.max_live_tokens(steps)), want, {rid: toks}, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", sorted(TINIES))
def test_mixed_with_pages_used_again(tiny, models, name, dtype) -> None:
    _, page, seed, reqs, want = tiny[name]
    for s in (seed, seed + 11):
        steps = cases.mixed(reqs, s)
        check(run_steps(models[name, dtype], page, steps, cases.max_live_tokens(steps)), want, reqs, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_and_first_tokens(tiny, models, dtype) -> None:
    """300 tokens one by one from the very first token of the sequence."""
    name = "B"
    folder, page, seed, _, _ = tiny[name]
    toks = random_prompt(300, TINIES[name][0]["vocab_size"], 77)
    pcfg, pw = plain.read_config(folder), plain.read_weights(folder, torch.float32)
    want = ({"d": plain.forward(pcfg, pw, toks)},
            {"d": plain.forward(pcfg, plain.read_weights(folder, torch.bfloat16), toks)})
    steps = [([("d", [t], [0])], []) for t in toks]
    steps[-1] = (steps[-1][0], ["d"])
    check(run_steps(models[name, dtype], page, steps, cases.max_live_tokens(steps)), want, {"d": toks}, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tiny, tmp_path, dtype) -> None:
    folder, _, seed, reqs, want = tiny["A"]
    steps = cases.mixed(reqs, seed + 3)
    lines = [json.dumps({"step": n, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in entries],
                         "end": end}) for n, (entries, end) in enumerate(steps)]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(cases.max_live_tokens(steps))],
                          input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [x for n in range(len(steps)) for x in ("done", str(n))]
    vocab = TINIES["A"][0]["vocab_size"]
    got: dict[str, dict[int, torch.Tensor]] = {}
    fed: dict[str, int] = {}
    for n, (entries, _) in enumerate(steps):
        data = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, vocab).copy())
        row = 0
        for rid, toks, places in entries:
            for p in places:
                got.setdefault(rid, {})[fed.get(rid, 0) + p] = data[row]
                row += 1
            fed[rid] = fed.get(rid, 0) + len(toks)
        assert row == data.shape[0]
    check(got, want, reqs, torch.float32 if dtype == "float32" else torch.bfloat16)
