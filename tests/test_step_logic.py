"""The step function, the cache manager and trace replay on the CPU, with the kernels'
plain references in the kernels' place: every way of cutting requests into steps must give
the plain implementation's logits. (The kernels themselves are tested on the GPU.)"""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

import plain_qwen3 as plain
import replay_cases as cases
from kernel_refs import use_references
from tiny_configs import TINIES, random_prompt, write_tiny

from tinyserve_b200.engine.replay import Replayer
from tinyserve_b200.model import DecoderModel

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 24, 40, 63], "C": [3, 50, 31]}


def _run(model_dir: Path, page: int, steps, max_tokens: int) -> dict[str, dict[int, torch.Tensor]]:
    """Replay ``steps``; returns logits by request id and absolute position."""
    model = DecoderModel.from_folder(model_dir, torch.float32, "cpu")
    rep = Replayer(model, max_tokens, page_size=page)
    got: dict[str, dict[int, torch.Tensor]] = {}
    fed: dict[str, int] = {}
    for entries, end in steps:
        logits = rep.run_step(entries, end)
        row = 0
        for rid, toks, places in entries:
            base = fed.get(rid, 0)
            for p in places:
                got.setdefault(rid, {})[base + p] = logits[row].clone()
                row += 1
            fed[rid] = base + len(toks)
    rep.cache.check_invariant()
    assert all(g.allocator.num_used == 0 for g in rep.cache.groups), "pages leaked"
    return got


@pytest.mark.parametrize("name", sorted(TINIES))
def test_every_cut_gives_the_plain_logits(name: str, tmp_path: Path) -> None:
    cfg, page, seed = TINIES[name]
    folder = write_tiny(tmp_path, name, torch.float32)
    pcfg, pw = plain.read_config(folder), plain.read_weights(folder, torch.float32)
    reqs = {f"r{i}": random_prompt(n, cfg["vocab_size"], 10 * seed + i) for i, n in enumerate(LENGTHS[name])}
    want = {rid: plain.forward(pcfg, pw, toks) for rid, toks in reqs.items()}
    with use_references():
        for rid, toks in reqs.items():
            for steps in (cases.whole(rid, toks), cases.tail_decoded(rid, toks, 32), cases.portions(rid, toks, seed)):
                got = _run(folder, page, steps, cases.max_live_tokens(steps))
                for pos, row in got[rid].items():
                    torch.testing.assert_close(row, want[rid][pos], atol=2e-5, rtol=2e-5)
                assert len(got[rid]) == len(toks)
        steps = cases.mixed(reqs, seed)
        got = _run(folder, page, steps, cases.max_live_tokens(steps))
        for rid, toks in reqs.items():
            assert len(got[rid]) == len(toks)
            for pos, row in got[rid].items():
                torch.testing.assert_close(row, want[rid][pos], atol=2e-5, rtol=2e-5)
