"""Generation through the Python entry point on the GPU: greedy tokens equal the plain
implementation's; decode graphs change nothing but the launch path; sampling is reproducible."""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import TINIES, random_prompt, write_tiny

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    out = {}
    for name, lens in (("A", [5, 17, 33]), ("B", [1, 9, 24, 40, 63])):
        cfg, page, seed = TINIES[name]
        folder = write_tiny(tmp_path_factory.mktemp(name), name, torch.bfloat16)
        prompts = [random_prompt(n, cfg["vocab_size"], 50 + i) for i, n in enumerate(lens)]
        pc, pw = plain.read_config(folder), plain.read_weights(folder, torch.float32)
        out[name] = (folder, page, prompts, [plain.greedy(pc, pw, p, 8) for p in prompts])
    return out


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("chunked", [False, True])
def test_greedy_float32_equals_plain(tiny, name, graphs, chunked) -> None:
    from tinyserve_b200 import LLM

    folder, page, prompts, want = tiny[name]
    llm = LLM.from_folder(folder, dtype="float32", page_size=page, num_pages=64, max_num_seqs=4,
                          max_batch_tokens=16 if chunked else 128, chunked_prefill=chunked, decode_graphs=graphs)
    assert llm.generate(prompts, 8) == want
    assert (llm.engine.runner.num_graph_steps > 0) == graphs
    assert all(g.allocator.num_used == 0 for g in llm.cache.groups)


@pytest.mark.parametrize("name", ["A", "B"])
def test_steps_launched_ahead_change_nothing(tiny, name) -> None:
    """Recorded decode steps launched before the tokens of the step before are read (the
    default with decode graphs): the same tokens as without, for greedy and seeded sampling,
    with requests of different lengths and an end token in the middle."""
    from tinyserve_b200 import LLM, SamplingParams

    folder, page, prompts, want = tiny[name]
    outs = []
    for ahead in (False, True):
        llm = LLM.from_folder(folder, dtype="float32", page_size=page, num_pages=64, max_num_seqs=4,
                              max_batch_tokens=128, decode_graphs=True, run_ahead=ahead)
        e = llm.engine
        eos = frozenset({want[1][3]})
        ids = [e.add_request(prompts[0], 8), e.add_request(prompts[1], 8, eos_ids=eos),
               e.add_request(prompts[2], 3, sampling=SamplingParams(temperature=0.9, top_p=0.8, seed=5))]
        while e.has_work():
            e.step()
        outs.append([e.requests[i].output for i in ids])
        assert (e.num_steps_ahead > 0) == ahead
        assert all(g.allocator.num_used == 0 for g in llm.cache.groups)
        assert outs[-1][0] == want[0] and outs[-1][1] == want[1][: want[1].index(want[1][3]) + 1]
    assert outs[0] == outs[1]


@pytest.mark.parametrize("name", ["A", "B"])
def test_everything_at_once_still_equals_plain(tiny, name) -> None:
    """Recorded decode steps, the recorded prompt portion, steps launched ahead, chunked prompts and
    a cache so small that requests are preempted and recomputed, together: greedy tokens still
    equal the plain implementation's, and every page comes back."""
    from tinyserve_b200 import LLM

    folder, page, _, _ = tiny[name]
    cfg = TINIES[name][0]
    pc, pw = plain.read_config(folder), plain.read_weights(folder, torch.float32)
    prompts = [random_prompt(n, cfg["vocab_size"], 80 + i) for i, n in enumerate([3, 29, 16, 41, 8, 33])]
    new = 12
    want = [plain.greedy(pc, pw, p, new) for p in prompts]
    longest = max(len(p) for p in prompts) + new
    pages = -(-longest // page) + 3                         # room for the longest request and little more
    llm = LLM.from_folder(folder, dtype="float32", page_size=page, num_pages=pages, max_num_seqs=4,
                          max_batch_tokens=16, chunked_prefill=True, decode_graphs=True)
    e = llm.engine
    assert e.runner.prefill_graphs, "the prompt portion of the step budget should have been recorded"
    ids = [e.add_request(p, new) for p in prompts[:4]]
    steps = 0
    while e.has_work():
        e.step()
        steps += 1
        if steps == 5:
            ids += [e.add_request(p, new) for p in prompts[4:]]     # late arrivals
    assert [e.requests[i].output for i in ids] == want
    assert e.scheduler.num_preemptions > 0 and e.num_steps_ahead > 0 and e.runner.num_graph_steps > 0
    assert all(g.allocator.num_used == 0 for g in llm.cache.groups)


def test_greedy_bfloat16_close_to_plain_and_tight_cache(tiny) -> None:
    from tinyserve_b200 import LLM

    """bfloat16 through ``Engine`` with recorded steps and a cache so tight that requests wait and
    are preempted: bf16 may flip a near-tie between two tokens, so it is not the tokens that are
    compared but every logits row the engine sampled from, on the sequence it went on to generate,
    with the tolerance of the replay tests. One request wholly wrong cannot pass."""
    from closeness import engine_logits_close_to_plain
    from tinyserve_b200 import LLM

    folder, page, prompts, _ = tiny["B"]
    pc = plain.read_config(folder)
    w32, w16 = plain.read_weights(folder, torch.float32), plain.read_weights(folder, torch.bfloat16)
    llm = LLM.from_folder(folder, dtype="bfloat16", page_size=page, num_pages=10, max_num_seqs=4,
                          max_batch_tokens=128, decode_graphs=True, record_logits=True)
    e = llm.engine
    ids = [e.add_request(p, 8) for p in prompts]
    while e.has_work():
        e.step()
    assert all(len(e.requests[i].output) == 8 for i in ids) and e.runner.num_graph_steps > 0
    n = engine_logits_close_to_plain(e, ids, prompts, lambda s: plain.forward(pc, w32, s), lambda s: plain.forward(pc, w16, s),
                                     torch.bfloat16)
    assert n == 8 * len(prompts)
    assert all(g.allocator.num_used == 0 for g in llm.cache.groups)


def test_graph_logits_equal_eager_logits(tiny) -> None:
    """The recorded decode step and the kernel-by-kernel one give the same logits up to the
    order of the split-K sums."""
    from tinyserve_b200.cache import CacheManager
    from tinyserve_b200.engine.step import ModelRunner, StepEntry
    from tinyserve_b200.model import DecoderModel

    folder, page, prompts, _ = tiny["A"]
    model = DecoderModel.from_folder(folder, torch.float32, "cuda")
    outs = []
    for graphs in (False, True):
        cache = CacheManager(model.cache_needs(), page_size=page, num_pages=32, max_requests=4,
                             dtype=torch.float32, device="cuda")
        runner = ModelRunner(model, cache)
        if graphs:
            runner.record_decode_graphs(4, 256)
        reqs = [cache.new_request() for _ in prompts]
        for r, p in zip(reqs, prompts):
            cache.append(r, len(p))
        runner.step([StepEntry(r, p) for r, p in zip(reqs, prompts)])
        rows = []
        for t in range(5):
            for r in reqs:
                cache.append(r, 1)
            rows.append(runner.step([StepEntry(r, [7 + t]) for r in reqs]).clone())
        assert (runner.num_graph_steps == 5) == graphs
        outs.append(torch.stack(rows))
    torch.testing.assert_close(outs[0], outs[1], atol=2e-5, rtol=2e-5)


@pytest.mark.parametrize("name", ["A", "B"])
def test_recorded_prompt_portion_equals_eager(tiny, name) -> None:
    """A prompt fed in portions of a fixed size: the recorded step of such a portion (on top of
    whatever the request already holds, pages scattered) gives the logits of the kernel-by-kernel
    step; portions of other sizes and steps of several requests are not taken by the recording."""
    from tinyserve_b200.cache import CacheManager
    from tinyserve_b200.engine.step import ModelRunner, StepEntry
    from tinyserve_b200.model import DecoderModel

    folder, page, prompts, _ = tiny[name]
    cfg = TINIES[name][0]
    model = DecoderModel.from_folder(folder, torch.float32, "cuda")
    prompt = random_prompt(59, cfg["vocab_size"], 3)
    portion = 12
    outs = []
    for graphs in (False, True):
        cache = CacheManager(model.cache_needs(), page_size=page, num_pages=40, max_requests=4,
                             dtype=torch.float32, device="cuda")
        runner = ModelRunner(model, cache)
        if graphs:
            runner.record_prefill_graph(portion, 128)
        other = cache.new_request()                     # scatters the pages of the request under test
        r = cache.new_request()
        rows, at = [], 0
        while at < len(prompt):
            n = min(portion, len(prompt) - at)
            cache.append(other, 3)
            cache.append(r, n)
            rows.append(runner.step([StepEntry(r, prompt[at: at + n])]).clone())
            at += n
        assert runner.num_graph_steps == (len(prompt) // portion if graphs else 0)
        cache.append(r, portion)
        assert runner.step([StepEntry(r, prompt[:portion])], [[]]) is None      # a portion that wants nothing
        cache.append(r, portion)
        cache.append(other, portion)
        two = runner.step([StepEntry(r, prompt[:portion]), StepEntry(other, prompt[:portion])])
        assert two.shape[0] == 2
        outs.append(torch.cat(rows))
    torch.testing.assert_close(outs[0], outs[1], atol=2e-5, rtol=2e-5)


def test_seeded_sampling_is_reproducible_and_batch_independent(tiny) -> None:
    from tinyserve_b200 import LLM, SamplingParams

    folder, page, prompts, _ = tiny["B"]
    p = SamplingParams(temperature=0.8, top_p=0.9, seed=7)
    alone = LLM.from_folder(folder, dtype="float32", page_size=page, num_pages=64, max_num_seqs=4).generate(
        [prompts[2]], 6, sampling=p)[0]
    llm = LLM.from_folder(folder, dtype="float32", page_size=page, num_pages=64, max_num_seqs=4,
                          max_batch_tokens=16, chunked_prefill=True)
    e = llm.engine
    others = [e.add_request(q, 6, sampling=SamplingParams(temperature=1.0, seed=i)) for i, q in enumerate(prompts[:2])]
    mine = e.add_request(prompts[2], 6, sampling=p)
    while e.has_work():
        e.step()
    assert e.requests[mine].output == alone and len(set(alone)) > 1
    assert all(len(e.requests[i].output) == 6 for i in others)


def test_command_line(tiny) -> None:
    folder, page, prompts, want = tiny["A"]
    ids = ",".join(str(t) for t in prompts[1])
    cmd = [sys.executable, str(ROOT / "bin" / "generate"), "--model-dir", str(folder), "--prompt-ids", ids,
           "--max-new-tokens", "8", "--dtype", "float32", "--block-size", str(page)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert f"new ids:    {want[1]}" in out.stdout
    out = subprocess.run(cmd + ["--no-cache", "--max-new-tokens", "3"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and f"new ids:    {want[1][:3]}" in out.stdout
    out = subprocess.run(cmd + ["--temperature", "0.8", "--top-p", "0.9", "--seed", "3", "--num-samples", "2"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "2 samples, 16 tokens" in out.stdout, out.stdout + out.stderr[-1000:]
