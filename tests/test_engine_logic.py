"""The engine (scheduler + step function + sampler) on the CPU with the kernels' references in
the kernels' place: greedy generation equals the plain implementation's under roomy, one-at-a-time
and tight caches and with chunked prefill; seeded sampling does not depend on batch-mates,
chunking or preemption (after upstream tests/test_engine.py:26-141, tests/test_sampling.py:163-183)."""

from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
from kernel_refs import use_references
from tiny_configs import TINIES, random_prompt, write_tiny

from tinyserve_b200.cache import CacheManager
from tinyserve_b200.engine import Engine
from tinyserve_b200.model import DecoderModel
from tinyserve_b200.sampling import SamplingParams

PROMPTS = {"A": [5, 17, 33], "B": [1, 9, 24, 40, 63]}
NEW = {"A": 8, "B": 6}


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    out = {}
    for name in ("A", "B"):
        cfg, page, seed = TINIES[name]
        folder = write_tiny(tmp_path_factory.mktemp(name), name, torch.float32)
        prompts = [random_prompt(n, cfg["vocab_size"], 50 + i) for i, n in enumerate(PROMPTS[name])]
        pc, pw = plain.read_config(folder), plain.read_weights(folder, torch.float32)
        want = [plain.greedy(pc, pw, p, NEW[name]) for p in prompts]
        out[name] = (DecoderModel.from_folder(folder, torch.float32, "cpu"), page, prompts, want)
    return out


def engine(model, page, num_pages, **kw) -> Engine:
    cache = CacheManager(model.cache_needs(), page_size=page, num_pages=num_pages, max_requests=8,
                         dtype=torch.float32, device="cpu")
    return Engine(model, cache, **kw)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("mode", ["roomy", "one_at_a_time", "tight", "chunked", "chunked_tight"])
def test_greedy_equals_plain(setup, name, mode) -> None:
    model, page, prompts, want = setup[name]
    longest = max(len(p) for p in prompts) + NEW[name]
    tight = -(-longest // page) + 1
    kw = {"roomy": dict(num_pages=200), "one_at_a_time": dict(num_pages=200, max_num_seqs=1),
          "tight": dict(num_pages=tight), "chunked": dict(num_pages=200, max_batch_tokens=16, chunked_prefill=True,
                                                          max_num_seqs=8),
          "chunked_tight": dict(num_pages=tight, max_batch_tokens=16, chunked_prefill=True, max_num_seqs=8)}[mode]
    with use_references():
        e = engine(model, page, **kw)
        got = e.generate(prompts, NEW[name])
    assert got == want
    assert len({tuple(w) for w in want}) > 1 and any(len(set(w)) > 1 for w in want), "degenerate oracle"
    assert all(g.allocator.num_used == 0 for g in e.cache.groups)
    assert all(t.ttft >= 0 for t in e.times.values())


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("chunked", [False, True])
def test_pages_run_out_newest_is_recomputed(setup, tmp_path, name, chunked) -> None:
    """Two requests that fit at first but cannot both grow: the newer one is preempted, later
    recomputed from its first token, and still generates the plain implementation's tokens."""
    model, page, _, _ = setup[name]
    cfg = TINIES[name][0]
    prompts = [random_prompt(page, cfg["vocab_size"], 70 + i) for i in range(2)]
    with use_references():
        e = engine(model, page, 3, max_batch_tokens=64, chunked_prefill=chunked, max_num_seqs=4)
        got = e.generate(prompts, 6)
    w = {k: v.float() for k, v in model.tensors.items()}
    want = [greedy_from_bound(cfg, w, q, 6) for q in prompts]
    assert got == want and e.scheduler.num_preemptions > 0
    assert e.requests[1].num_preemptions > 0 and e.requests[0].num_preemptions == 0


def greedy_from_bound(cfg, bound, prompt, n):
    """The plain implementation on the tensors the model holds (merged ones split back)."""
    w = {}
    hq, hkv, d, inter = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["intermediate_size"]
    for k, v in bound.items():
        if k.endswith("qkv_proj.weight"):
            p = k[: -len("qkv_proj.weight")]
            w[p + "q_proj.weight"], w[p + "k_proj.weight"], w[p + "v_proj.weight"] = v.split([hq * d, hkv * d, hkv * d])
        elif k.endswith("gate_up_proj.weight"):
            p = k[: -len("gate_up_proj.weight")]
            w[p + "gate_proj.weight"], w[p + "up_proj.weight"] = v.split([inter, inter])
        else:
            w[k] = v
    return plain.greedy(dict(cfg), w, prompt, n)


def test_seeded_sampling_ignores_batch_chunking_and_preemption(setup) -> None:
    model, page, prompts, _ = setup["B"]
    p = SamplingParams(temperature=0.8, top_p=0.9, seed=1234)
    with use_references():
        alone = engine(model, page, 200).generate([prompts[3]], 6, sampling=p)[0]
        e = engine(model, page, 200, max_batch_tokens=16, chunked_prefill=True, max_num_seqs=8)
        ids = [e.add_request(q, 6, sampling=SamplingParams(temperature=1.1, seed=i)) for i, q in enumerate(prompts[:3])]
        mine = e.add_request(prompts[3], 6, sampling=p)
        while e.has_work():
            e.step()
        q8, other = random_prompt(page, 384, 91), random_prompt(page, 384, 92)
        alone8 = engine(model, page, 200).generate([q8], 6, sampling=p)[0]
        tight = engine(model, page, 3)
        ids2 = [tight.add_request(q, 6, sampling=p) for q in (other, q8)]
        while tight.has_work():
            tight.step()
    assert e.requests[mine].output == alone
    assert tight.requests[ids2[1]].num_preemptions > 0 and tight.requests[ids2[1]].output == alone8
    assert len(set(alone)) > 1
    assert ids and all(len(e.requests[i].output) == 6 for i in ids)


def test_temperature_zero_and_logprobs(setup) -> None:
    model, page, prompts, want = setup["A"]
    with use_references():
        e = engine(model, page, 200)
        a = e.add_request(prompts[1], 4, sampling=SamplingParams(temperature=0.0, logprobs=3))
        b = e.add_request(prompts[2], 4, sampling=SamplingParams(temperature=0.9))   # mixed batch
        while e.has_work():
            e.step()
    assert e.requests[a].output == want[1][:4]
    lps = e.logprobs[a]
    assert len(lps) == 4 and all(len(x.top) == 3 and x.top[0][0] == t and abs(x.top[0][1] - x.logprob) < 1e-6
                                 for x, t in zip(lps, e.requests[a].output))
    assert len(e.requests[b].output) == 4


def test_eos_stops_and_bad_requests_are_refused(setup) -> None:
    model, page, prompts, want = setup["A"]
    with use_references():
        e = engine(model, page, 200)
        out = e.generate([prompts[0]], 8, eos_ids=frozenset({want[0][2]}))[0]
        first = want[0].index(want[0][2])
        assert out == want[0][: first + 1]
        with pytest.raises(ValueError, match="token id"):
            e.add_request([0, 256], 2)
        with pytest.raises(ValueError):
            e.add_request([], 2)
        rid = e.add_request(prompts[0], 3)
        e.step()
        e.abort(rid)
        assert not e.has_work() and all(g.allocator.num_used == 0 for g in e.cache.groups)
        e.release(rid)
        assert rid not in e.requests


class _ReplayingRunner:
    """Makes the CPU engine believe its decode steps are recorded ones, so that it launches
    steps ahead: a step launched ahead takes its tokens from the sampler's output tensor, as
    the recorded step does on the device."""

    @staticmethod
    def wrap(runner):
        from tinyserve_b200.engine.step import StepEntry

        plain_step = runner.step
        runner.graph_max_context = 10 ** 9
        runner.replays = lambda entries, want=None: (
            all(len(e.tokens) == 1 for e in entries) and (want is None or all(list(w) == [0] for w in want)))

        def step(entries, want=None, tokens_from=None):
            if tokens_from is not None:
                toks = tokens_from[: len(entries)].tolist()
                entries = [StepEntry(e.cache, [t]) for e, t in zip(entries, toks)]
            return plain_step(entries, want)

        runner.step = step
        return runner


@pytest.mark.parametrize("name", ["A", "B"])
def test_steps_launched_ahead_change_nothing(setup, name) -> None:
    """With decode steps launched before the tokens of the step before are read: the same
    tokens as without, for greedy and seeded sampling, different lengths, an end token in the
    middle (the token run too many is dropped), a request that joins late and an abort."""
    model, page, prompts, want = setup[name]
    outs = []
    for ahead in (False, True):
        with use_references():
            e = engine(model, page, 200, run_ahead=ahead)
            _ReplayingRunner.wrap(e.runner)
            eos = frozenset({want[1][3]})
            ids = [e.add_request(prompts[0], NEW[name]),
                   e.add_request(prompts[1], NEW[name], eos_ids=eos),
                   e.add_request(prompts[2], 3, sampling=SamplingParams(temperature=0.9, top_p=0.8, seed=5))]
            steps = 0
            late = doomed = None
            while e.has_work():
                e.step()
                steps += 1
                if steps == 3:
                    late = e.add_request(prompts[0][:2], 4, sampling=SamplingParams(temperature=0.7, seed=9))
                    doomed = e.add_request(prompts[1], 50)
                if steps == 6:
                    e.abort(doomed)
            outs.append([e.requests[i].output for i in ids + [late]])
            assert (e.num_steps_ahead > 0) == ahead
            assert all(g.allocator.num_used == 0 for g in e.cache.groups)
            assert e.requests[ids[0]].output == want[0]
            assert e.requests[ids[1]].output == want[1][: want[1].index(want[1][3]) + 1]
    assert outs[0] == outs[1]
