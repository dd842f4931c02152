"""The scheduler's decisions, with a fake model: the next token is a fixed function of the
tokens so far (after upstream tests/test_scheduler.py:22-33), so any scheduling mistake that
loses, repeats or reorders tokens changes the output."""

from __future__ import annotations

import random

import pytest
import torch

from tinyserve_b200.cache import CacheManager
from tinyserve_b200.engine.request import Request, Status
from tinyserve_b200.engine.scheduler import Scheduler
from tinyserve_b200.parts.base import KVNeed, StateNeed


def fake_next(tokens: list[int]) -> int:
    return (sum((i + 1) * t for i, t in enumerate(tokens)) + len(tokens)) % 97


def expected(prompt: list[int], n: int) -> list[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        out.append(fake_next(toks))
        toks.append(out[-1])
    return out


def make(num_pages=8, page=4, seqs=4, budget=64, chunked=False, needs=None) -> Scheduler:
    cache = CacheManager(needs or [KVNeed(1, 16)], page_size=page, num_pages=num_pages, max_requests=seqs,
                         dtype=torch.float32, device="cpu", allocate_memory=False)
    return Scheduler(cache, seqs, budget, chunked_prefill=chunked)


def run(s: Scheduler, reqs: list[Request], max_steps: int = 10_000) -> list[list[tuple[int, int]]]:
    """Drive the scheduler to the end; returns, per step, (request id, tokens run)."""
    seen: dict[int, list[int]] = {r.request_id: [] for r in reqs}     # what the "cache" holds per request
    log = []
    for _ in range(max_steps):
        if not s.has_work():
            break
        s.schedule()
        step = s.scheduled()
        assert step, "no progress"
        assert sum(r.num_scheduled for r in step) <= s.max_batch_tokens
        assert len(s.running) <= s.max_num_seqs
        sampled, toks = [], []
        for r in step:
            end = r.cache.num_tokens
            new = r.tokens[end - r.num_scheduled: end]
            if end - r.num_scheduled == 0:
                seen[r.request_id] = []                                # (re)computed from its first token
            assert len(seen[r.request_id]) == end - r.num_scheduled, "tokens fed out of order"
            seen[r.request_id] += new
            if not r.in_prefill():
                sampled.append(r)
                toks.append(fake_next(seen[r.request_id]))
        log.append([(r.request_id, r.num_scheduled) for r in step])
        s.update(sampled, toks)
        s.cache.check_invariant()
    assert not s.has_work(), "did not finish (livelock?)"
    assert all(g.allocator.num_used == 0 for g in s.cache.groups), "pages leaked"
    return log


def test_admission_is_first_come_first_served_and_respects_the_budget() -> None:
    s = make(num_pages=64, budget=10)
    reqs = [Request(i, [i + 1] * n, 2) for i, n in enumerate([6, 6, 2])]
    for r in reqs:
        s.add(r)
    s.schedule()
    assert [r.request_id for r in s.scheduled()] == [0]       # 6 + 6 > 10; request 2 may not overtake
    s.update([reqs[0]], [fake_next(reqs[0].tokens)])
    s.schedule()
    assert [(r.request_id, r.num_scheduled) for r in s.scheduled()] == [(0, 1), (1, 6), (2, 2)]


def test_refuses_what_can_never_fit() -> None:
    s = make(num_pages=4, page=4, budget=8)
    with pytest.raises(ValueError, match="one step"):
        s.add(Request(0, [1] * 8, 2))                          # 9 tokens to recompute at once > 8
    with pytest.raises(ValueError, match="cache holds"):
        make(num_pages=2, page=4, budget=64).add(Request(0, [1] * 8, 2))
    with pytest.raises(ValueError):
        Request(1, [], 1)
    with pytest.raises(ValueError):
        Request(1, [1], 0)
    with pytest.raises(ValueError, match="chunked"):
        make(seqs=8, budget=4, chunked=True)


def test_out_of_pages_preempts_the_newest_and_recomputes() -> None:
    s = make(num_pages=4, page=4, seqs=4, budget=64)          # 16 tokens of cache for two growing requests
    a, b = Request(0, [3] * 7, 6), Request(1, [5] * 7, 6)
    s.add(a), s.add(b)
    log = run(s, [a, b])
    assert s.num_preemptions >= 1 and b.num_preemptions >= 1 and a.num_preemptions == 0
    assert a.output == expected([3] * 7, 6) and b.output == expected([5] * 7, 6)
    # after the preemption b comes back with prompt + output as one portion
    assert any(rid == 1 and n > 7 for step in log for rid, n in step)


def test_a_lone_request_preempts_itself_only_if_it_must() -> None:
    s = make(num_pages=3, page=4, budget=64)
    a = Request(0, [2] * 5, 8)                                 # needs 12 tokens: exactly the cache
    s.add(a)
    run(s, [a])
    assert a.output == expected([2] * 5, 8) and a.num_preemptions == 0


def test_chunked_prefill_portions_and_decodes_together() -> None:
    s = make(num_pages=64, page=4, seqs=4, budget=8, chunked=True)
    a, b = Request(0, [1, 2, 3], 5), Request(1, list(range(1, 21)), 3)
    s.add(a), s.add(b)
    log = run(s, [a, b])
    assert log[0] == [(0, 3), (1, 5)]                          # b's prompt is cut to what the budget leaves
    assert log[1] == [(0, 1), (1, 7)] and log[2] == [(0, 1), (1, 7)] and log[3] == [(0, 1), (1, 1)]
    assert a.output == expected([1, 2, 3], 5) and b.output == expected(list(range(1, 21)), 3)


def test_mid_prompt_request_samples_nothing() -> None:
    s = make(num_pages=64, budget=4, chunked=True)
    a = Request(0, [1] * 10, 2)
    s.add(a)
    s.schedule()
    assert a.in_prefill()
    with pytest.raises(ValueError, match="still in its prompt"):
        s.update([a], [5])


def test_abort_gives_everything_back() -> None:
    s = make(num_pages=8, needs=[KVNeed(1, 16), StateNeed((4,))])
    a, b = Request(0, [1] * 6, 4), Request(1, [2] * 6, 4)
    s.add(a), s.add(b)
    s.schedule()
    s.abort(a), s.abort(b), s.abort(a)
    assert not s.has_work() and s.cache.groups[0].allocator.num_used == 0 and s.cache.state_pool.num_free == 4


def test_state_slots_limit_admission() -> None:
    cache = CacheManager([KVNeed(1, 16), StateNeed((4,))], page_size=4, num_pages=64, max_requests=2,
                         dtype=torch.float32, device="cpu", allocate_memory=False)
    s = Scheduler(cache, max_num_seqs=8, max_batch_tokens=64)
    reqs = [Request(i, [i + 1] * 3, 2) for i in range(3)]
    for r in reqs:
        s.add(r)
    log = run(s, reqs)
    assert [rid for rid, _ in log[0]] == [0, 1]                # the third waits for a free slot
    assert [r.output for r in reqs] == [expected([i + 1] * 3, 2) for i in range(3)]


@pytest.mark.parametrize("seed", range(40))
def test_random_workloads_finish_right_and_leak_nothing(seed) -> None:
    rng = random.Random(seed)
    page = rng.choice([1, 3, 4, 16])
    chunked = rng.random() < 0.5
    seqs = rng.randint(1, 5)
    budget = rng.randint(max(seqs, 4), 40)
    window = rng.choice([None, None, 6])
    needs = [KVNeed(1, 16), KVNeed(1, 16, window=window)]
    reqs = [Request(i, [rng.randrange(97) for _ in range(rng.randint(1, 24))], rng.randint(1, 12))
            for i in range(rng.randint(1, 9))]
    longest = max(r.max_cached_tokens for r in reqs)
    if not chunked:
        budget = max(budget, longest)
    num_pages = -(-longest // page) + rng.randint(0, 6)
    s = make(num_pages=num_pages, page=page, seqs=seqs, budget=budget, chunked=chunked, needs=needs)
    pending = list(reqs)
    for r in pending[: len(pending) // 2]:
        s.add(r)
    late = pending[len(pending) // 2:]
    seen: dict[int, list[int]] = {r.request_id: [] for r in reqs}
    steps = 0
    while s.has_work() or late:
        if late and (not s.has_work() or rng.random() < 0.3):
            s.add(late.pop(0))                                  # requests join while others run
        s.schedule()
        step = s.scheduled()
        assert step
        sampled, toks = [], []
        for r in step:
            end = r.cache.num_tokens
            if end - r.num_scheduled == 0:
                seen[r.request_id] = []
            assert len(seen[r.request_id]) == end - r.num_scheduled
            seen[r.request_id] += r.tokens[end - r.num_scheduled: end]
            if not r.in_prefill():
                sampled.append(r)
                toks.append(fake_next(seen[r.request_id]))
        s.update(sampled, toks)
        s.cache.check_invariant()
        steps += 1
        assert steps < 5000, "livelock"
    assert all(r.status is Status.FINISHED and r.output == expected(r.prompt, r.max_new_tokens) for r in reqs)
    assert all(g.allocator.num_used == 0 for g in s.cache.groups)


def test_schedule_ahead_reserves_only_what_needs_no_decision() -> None:
    """The next decode step may be reserved before this step's tokens are known only if nobody
    waits, nobody is about to reach its length limit, and a token fits for everybody."""
    s = make(num_pages=4, page=4, seqs=2)
    a, b = Request(0, [1, 2, 3], 6), Request(1, [4, 5], 6)
    s.add(a)
    s.add(b)
    s.schedule()
    assert s.schedule_ahead() is None                       # they ran their prompts (3 and 2 tokens), not one token
    s.update([a, b], [7, 8])
    s.schedule()                                            # one token each
    free = s.cache.groups[0].allocator.num_free
    ahead = s.schedule_ahead()
    assert ahead == [a, b] and a.num_pending() == -1 and b.num_pending() == -1
    assert s.cache.groups[0].allocator.num_free == free - 1   # a's fifth token opens its second page
    s.update([a, b], [9, 10])                               # the tokens of the step before arrive
    assert a.num_pending() == 0 and not a.in_prefill() and a.output == [7, 9]
    # a third request waits: admission is a decision, so nothing is reserved ahead
    s.add(Request(2, [1], 2))
    assert s.schedule_ahead() is None
    s.waiting.clear()
    s.update([a, b], [11, 12])
    s.schedule()
    # pages: a (6 cached) and b (5 cached) hold 2 pages each of the 4; a token more fits both
    assert s.schedule_ahead() == [a, b]
    s.update([a, b], [13, 14])
    s.update([a, b], [15, 16])
    s.schedule()
    # both now hold 8 tokens = 2 full pages, no page is free: the next token fits nobody
    assert s.cache.groups[0].allocator.num_free == 0 and s.schedule_ahead() is None
    s.cache.check_invariant()


def test_schedule_ahead_stops_before_the_length_limit_and_survives_an_end_token() -> None:
    s = make(num_pages=16, page=4, seqs=2)
    a, b = Request(0, [1, 2], 3), Request(1, [3], 9, eos_ids=frozenset({50}))
    s.add(a)
    s.add(b)
    s.schedule()
    s.update([a, b], [7, 8])
    s.schedule()
    # a has 1 of 3 tokens; the token under way is its second, so a third step is still its own
    assert s.schedule_ahead() == [a, b]
    s.update([a, b], [9, 50])                               # b draws its end token: it leaves, the extra room with it
    assert b.status is Status.FINISHED and b.cache is None and s.running == [a]
    # a's step ahead was its last (third token): nothing more may be reserved
    assert s.schedule_ahead() is None
    s.update([a], [11])
    assert a.status is Status.FINISHED and not s.has_work()
    assert all(g.allocator.num_used == 0 for g in s.cache.groups)


def test_a_portion_cut_down_to_one_token_is_charged_to_the_budget() -> None:
    """Two requests in mid-prompt and room for one more token in the step: the first gets it, the
    second waits (it keeps its place and its cache); the step never exceeds ``max_batch_tokens``."""
    s = make(num_pages=64, page=4, seqs=4, budget=4, chunked=True)
    reqs = [Request(0, [1] * 3, 8), Request(1, [2] * 12, 2), Request(2, [3] * 12, 2), Request(3, [4] * 12, 2)]
    for r in reqs:
        r.cache = s.cache.new_request()
        r.status = Status.RUNNING
        s.running.append(r)
    # request 0 decodes; request 1 has 2 prompt tokens left (they fit); 2 and 3 are in mid-prompt
    s.cache.append(reqs[0].cache, 3)
    reqs[0].output.append(5)
    s.cache.append(reqs[1].cache, 10)
    s.cache.append(reqs[2].cache, 4)
    s.cache.append(reqs[3].cache, 4)
    s.schedule()
    assert [(r.request_id, r.num_scheduled) for r in s.running] == [(0, 1), (1, 2), (2, 1), (3, 0)]
    assert sum(r.num_scheduled for r in s.scheduled()) == s.max_batch_tokens
