"""Ways of cutting the same requests into steps, shared by the host-only and the GPU tests.

A *schedule* is a list of steps; a step is ``(entries, end)`` with ``entries`` a list of
``(request id, token list, wanted places)`` and ``end`` the ids that finish after it."""

from __future__ import annotations

import random

Step = tuple[list[tuple[str, list[int], list[int]]], list[str]]


def whole(rid: str, tokens: list[int]) -> list[Step]:
    """The request alone, all tokens in one step, every place wanted."""
    return [([(rid, tokens, list(range(len(tokens))))], [rid])]


def tail_decoded(rid: str, tokens: list[int], tail: int = 32) -> list[Step]:
    """Most of it in one step, the last ``tail`` tokens one by one."""
    head = max(1, len(tokens) - tail)
    steps: list[Step] = [([(rid, tokens[:head], list(range(head)))], [])]
    for i in range(head, len(tokens)):
        steps.append(([(rid, [tokens[i]], [0])], []))
    steps[-1] = (steps[-1][0], [rid])
    return steps


def portions(rid: str, tokens: list[int], seed: int, sizes: tuple[int, ...] = (2, 3, 5, 2, 17, 8, 2, 31)) -> list[Step]:
    """Portions of changing size, down to two tokens (and single tokens at the end)."""
    rng = random.Random(seed)
    steps: list[Step] = []
    at, i = 0, 0
    while at < len(tokens):
        n = sizes[i % len(sizes)] if i < len(sizes) else rng.choice([1, 2, 4, 9, 16])
        n = min(n, len(tokens) - at)
        steps.append(([(rid, tokens[at: at + n], list(range(n)))], []))
        at += n
        i += 1
    steps[-1] = (steps[-1][0], [rid])
    return steps


def mixed(requests: dict[str, list[int]], seed: int, max_live: int = 4) -> list[Step]:
    """Up to ``max_live`` requests at a time; each step gives some of them a portion of their
    prompt or a single token, leaves others out, and starts a new request when one ends, so
    that pages are given back and used again."""
    rng = random.Random(seed)
    waiting = list(requests)
    live: dict[str, int] = {}       # id -> tokens fed so far
    steps: list[Step] = []
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        ids = list(live)
        rng.shuffle(ids)
        chosen = ids[: rng.randint(1, len(ids))]
        for rid in sorted(chosen, key=list(requests).index):
            toks, fed = requests[rid], live[rid]
            left = len(toks) - fed
            n = min(left, rng.choice([1, 1, 2, 3, 7, 16, 40]))
            entries.append((rid, toks[fed: fed + n], list(range(n))))
            live[rid] = fed + n
            if live[rid] == len(toks):
                end.append(rid)
        for rid in end:
            del live[rid]
        steps.append((entries, end))
    return steps


def max_live_tokens(steps: list[Step], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    most = 0
    for entries, end in steps:
        for rid, toks, _ in entries:
            held[rid] = held.get(rid, 0) + len(toks)
        most = max(most, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in end:
            held.pop(rid, None)
    return most
