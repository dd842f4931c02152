"""The path that the benchmark times, checked for its logits: decode steps and prompt portions that
are REPLAYED from CUDA graphs at the Qwen3-0.6B layer widths (2 layers, the real vocabulary), with
programmatic dependent launch on every kernel class, the weight prefetch on a side stream inside
the recording, key ranges merged in clusters, the norms folded into the products, and steps
launched ahead of the tokens.

Every replayed row is held (a) against the plain implementation, with the tolerance of the replay
tests, and (b) against the very same step launched kernel by kernel with programmatic launch off:
a kernel that read something before its wait for the kernels before it, a stale row of a
recording's block-table cache or a wrong padding row would show in (b) at once. Requests leave and
others take their rows and pages between replays. After upstream tests/test_cuda_graphs.py:75-131,
153-189 (graph and eager logits agree; padding rows harm nobody; requests come and go)."""

from __future__ import annotations

import random

import pytest
import torch

import plain_qwen3 as plain
from test_replay_gpu import close_enough
from tiny_configs import REAL_0_6B, random_prompt

pytestmark = pytest.mark.gpu
VOCAB = REAL_0_6B["vocab_size"]
PAGE = 16


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model

    folder = write_random_model(tmp_path_factory.mktemp("real06"), config_from_dict(REAL_0_6B), 11, torch.bfloat16,
                                std_scale=2.0)
    pcfg = plain.read_config(folder)
    return folder, pcfg, plain.read_weights(folder, torch.float32), plain.read_weights(folder, torch.bfloat16)


@torch.inference_mode()
def plain_rows(pcfg, w, tokens: list[int], places: list[int]) -> torch.Tensor:
    """The plain implementation's logits at ``places`` only (a [T, vocab] array of a thousand tokens
    would not fit): its own parts, composed as its ``forward`` composes them."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    cos, sin = plain.rope_angles(pcfg["head_dim"], float(pcfg["rope_theta"]), torch.arange(len(tokens)))
    x = plain.embed(w["model.embed_tokens.weight"], ids)
    for i in range(pcfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = plain.mlp_block(plain.attention_block(x, w, p, pcfg, cos, sin), w, p, pcfg)
    return plain.head(x[torch.as_tensor(places)], w, pcfg)


class Fleet:
    """Requests that decode side by side through one ``ModelRunner`` with recorded steps."""

    def __init__(self, model, buckets, max_context=2048, pages=6000, prefill_graphs=()):
        from tinyserve_b200.cache import CacheManager
        from tinyserve_b200.engine.step import ModelRunner

        self.model = model
        self.cache = CacheManager(model.cache_needs(), page_size=PAGE, num_pages=pages, max_requests=64,
                                  dtype=model.dtype, device=model.device)
        for g in self.cache.groups:
            g.kv.fill_(float("nan"))             # a read outside a request's own tokens shows
        self.runner = ModelRunner(model, self.cache)
        self.runner.record_decode_graphs(max(buckets), max_context, buckets=buckets)
        for t in prefill_graphs:
            self.runner.record_prefill_graph(t, max_context)
        self.tokens: dict[int, list[int]] = {}
        self.caches: dict[int, object] = {}
        self.rng = random.Random(7)
        self.next_id = 0

    def admit(self, length: int) -> int:
        """A new request whose first ``length - 1`` tokens are already in the cache (run kernel by
        kernel, several requests to a step elsewhere; here one at a time)."""
        from tinyserve_b200.engine.step import StepEntry

        rid = self.next_id
        self.next_id += 1
        toks = random_prompt(length, VOCAB, 1000 + rid)
        self.tokens[rid], self.caches[rid] = toks, self.cache.new_request()
        if length > 1:
            self.cache.append(self.caches[rid], length - 1)
            self.runner.step([StepEntry(self.caches[rid], toks[:-1])], [[]])
        return rid

    def leave(self, rid: int) -> None:
        self.cache.free(self.caches.pop(rid))
        del self.tokens[rid]

    def decode(self, order: list[int], eager_too: bool = True) -> tuple[torch.Tensor, torch.Tensor | None]:
        """One decode step of the requests in ``order`` (each feeds its last token): the replayed
        logits and, for comparison, those of the same step launched kernel by kernel without
        programmatic launch (the step rewrites the same cache rows, so running it twice is safe)."""
        from tinyserve_b200.engine.step import StepEntry
        from tinyserve_b200.kernels import ops

        entries = []
        for rid in order:
            self.cache.append(self.caches[rid], 1)
            entries.append(StepEntry(self.caches[rid], [self.tokens[rid][-1]]))
        runner = self.runner
        assert runner.replays(entries)
        steps = runner.num_graph_steps
        got = runner.step(entries).clone()
        assert runner.num_graph_steps == steps + 1
        eager = None
        if eager_too:
            graphs, runner.graphs, runner.tune_launch_overlap = runner.graphs, {}, False
            mask = ops._pdl_mask
            try:
                ops.set_programmatic_launch(0)
                eager = runner.step(entries).clone()
            finally:
                ops.set_programmatic_launch(mask)
                runner.graphs, runner.tune_launch_overlap = graphs, True
        ops.check_device_errors()
        return got, eager

    def grow(self, order: list[int]) -> None:
        for rid in order:
            self.tokens[rid].append(self.rng.randrange(VOCAB))


def same_step(got: torch.Tensor, eager: torch.Tensor, exact: bool, dtype) -> None:
    """A replayed step against the same step launched kernel by kernel. With as many rows as the
    recording has, both run the same kernels on the same data in the same order and must agree bit
    for bit. With fewer live rows than the recording's, the recording still computes all its rows:
    key ranges are cut differently and a library product may pick another kernel for another row
    count, so sums are formed in another order; then the difference must be rounding, a small
    fraction of the logits' own size, where any stale table row or early read would be gross."""
    if exact:
        assert torch.equal(got, eager), f"replayed and eager logits differ by {float((got - eager).abs().max())}"
        return
    rel = float((got - eager).pow(2).mean().sqrt() / eager.pow(2).mean().sqrt())
    assert rel <= (2e-2 if dtype == torch.bfloat16 else 2e-5), f"replayed and eager logits differ by {rel:.2e} of their size"


def check_rows(fleet: Fleet, order: list[int], got: torch.Tensor, eager: torch.Tensor | None, oracle_rows: list[int],
               real, dtype) -> None:
    _, pcfg, w32, w16 = real
    assert not got.isnan().any(), "NaN in replayed logits (a read outside the request's pages?)"
    if eager is not None:
        same_step(got, eager, exact=dtype == torch.bfloat16 and len(order) in fleet.runner.graphs, dtype=dtype)
    for j in oracle_rows:
        toks = fleet.tokens[order[j]]
        want32 = plain_rows(pcfg, w32, toks, [len(toks) - 1])
        want16 = plain_rows(pcfg, w16, toks, [len(toks) - 1]) if dtype == torch.bfloat16 else None
        close_enough(got[j: j + 1].float().cpu(), want32, want16, dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_replayed_decode_steps_match_eager_and_plain(real, dtype) -> None:
    """Batch 64 with contexts from 1 to ~1,100 (the grid of three-warp CTAs), batch 8 at ~1,030
    (five key ranges merged in a cluster, norms folded into the products), batch 12 (the
    two-column-tile skinny variants), batch 40 (library products), batch 1; three steps each, with
    requests leaving and others taking over their rows and pages in between."""
    from tinyserve_b200.model import DecoderModel

    model = DecoderModel.from_folder(real[0], dtype, "cuda")
    fleet = Fleet(model, buckets=[1, 8, 16, 64])
    rng = random.Random(3)
    full = dtype == torch.bfloat16
    plan = [(64, lambda i: 1 + (i * 53) % 1100 if i else 1100), (8, lambda i: 1024 + i), (12, lambda i: 40 + 90 * i),
            (40, lambda i: 3 + 27 * i), (1, lambda i: 700)]
    if not full:
        plan = [(64, lambda i: 1 + (i * 53) % 300 if i else 700), (8, lambda i: 300 + i), (12, lambda i: 40 + 30 * i)]
    live: list[int] = []
    for batch, length in plan:
        # some of the old requests leave, the rest stay (their rows move), new ones fill the batch
        rng.shuffle(live)
        for rid in live[batch // 2:]:
            fleet.leave(rid)
        live = live[: batch // 2]
        live += [fleet.admit(length(i)) for i in range(batch - len(live))]
        rng.shuffle(live)
        for step in range(3):
            got, eager = fleet.decode(live)
            lens = [len(fleet.tokens[r]) for r in live]
            rows = sorted({lens.index(min(lens)), lens.index(max(lens)), 0, len(live) - 1, rng.randrange(len(live))})
            check_rows(fleet, live, got, eager, rows if step != 1 else rows[:1], real, dtype)
            fleet.grow(live)
            if step == 0 and len(live) > 2:
                # one request ends between two replays of the same recording: its row is taken by the last one
                fleet.leave(live.pop(1))
                live.insert(1, live.pop())
    for rid in list(live):
        fleet.leave(rid)
    fleet.cache.check_invariant()
    assert all(g.allocator.num_used == 0 for g in fleet.cache.groups)


def test_replayed_prompt_portions_match_eager_and_plain(real) -> None:
    """Recorded steps of 2,048 and 512 prompt tokens, the second on top of the first one's context,
    then a rest launched kernel by kernel: logits at the end of every portion."""
    from tinyserve_b200.engine.step import StepEntry
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    _, pcfg, w32, w16 = real
    model = DecoderModel.from_folder(real[0], torch.bfloat16, "cuda")
    fleet = Fleet(model, buckets=[1], max_context=4096, pages=600, prefill_graphs=(2048, 512))
    runner, cache = fleet.runner, fleet.cache
    toks = random_prompt(2048 + 512 + 37, VOCAB, 77)
    cuts = [(0, 2048), (2048, 2560), (2560, len(toks))]
    results = {}
    for mode in ("replayed", "eager"):
        req = cache.new_request()
        if mode == "eager":
            saved, runner.prefill_graphs, runner.tune_launch_overlap = runner.prefill_graphs, {}, False
            ops.set_programmatic_launch(0)
        before = runner.num_graph_steps
        rows = []
        for a, b in cuts:
            cache.append(req, b - a)
            rows.append(runner.step([StepEntry(req, toks[a:b])]).clone())
        assert runner.num_graph_steps - before == (2 if mode == "replayed" else 0)
        if mode == "eager":
            runner.prefill_graphs, runner.tune_launch_overlap = saved, True
            ops.set_programmatic_launch(ops.PREFILL_PDL_MASK)
        ops.check_device_errors()
        cache.free(req)
        results[mode] = torch.cat(rows)
    same_step(results["replayed"], results["eager"], exact=True, dtype=torch.bfloat16)
    places = [b - 1 for _, b in cuts]
    close_enough(results["replayed"].float().cpu(), plain_rows(pcfg, w32, toks, places),
                 plain_rows(pcfg, w16, toks, places), torch.bfloat16)


@pytest.mark.parametrize("ahead", [True, False])
def test_engine_with_recorded_steps_launched_ahead(real, ahead) -> None:
    """Through ``Engine``: eight requests of different lengths, recorded decode steps (launched ahead
    of their tokens or not), forty tokens, one request ending on an end token half-way. Every
    logits row the engine sampled from is held against the plain implementation on the request's
    final token sequence."""
    from tinyserve_b200 import LLM

    _, pcfg, w32, w16 = real
    prompts = [random_prompt(n, VOCAB, 300 + n) for n in (1000, 3, 517, 64, 65, 1023, 250, 130)]

    def run(eos_for_3: frozenset[int]):
        llm = LLM.from_folder(real[0], dtype="bfloat16", page_size=PAGE, num_pages=1024, max_num_seqs=8,
                              max_batch_tokens=2048, chunked_prefill=True, decode_graphs=True, run_ahead=ahead,
                              graph_max_context=2048, record_logits=True)
        e = llm.engine
        ids = [e.add_request(p, 40, eos_ids=eos_for_3 if i == 3 else frozenset()) for i, p in enumerate(prompts)]
        while e.has_work():
            e.step()
        assert all(g.allocator.num_used == 0 for g in llm.cache.groups)
        return e, ids

    e, ids = run(frozenset())
    first = e.requests[ids[3]].output
    stop = first[20]
    e, ids = run(frozenset({stop}))
    outs = [e.requests[i].output for i in ids]
    assert outs[3][-1] == stop and len(outs[3]) == first.index(stop) + 1 <= 21
    assert all(len(o) == 40 for j, o in enumerate(outs) if j != 3)
    assert e.runner.num_graph_steps > 30 and (e.num_steps_ahead > 20) == ahead
    by_req: dict[int, dict[int, torch.Tensor]] = {}
    for rid, pos, row in e.logits_log:
        by_req.setdefault(rid, {})[pos] = row
    for j, rid in enumerate(ids):
        seq = prompts[j] + outs[j]
        # every position from the prompt's last token on was sampled from once (a step run ahead of an
        # end token adds one more row, past the end, which is ignored)
        places = list(range(len(prompts[j]) - 1, len(seq) - 1))
        assert set(places) <= set(by_req[rid])
        rows = torch.stack([by_req[rid][p] for p in places]).float().cpu()
        assert [int(r.argmax()) for r in rows] == outs[j]
        pick = sorted({0, 1, len(places) // 2, len(places) - 1})
        at = [places[i] for i in pick]
        close_enough(rows[pick], plain_rows(pcfg, w32, seq, at), plain_rows(pcfg, w16, seq, at), torch.bfloat16)


def test_a_row_at_sixteen_and_at_seventeen_rows(real) -> None:
    """Up to 16 rows the RMSNorm is folded into the products around it (the product reads a bf16 copy
    of the stream, multiplies by the norm weight and scales the finished sums by rstd), from 17 rows
    on it is a kernel of its own (norm, cast, times weight, as upstream rounds): the rounding points
    differ, so a request's logits depend, within bf16 rounding, on the batch-size bucket it runs
    in. Both must be as close to the oracle as the plain implementation's own bf16 run, and their
    difference is bounded by that run's error."""
    from tinyserve_b200.engine.step import StepEntry
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    _, pcfg, w32, w16 = real
    model = DecoderModel.from_folder(real[0], torch.bfloat16, "cuda")
    fleet = Fleet(model, buckets=[16, 32])
    ids = [fleet.admit(40 + 7 * i) for i in range(17)]
    entries = []
    for rid in ids:
        fleet.cache.append(fleet.caches[rid], 1)
        entries.append(StepEntry(fleet.caches[rid], [fleet.tokens[rid][-1]]))
    normed = []
    real_normed = ops.gemm_normed
    ops.gemm_normed = lambda *a, **k: (normed.append(a[0].shape[0]), real_normed(*a, **k))[1]
    try:
        saved, fleet.runner.graphs = fleet.runner.graphs, {}      # kernel by kernel, so that the calls can be seen
        at16 = fleet.runner.step(entries[:16]).float().cpu()
        seen16 = list(normed)
        at17 = fleet.runner.step(entries).float().cpu()
        fleet.runner.graphs = saved
    finally:
        ops.gemm_normed = real_normed
    assert seen16 and len(normed) == len(seen16), "16 rows fold the norms into the products, 17 rows do not"
    for j, rid in enumerate(ids[:16:2]):
        j *= 2
        toks = fleet.tokens[rid]
        want32, want16 = plain_rows(pcfg, w32, toks, [len(toks) - 1]), plain_rows(pcfg, w16, toks, [len(toks) - 1])
        close_enough(at16[j: j + 1], want32, want16, torch.bfloat16)
        close_enough(at17[j: j + 1], want32, want16, torch.bfloat16)
        between = float((at16[j] - at17[j]).pow(2).mean().sqrt())
        assert between <= 1.25 * float((want16 - want32).pow(2).mean().sqrt()) + 1e-3
