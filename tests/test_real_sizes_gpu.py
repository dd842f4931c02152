"""The Qwen3-0.6B layer sizes (hidden 1024, 16/8 heads of 128, intermediate 3072, the real
vocabulary of 151,936, tied embeddings) with two layers and random weights: float32 logits equal
the plain implementation's under whole, tail-decoded and chunked feeding; bfloat16 stays within
the plain implementation's own bfloat16 error. These are the sizes at which the tensor-core
kernels (skinny product, tcgen05 product, tensor-core attention) take over from the generic ones."""

from __future__ import annotations

import pytest
import torch

import plain_qwen3 as plain
import replay_cases as cases
from test_replay_gpu import check, run_steps
from tiny_configs import REAL_0_6B as REAL, REAL_8B, random_prompt

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model

    folder = write_random_model(tmp_path_factory.mktemp("real"), config_from_dict(REAL), 3, torch.bfloat16, std_scale=2.0)
    reqs = {"a": random_prompt(150, 151936, 1), "b": random_prompt(37, 151936, 2)}
    pcfg = plain.read_config(folder)
    w32, w16 = plain.read_weights(folder, torch.float32), plain.read_weights(folder, torch.bfloat16)
    want = ({r: plain.forward(pcfg, w32, t) for r, t in reqs.items()},
            {r: plain.forward(pcfg, w16, t) for r, t in reqs.items()})
    return folder, reqs, want


@pytest.mark.parametrize("dtype,variant", [(torch.float32, "default"), (torch.bfloat16, "default"),
                                           (torch.bfloat16, "separate_rope"), (torch.bfloat16, "separate_norms")])
def test_real_layer_sizes_under_every_cut(real, dtype, variant, monkeypatch) -> None:
    """By default steps of decode tokens alone take the fused q/k-norm + rotation + cache write +
    attention kernel and, for a few bf16 rows, fold the RMSNorms into the products around them.
    ``separate_rope``: the q/k-norm, rotation and cache write run as a kernel of their own before
    the attention kernel. ``separate_norms``: the RMSNorms run as kernels of their own."""
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    fused_norm_calls = []
    if variant == "separate_norms":
        monkeypatch.setattr(ops, "FUSE_STREAM_NORM", False)
    else:
        normed = ops.gemm_normed
        monkeypatch.setattr(ops, "gemm_normed", lambda *a, **k: (fused_norm_calls.append(1), normed(*a, **k))[1])
    calls = []
    fused = ops.decode_attention_fused
    monkeypatch.setattr(ops, "decode_attention_fused", lambda *a, **k: (calls.append(1), fused(*a, **k))[1])
    if variant == "separate_rope":
        monkeypatch.setattr(ops, "FUSED_DECODE_MAX_ROWS", 0)
    folder, reqs, want = real
    model = DecoderModel.from_folder(folder, dtype, "cuda")
    plans = [cases.mixed(reqs, 5)]
    for rid, toks in reqs.items():
        plans += [cases.whole(rid, toks), cases.tail_decoded(rid, toks, 32), cases.portions(rid, toks, 2)]
    for steps in plans:
        got = run_steps(model, 16, steps, cases.max_live_tokens(steps))
        check(got, want, {r: reqs[r] for r in got}, dtype)
    if dtype == torch.bfloat16:
        assert bool(calls) == (variant != "separate_rope")
    if dtype == torch.bfloat16:
        assert bool(fused_norm_calls) == (variant != "separate_norms")


@pytest.fixture(scope="module")
def real_8b(tmp_path_factory):
    """The Qwen3-8B widths (hidden 4096, 32 / 8 heads of 128, intermediate 12,288, the real
    vocabulary, untied head), one layer."""
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model

    folder = write_random_model(tmp_path_factory.mktemp("real8b"), config_from_dict(REAL_8B), 4, torch.bfloat16, std_scale=1.0)
    reqs = {"a": random_prompt(150, 151936, 5), "b": random_prompt(37, 151936, 6)}
    pcfg = plain.read_config(folder)
    w32, w16 = plain.read_weights(folder, torch.float32), plain.read_weights(folder, torch.bfloat16)
    want = ({r: plain.forward(pcfg, w32, t) for r, t in reqs.items()},
            {r: plain.forward(pcfg, w16, t) for r, t in reqs.items()})
    return folder, reqs, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_8b_layer_widths_under_every_cut(real_8b, dtype, monkeypatch) -> None:
    """At these widths another set of kernels runs than at the 0.6B ones: the decode rows' products
    leave the skinny kernel for the library (the matrices are larger than it is tuned for), the
    norms run as kernels of their own (the stream is wider than the fusion takes), products of a
    hundred-odd rows go to the library too (their tiles would not fill the machine), and four
    query heads share a kv head. The test also checks that those are the kernels that ran."""
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    seen = {"mm": 0, "tcgen05": 0, "norm": 0, "normed": 0, "skinny": 0, "fused_attention": 0}

    def counted(name, fn):
        def wrapper(*a, **k):
            seen[name] += 1
            return fn(*a, **k)
        return wrapper

    monkeypatch.setattr(ops.torch, "mm", counted("mm", torch.mm))
    for name, attr in (("tcgen05", "gemm_tcgen05"), ("norm", "add_rms_norm"), ("normed", "gemm_normed"),
                       ("skinny", "gemm_skinny"), ("fused_attention", "decode_attention_fused")):
        monkeypatch.setattr(ops, attr, counted(name, getattr(ops, attr)))
    folder, reqs, want = real_8b
    model = DecoderModel.from_folder(folder, dtype, "cuda")
    plans = [cases.mixed(reqs, 5)]
    for rid, toks in reqs.items():
        plans += [cases.whole(rid, toks), cases.tail_decoded(rid, toks, 32), cases.portions(rid, toks, 2)]
    for steps in plans:
        got = run_steps(model, 16, steps, cases.max_live_tokens(steps))
        check(got, want, {r: reqs[r] for r in got}, dtype)
    ops.check_device_errors()
    assert seen["norm"] > 0 and seen["normed"] == 0
    if dtype == torch.bfloat16:
        # (the only tcgen05 product here is the output head over a whole prompt's 150 rows: 1,188 tiles)
        assert seen["mm"] > 100 and seen["tcgen05"] <= 2 and seen["fused_attention"] > 0
        assert seen["skinny"] > 0          # the output head of a few rows still streams through the skinny kernel
    else:
        assert seen["mm"] == 0 and seen["tcgen05"] == 0


def test_8b_layer_widths_long_prompt_on_the_tcgen05_products(real_8b, monkeypatch) -> None:
    """A prompt of 1,100 tokens at the 8B widths: nine row tiles, so the output, gate/up (with the
    activation in its epilogue) and down products fill the machine and run on this engine's tcgen05
    kernel, the prompt's attention on the tcgen05 attention kernel; then three tokens decoded one by
    one. Logits at the tile edges and at the end against the plain implementation."""
    from test_recorded_steps_gpu import plain_rows
    from test_replay_gpu import close_enough
    from tinyserve_b200.engine.replay import Replayer
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.model import DecoderModel

    seen = {"tcgen05": 0, "swiglu": 0}
    plain_gemm, fused = ops.gemm_tcgen05, ops._fn("ts_gemm_tcgen05_swiglu")
    monkeypatch.setattr(ops, "gemm_tcgen05", lambda *a, **k: (seen.__setitem__("tcgen05", seen["tcgen05"] + 1), plain_gemm(*a, **k))[1])
    monkeypatch.setitem(ops._fns, "ts_gemm_tcgen05_swiglu",
                        lambda *a: (seen.__setitem__("swiglu", seen["swiglu"] + 1), fused(*a))[1])
    folder = real_8b[0]
    pcfg = plain.read_config(folder)
    w32, w16 = plain.read_weights(folder, torch.float32), plain.read_weights(folder, torch.bfloat16)
    toks = random_prompt(1103, 151936, 9)
    rep = Replayer(DecoderModel.from_folder(folder, torch.bfloat16, "cuda"), 1152, page_size=16)
    for g in rep.cache.groups:
        g.kv.fill_(float("nan"))
    places = [0, 127, 128, 1023, 1099]
    got = [rep.run_step([("a", toks[:1100], places)]).float().cpu()]
    for i in range(1100, 1103):
        got.append(rep.run_step([("a", [toks[i]], [0])], ["a"] if i == 1102 else []).float().cpu())
    ops.check_device_errors()
    assert seen["tcgen05"] >= 2 and seen["swiglu"] >= 1
    rows = torch.cat(got)
    assert not rows.isnan().any()
    at = places + [1100, 1101, 1102]
    close_enough(rows, plain_rows(pcfg, w32, toks, at), plain_rows(pcfg, w16, toks, at), torch.bfloat16)
