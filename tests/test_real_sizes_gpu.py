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
from tiny_configs import random_prompt

pytestmark = pytest.mark.gpu

REAL = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 1024,
    "intermediate_size": 3072, "num_hidden_layers": 2, "num_attention_heads": 16, "num_key_value_heads": 8,
    "head_dim": 128, "hidden_act": "silu", "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "max_position_embeddings": 4096, "tie_word_embeddings": True,
}


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
