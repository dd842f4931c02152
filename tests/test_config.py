"""Typed configuration and the architecture registry."""

from __future__ import annotations

import json

import pytest

import tinyserve_b200.architectures  # noqa: F401
from tinyserve_b200.architectures.qwen3 import Qwen3Config
from tinyserve_b200.config import (ModelConfig, UnsupportedConfigError, config_from_dict,
                                   known_architectures, load_config, register_architecture)
from tiny_configs import TINY_A, TINY_B


def test_reads_the_architectures_own_keys() -> None:
    c = config_from_dict(TINY_B)
    assert isinstance(c, Qwen3Config)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_layers) == (384, 80, 176, 3)
    assert (c.num_heads, c.num_kv_heads, c.head_dim) == (4, 1, 32)
    assert c.q_size == 128 and c.kv_size == 32           # q width need not equal the hidden width
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 1e6 and c.tie_word_embeddings is False


def test_defaults_follow_upstream() -> None:
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "tie_word_embeddings", "rope_theta")}
    d["rope_parameters"] = {"rope_theta": 5e5, "rope_type": "default"}
    c = config_from_dict(d)
    assert c.head_dim == 64 // 4 and c.tie_word_embeddings is False and c.rope_theta == 5e5


@pytest.mark.parametrize("change,word", [
    ({"architectures": ["LlamaForCausalLM"]}, "unknown architecture"),
    ({"architectures": []}, "architectures"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"rope_parameters": {"rope_type": "yarn", "rope_theta": 1e6}}, "rope_parameters"),
    ({"use_sliding_window": True}, "sliding"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"rope_theta": None}, "rope_theta"),
    ({"head_dim": 15}, "even"),
])
def test_rejections(change, word) -> None:
    with pytest.raises(UnsupportedConfigError, match=word):
        config_from_dict({**TINY_A, **change})


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "rms_norm_eps",
                                 "max_position_embeddings"])
def test_required_keys(key) -> None:
    d = dict(TINY_A)
    del d[key]
    with pytest.raises((UnsupportedConfigError, KeyError)):
        config_from_dict(d)


def test_round_trip_and_spec(tmp_path) -> None:
    c = config_from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(tmp_path) == c
    spec = c.to_spec()
    assert len(spec.layers) == 3 and [x.layer for x in spec.order] == [0, 1, 2]
    assert set(spec.layers[0].parts) == {"mixer", "feed_forward", "mixer_norm", "feed_forward_norm"}
    a = spec.layers[0].parts["mixer"].args
    assert a["scale"] == 32 ** -0.5 and a["qk_norm"] and a["qk_norm_eps"] == 1e-5 and a["window"] is None
    assert spec.layers[0].position.args["theta"] == 1e6
    assert spec.head.args["tied"] is False and spec.head.args["name"] == "lm_head.weight"
    assert config_from_dict(TINY_A).to_spec().head.args["name"] == "model.embed_tokens.weight"


def test_registry_takes_another_architecture() -> None:
    class Other(ModelConfig):
        architecture = "OtherForCausalLM"

        @classmethod
        def from_dict(cls, d):
            return cls()

    register_architecture("OtherForCausalLM", Other)
    assert "OtherForCausalLM" in known_architectures()
    assert isinstance(config_from_dict({"architectures": ["OtherForCausalLM"]}), Other)
    with pytest.raises(ValueError):
        register_architecture("OtherForCausalLM", Qwen3Config)


def test_a_head_size_the_kernels_do_not_take_is_refused_when_the_model_is_built() -> None:
    """head_dim 40 is a legal Qwen3 config.json (even, so rotary pairs exist), but the attention
    kernels take head sizes in steps of 16 up to 256: the parts say so when they are built, before
    any weight is loaded or any cache allocated."""
    from tinyserve_b200.model import build_parts

    c = config_from_dict({**TINY_A, "head_dim": 40})
    with pytest.raises(ValueError, match="head_dim=40.*steps of 16"):
        build_parts(c.to_spec())
    build_parts(config_from_dict({**TINY_A, "head_dim": 48}).to_spec())
