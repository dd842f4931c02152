"""Loading safetensors by name: one clear error; merged and split forms; tied heads; the
random-weights mode."""

from __future__ import annotations

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import load_file, save_file

import tinyserve_b200.architectures  # noqa: F401
from tinyserve_b200.config import config_from_dict
from tinyserve_b200.model import DecoderModel, build_parts
from tinyserve_b200.weights import WeightLoadError, checkpoint_names, load_tensors, merge_specs, write_random_model
from tiny_configs import TINY_A, TINY_B, write_tiny


def test_random_folder_has_the_checkpoint_names(tmp_path) -> None:
    folder = write_tiny(tmp_path, "B", torch.bfloat16)
    cfg = config_from_dict(TINY_B)
    names = checkpoint_names(merge_specs(build_parts(cfg.to_spec()).tensor_specs()))
    assert len(names) == 11 * 3 + 3                       # 11 per layer + embedding + final norm + head
    with safe_open(str(folder / "model.safetensors"), framework="pt") as f:
        assert set(f.keys()) == set(names)
        assert f.get_tensor("model.layers.0.self_attn.q_proj.weight").shape == (128, 80)
        assert f.get_tensor("model.layers.0.self_attn.q_proj.weight").dtype == torch.bfloat16
    assert load_config_equal(folder, cfg)


def load_config_equal(folder, cfg) -> bool:
    from tinyserve_b200.config import load_config

    return load_config(folder) == cfg


def test_same_seed_same_weights_other_seed_other_weights(tmp_path) -> None:
    cfg = config_from_dict(TINY_A)
    a = load_file(str(write_random_model(tmp_path / "a", cfg, 3, torch.float32) / "model.safetensors"))
    b = load_file(str(write_random_model(tmp_path / "b", cfg, 3, torch.float32) / "model.safetensors"))
    c = load_file(str(write_random_model(tmp_path / "c", cfg, 4, torch.float32) / "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    norm = a["model.layers.0.input_layernorm.weight"]
    assert abs(float(norm.mean()) - 1.0) < 0.05 and float(a["model.embed_tokens.weight"].std()) < 0.03


def test_loads_split_and_merged_forms_alike(tmp_path) -> None:
    folder = write_tiny(tmp_path / "split", "A", torch.float32)
    m1 = DecoderModel.from_folder(folder, torch.float32, "cpu")
    t = load_file(str(folder / "model.safetensors"))
    merged = {}
    for k, v in t.items():
        if "q_proj" in k:
            p = k.replace("q_proj.weight", "")
            merged[p + "qkv_proj.weight"] = torch.cat([t[p + "q_proj.weight"], t[p + "k_proj.weight"], t[p + "v_proj.weight"]])
        elif "gate_proj" in k:
            p = k.replace("gate_proj.weight", "")
            merged[p + "gate_up_proj.weight"] = torch.cat([t[p + "gate_proj.weight"], t[p + "up_proj.weight"]])
        elif not any(s in k for s in ("k_proj", "v_proj", "up_proj")):
            merged[k] = v
    (tmp_path / "merged").mkdir()
    save_file(merged, str(tmp_path / "merged" / "model.safetensors"))
    (tmp_path / "merged" / "config.json").write_text((folder / "config.json").read_text())
    m2 = DecoderModel.from_folder(tmp_path / "merged", torch.float32, "cpu")
    assert all(torch.equal(m1.tensors[k], m2.tensors[k]) for k in m1.tensors)
    assert m1.tensors["model.layers.1.self_attn.qkv_proj.weight"].shape == (64 + 2 * 32, 64)


def test_sharded_folder_and_tied_copy_of_the_head(tmp_path) -> None:
    folder = write_tiny(tmp_path, "A", torch.float32)
    t = load_file(str(folder / "model.safetensors"))
    (folder / "model.safetensors").unlink()
    names = sorted(t)
    save_file({k: t[k] for k in names[::2]}, str(folder / "model-00001-of-00002.safetensors"))
    rest = {k: t[k] for k in names[1::2]}
    rest["lm_head.weight"] = t["model.embed_tokens.weight"].clone()     # a tied checkpoint may ship it
    save_file(rest, str(folder / "model-00002-of-00002.safetensors"))
    m = DecoderModel.from_folder(folder, torch.float32, "cpu")
    assert m.parts.head.weight is m.parts.embedding.table               # tied: the same tensor


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path) -> None:
    folder = write_tiny(tmp_path, "B", torch.float32)
    t = load_file(str(folder / "model.safetensors"))
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    t["model.layers.2.self_attn.o_proj.weight"] = torch.zeros(80, 64)
    t["lm_head.weight"] = torch.zeros(384, 81)
    save_file(t, str(folder / "model.safetensors"))
    with pytest.raises(WeightLoadError) as e:
        DecoderModel.from_folder(folder, torch.float32, "cpu")
    msg = str(e.value)
    assert "2 missing" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "1 unexpected" in msg and "rotary_emb.inv_freq" in msg
    assert "2 with a wrong shape" in msg and "o_proj.weight: shape (80, 64), expected (80, 128)" in msg
    assert "lm_head.weight: shape (384, 81)" in msg


def test_dtype_rules(tmp_path) -> None:
    folder = write_tiny(tmp_path, "A", torch.float32)
    m = DecoderModel.from_folder(folder, torch.bfloat16, "cpu")
    assert all(v.dtype == torch.bfloat16 for v in m.tensors.values())
    from tinyserve_b200.parts.base import TensorSpec

    save_file({"w": torch.ones(4, 4), "s": torch.ones(3), "t": torch.arange(5, dtype=torch.int64)},
              str(tmp_path / "x.safetensors"))
    (tmp_path / "model.safetensors").unlink()
    got = load_tensors(tmp_path, [TensorSpec("w", (4, 4)), TensorSpec("s", (3,), keep_32bit=True),
                                  TensorSpec("t", (5,), integer=True)], torch.bfloat16, "cpu")
    assert got["w"].dtype == torch.bfloat16 and got["s"].dtype == torch.float32 and got["t"].dtype == torch.int32


def test_no_files_and_non_finite(tmp_path) -> None:
    with pytest.raises(WeightLoadError, match="no \\*.safetensors"):
        load_tensors(tmp_path, [], torch.float32, "cpu")
    folder = write_tiny(tmp_path, "A", torch.float32)
    t = load_file(str(folder / "model.safetensors"))
    t["model.norm.weight"][3] = float("inf")
    save_file(t, str(folder / "model.safetensors"))
    with pytest.raises(WeightLoadError, match="inf or nan"):
        DecoderModel.from_folder(folder, torch.float32, "cpu")
