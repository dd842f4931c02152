"""The plain implementation against logits made by the upstream engine's own model code
(``tests/golden/``), and a few properties of its parts."""

from __future__ import annotations

import math
from pathlib import Path

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

import plain_qwen3 as plain
from golden.make_golden import weights_checksum
from tiny_configs import TINIES, write_tiny

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", sorted(TINIES))
def test_plain_matches_upstream_logits(name: str, tmp_path: Path) -> None:
    """The golden file holds upstream's own logits AND the weights they were made with. The
    weights are re-made here from the same seed; should this torch build draw other values, the
    stored ones take their place, so the formulas are always held against upstream's output."""
    with safe_open(str(GOLDEN / f"tiny_{name}.safetensors"), framework="pt", device="cpu") as f:
        ids = f.get_tensor("token_ids").tolist()
        want = f.get_tensor("logits")
        digest = f.metadata()["weights_sha256"]
        stored = {k[2:]: f.get_tensor(k) for k in f.keys() if k.startswith("w.")}
    assert stored, "the golden file holds no weights: make it again with tests/golden/make_golden.py"
    folder = write_tiny(tmp_path, name, torch.float32)
    if weights_checksum(folder) != digest:
        save_file(stored, str(folder / "model.safetensors"))       # same config.json, upstream's weights
        assert weights_checksum(folder) == digest
    got = plain.forward_folder(folder, ids, torch.float32)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


def test_stored_golden_weights_alone_reproduce_upstream_logits(tmp_path: Path) -> None:
    """The fallback of the test above, exercised: the weights stored in the golden file, without
    the random-weights mode."""
    name = "A"
    with safe_open(str(GOLDEN / f"tiny_{name}.safetensors"), framework="pt", device="cpu") as f:
        ids, want = f.get_tensor("token_ids").tolist(), f.get_tensor("logits")
        stored = {k[2:]: f.get_tensor(k) for k in f.keys() if k.startswith("w.")}
    folder = write_tiny(tmp_path, name, torch.float32)
    save_file(stored, str(folder / "model.safetensors"))
    torch.testing.assert_close(plain.forward_folder(folder, ids, torch.float32), want, atol=1e-5, rtol=1e-5)


def test_rms_norm_by_hand() -> None:
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    y = plain.rms_norm(x, w, 0.0)
    r = math.sqrt(12.5)
    torch.testing.assert_close(y, torch.tensor([[3 / r * 2, 4 / r * 0.5]]))


def test_rope_keeps_norm_and_depends_on_relative_position() -> None:
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 16, generator=g)
    k = torch.randn(1, 1, 16, generator=g)

    def dot(pq: int, pk: int) -> float:
        cq, sq = plain.rope_angles(16, 1e4, torch.tensor([pq]))
        ck, sk = plain.rope_angles(16, 1e4, torch.tensor([pk]))
        return float((plain.apply_rope(q, cq, sq) * plain.apply_rope(k, ck, sk)).sum())

    c, s = plain.rope_angles(16, 1e4, torch.tensor([7]))
    torch.testing.assert_close(plain.apply_rope(q, c, s).norm(), q.norm())
    assert abs(dot(5, 2) - dot(105, 102)) < 1e-4


def test_attention_is_causal_and_groups_heads() -> None:
    g = torch.Generator().manual_seed(1)
    q = torch.randn(6, 4, 8, generator=g)
    k = torch.randn(6, 2, 8, generator=g)
    v = torch.randn(6, 2, 8, generator=g)
    full = plain.causal_gqa_attention(q, k, v, 8 ** -0.5)
    part = plain.causal_gqa_attention(q[:4], k[:4], v[:4], 8 ** -0.5)
    torch.testing.assert_close(full[:4], part)            # later tokens change nothing earlier
    v2 = v.clone()
    v2[:, 1] += 1.0                                       # kv head 1 serves query heads 2, 3
    moved = plain.causal_gqa_attention(q, k, v2, 8 ** -0.5)
    torch.testing.assert_close(moved[:, :2], full[:, :2])
    torch.testing.assert_close(moved[:, 2:], full[:, 2:] + 1.0)


def test_window_one_sees_only_itself() -> None:
    g = torch.Generator().manual_seed(2)
    q = torch.randn(5, 2, 8, generator=g)
    k = torch.randn(5, 2, 8, generator=g)
    v = torch.randn(5, 2, 8, generator=g)
    torch.testing.assert_close(plain.causal_gqa_attention(q, k, v, 1.0, window=1), v)
