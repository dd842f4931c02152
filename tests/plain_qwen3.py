"""A plain, slow implementation of the dense Qwen3 decoder, written from the formulas of the
upstream engine (princemittalr/tinyserve). Whole sequences, no cache, no batching, PyTorch
on the CPU, one function per part; it shares no code with ``tinyserve_b200``. It reads
``config.json`` and ``*.safetensors`` itself. ``tests/golden/`` holds logits that the
upstream model code itself produced for two tiny random models; ``test_plain.py`` checks
this file against them.

Rounding: every function computes in 32-bit where upstream does and rounds to the working
dtype where upstream does, so ``dtype=torch.bfloat16`` follows upstream's half-precision
contract and ``dtype=torch.float32`` is exact 32-bit.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors import safe_open


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = cast(x32 * rsqrt(mean(x32^2) + eps)) * weight  -- src/tinyserve/layers.py:35-38."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return xf.to(x.dtype) * weight


def rope_angles(head_dim: int, theta: float, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """inv_freq = theta^(-2i/D) and angle = pos * inv_freq in float64; cos, sin rounded to
    float32, laid out [T, D/2]  -- src/tinyserve/layers.py:61-65."""
    two_i = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv_freq = theta ** (-two_i / head_dim)
    angles = torch.outer(positions.to(torch.float64), inv_freq)
    return angles.cos().float(), angles.sin().float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing (i, i + D/2) in 32-bit, cast once  -- src/tinyserve/layers.py:84-91.
    x is [T, H, D]; cos/sin are [T, D/2]."""
    half = x.shape[-1] // 2
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                         window: int | None = None) -> torch.Tensor:
    """softmax(scale * q k^T + causal mask) v for one sequence, in 32-bit, cast to q's dtype;
    query head h reads kv head h // (Hq / Hkv)  -- src/tinyserve/attention.py:40-59. The
    optional window (keys j with i - window < j <= i) is not in upstream; it serves the
    tests of windowed page groups."""
    t, hq, _ = q.shape
    group = hq // k.shape[1]
    kf = k.float().repeat_interleave(group, dim=1)
    vf = v.float().repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q.float(), kf) * scale
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    hidden = j > i
    if window is not None:
        hidden = hidden | (j <= i - window)
    scores = scores.masked_fill(hidden, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", probs, vf).to(q.dtype)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x W^T, W stored [out, in], no bias  -- src/tinyserve/model.py:156,173,178-179."""
    return torch.nn.functional.linear(x, w)


def swiglu(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x))  -- src/tinyserve/layers.py:94-115."""
    return linear(torch.nn.functional.silu(linear(x, gate_w)) * linear(x, up_w), down_w)


def embed(table: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
    """Row gather, no scaling  -- src/tinyserve/model.py:192."""
    return table[token_ids]


def attention_block(x: torch.Tensor, w: dict[str, torch.Tensor], p: str, cfg: dict, cos, sin,
                    window: int | None = None) -> torch.Tensor:
    """Pre-norm attention with per-head q/k RMSNorm before the rotation and a residual add
    -- src/tinyserve/model.py:154-173."""
    t = x.shape[0]
    hq, hkv, d, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = linear(h, w[p + "self_attn.q_proj.weight"]).view(t, hq, d)
    k = linear(h, w[p + "self_attn.k_proj.weight"]).view(t, hkv, d)
    v = linear(h, w[p + "self_attn.v_proj.weight"]).view(t, hkv, d)
    q = rms_norm(q, w[p + "self_attn.q_norm.weight"], eps)
    k = rms_norm(k, w[p + "self_attn.k_norm.weight"], eps)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    a = causal_gqa_attention(q, k, v, d ** -0.5, window)
    return x + linear(a.reshape(t, hq * d), w[p + "self_attn.o_proj.weight"])


def mlp_block(x: torch.Tensor, w: dict[str, torch.Tensor], p: str, cfg: dict) -> torch.Tensor:
    """Pre-norm SwiGLU with a residual add  -- src/tinyserve/model.py:176-179."""
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    return x + swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])


def head(x: torch.Tensor, w: dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """Final norm, then float32(x W_head^T); W_head is the embedding table when tied
    -- src/tinyserve/model.py:129-130,199,208."""
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    table = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, table).float()


def read_config(model_dir: str | Path) -> dict:
    """The keys upstream reads, with its defaults  -- src/tinyserve/config.py:54-73."""
    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    cfg = dict(cfg)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    if cfg.get("rope_theta") is None:
        cfg["rope_theta"] = cfg["rope_parameters"]["rope_theta"]
    return cfg


def read_weights(model_dir: str | Path, dtype: torch.dtype) -> dict[str, torch.Tensor]:
    """Every tensor of every *.safetensors file, cast to dtype  -- src/tinyserve/weights.py:62-99."""
    out: dict[str, torch.Tensor] = {}
    for file in sorted(Path(model_dir).glob("*.safetensors")):
        with safe_open(str(file), framework="pt", device="cpu") as f:
            for name in f.keys():
                out[name] = f.get_tensor(name).to(dtype)
    return out


@torch.inference_mode()
def forward(cfg: dict, w: dict[str, torch.Tensor], token_ids: list[int] | torch.Tensor) -> torch.Tensor:
    """[T] token ids of one sequence -> [T, vocab] float32 logits, no cache
    -- src/tinyserve/model.py:181-222."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    cos, sin = rope_angles(cfg["head_dim"], float(cfg["rope_theta"]), positions)
    x = embed(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = attention_block(x, w, p, cfg, cos, sin)
        x = mlp_block(x, w, p, cfg)
    return head(x, w, cfg)


def forward_folder(model_dir: str | Path, token_ids, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return forward(read_config(model_dir), read_weights(model_dir, dtype), token_ids)


def greedy(cfg: dict, w: dict[str, torch.Tensor], prompt: list[int], max_new_tokens: int) -> list[int]:
    """Re-run the whole sequence for every token  -- src/tinyserve/model.py:359-376."""
    ids = list(prompt)
    new: list[int] = []
    for _ in range(max_new_tokens):
        nxt = int(forward(cfg, w, ids)[-1].argmax())
        new.append(nxt)
        ids.append(nxt)
    return new
