"""The framework takes parts and architectures it has never seen, without a change to its
files: a toy mixer with state of its own, a toy feed-forward that routes every token to one
of three experts, a toy position encoding with its own angles (all three defined HERE), a
layer with a sliding window, a partial interleaved rotation, a layer that runs twice and a
call that reads another call's cache are registered, built from a config.json, loaded, and
replayed under every cut of the work against a plain implementation of the same toy. (The toy
is no model of anyone's.)"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

import pytest
import torch

import plain_qwen3 as plain
import replay_cases as cases
from tiny_configs import random_prompt

from tinyserve_b200.config import LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec, register_architecture
from tinyserve_b200.parts import (
    FeedForward, Mixer, PositionEncoding, StateNeed, TensorSpec, register_feed_forward, register_mixer,
    register_position_encoding,
)
from tinyserve_b200.parts.rope import RotaryTables

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------- the toy mixer
class ToyEMAMixer(Mixer):
    """s_t = decay * s_{t-1} + x_t Win^T;  y_t = s_t Wout^T, with s in a state slot per request."""

    def __init__(self, prefix: str, hidden_size: int) -> None:
        self.prefix, self.h = prefix, hidden_size

    def cache_need(self) -> StateNeed:
        return StateNeed((self.h,), torch.float32)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p = prefix + self.prefix
        return [TensorSpec(p + "in.weight", (self.h, self.h)), TensorSpec(p + "out.weight", (self.h, self.h)),
                TensorSpec(p + "decay_logit", (self.h,), std=1.0, keep_32bit=True)]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p = prefix + self.prefix
        self.w_in, self.w_out = tensors[p + "in.weight"], tensors[p + "out.weight"]
        self.decay = torch.sigmoid(tensors[p + "decay_logit"].float())

    def forward(self, x, ctx, cache, writes_cache, position):
        out = ctx.arena.take((x.shape[0], self.h), ctx.dtype)
        u = (x.float() @ self.w_in.float().t())
        row = 0
        for n, slot in zip(ctx.query_lens, ctx.state_slots_host):
            s = cache.state[slot]
            ys = []
            for i in range(n):
                s = self.decay * s + u[row + i]
                ys.append(s)
            cache.state[slot] = s
            out[row: row + n] = (torch.stack(ys) @ self.w_out.float().t()).to(ctx.dtype)
            row += n
        return out


# ------------------------------------------------- the toy feed-forward with routing
class ToyRoutedFFN(FeedForward):
    """Every token goes to the one expert with the largest router logit (32-bit) and gets
    p_e * W2_e relu(W1_e x), p the softmax of the router logits."""

    def __init__(self, prefix: str, hidden_size: int, expert_size: int, num_experts: int) -> None:
        self.prefix, self.h, self.f, self.e = prefix, hidden_size, expert_size, num_experts

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p = prefix + self.prefix
        return [TensorSpec(p + "router.weight", (self.e, self.h), std=0.05, keep_32bit=True),
                TensorSpec(p + "w1", (self.e * self.f, self.h)), TensorSpec(p + "w2", (self.e * self.h, self.f))]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p = prefix + self.prefix
        self.router = tensors[p + "router.weight"].float()
        self.w1 = tensors[p + "w1"].view(self.e, self.f, self.h)
        self.w2 = tensors[p + "w2"].view(self.e, self.h, self.f)

    def forward(self, x, ctx):
        logits = x.float() @ self.router.t()
        prob, expert = torch.softmax(logits, dim=-1).max(dim=-1)
        out = ctx.arena.take(tuple(x.shape), ctx.dtype)
        for e in range(self.e):
            rows = (expert == e).nonzero().flatten()
            hid = torch.relu(x[rows] @ self.w1[e].t())
            out[rows] = ((hid @ self.w2[e].t()).float() * prob[rows, None]).to(ctx.dtype)
        return out


# ------------------------------------------------------ the toy position encoding
class ToyLinearRotary(PositionEncoding):
    """Rotation angles position * (i + 1) * step: frequencies in a line, not in a geometric row.
    Hands the mixer the same kind of tables as the built-in encoding, made its own way."""

    def __init__(self, rotary_dim: int, step: float) -> None:
        self.rotary_dim, self.step = rotary_dim, step

    def key(self) -> Any:
        return ("toy_linear", self.rotary_dim, self.step)

    def prepare(self, ctx) -> RotaryTables:
        half = self.rotary_dim // 2
        freq = torch.arange(1, half + 1, dtype=torch.float64, device=ctx.positions.device) * self.step
        angle = ctx.positions.double()[:, None] * freq
        cos = ctx.arena.take_step((ctx.num_tokens, half), torch.float32)
        sin = ctx.arena.take_step((ctx.num_tokens, half), torch.float32)
        cos.copy_(angle.cos())
        sin.copy_(angle.sin())
        return RotaryTables(cos, sin, self.rotary_dim, False)


# ------------------------------------------------------------ the toy architecture
@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    vocab_size: int = 97
    hidden_size: int = 48
    window: int = 6
    eps: float = 1e-5
    architecture = "ToyHybridForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(d["vocab_size"], d["hidden_size"], d["window"], d["eps"])

    def to_dict(self):
        return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "window": self.window, "eps": self.eps}

    def to_spec(self) -> ModelSpec:
        h = self.hidden_size

        def norm(name):
            return PartSpec("rms_norm", {"name": name, "size": h, "eps": self.eps})

        def ffn(i):
            return PartSpec("swiglu", {"prefix": "mlp.", "hidden_size": h, "intermediate_size": i})

        l0 = LayerSpec("layers.0.", "prenorm",
                       PartSpec("gqa_attention", {"prefix": "attn.", "hidden_size": h, "num_heads": 4, "num_kv_heads": 2,
                                                  "head_dim": 16, "scale": 0.25, "window": self.window}),
                       ffn(64), norm("n1.weight"), norm("n2.weight"),
                       PartSpec("toy_linear_rotary", {"rotary_dim": 16, "step": 0.013}))
        l1 = LayerSpec("layers.1.", "prenorm", PartSpec("toy_ema", {"prefix": "ema.", "hidden_size": h}),
                       PartSpec("toy_routed", {"prefix": "moe.", "hidden_size": h, "expert_size": 40, "num_experts": 3}),
                       norm("n1.weight"), norm("n2.weight"), None)
        l2 = LayerSpec("layers.2.", "prenorm",
                       PartSpec("gqa_attention", {"prefix": "attn.", "hidden_size": h, "num_heads": 2, "num_kv_heads": 2,
                                                  "head_dim": 32, "scale": 32 ** -0.5, "qk_norm": True,
                                                  "qk_norm_eps": self.eps}),
                       ffn(64), norm("n1.weight"), norm("n2.weight"),
                       PartSpec("rope", {"head_dim": 32, "rotary_dim": 16, "theta": 5e3, "pairing": "interleaved"}))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=h, layers=(l0, l1, l2),
            order=(LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(0), LayerCall(2, reads_cache_of=2)),
            embedding=PartSpec("token_embedding", {"name": "embed.weight", "vocab_size": self.vocab_size, "hidden_size": h}),
            final_norm=norm("final_norm.weight"),
            head=PartSpec("lm_head", {"name": "head.weight", "tied": False, "vocab_size": self.vocab_size, "hidden_size": h}),
            max_position_embeddings=1024)


register_mixer("toy_ema", ToyEMAMixer, replace=True)
register_feed_forward("toy_routed", ToyRoutedFFN, replace=True)
register_position_encoding("toy_linear_rotary", ToyLinearRotary, replace=True)
register_architecture("ToyHybridForCausalLM", ToyConfig, replace=True)


# ------------------------------------------------------------ its plain implementation
def rope_partial_interleaved(x, positions, rotary_dim, theta):
    cos, sin = plain.rope_angles(rotary_dim, theta, positions)
    xf = x.float()
    rot, rest = xf[..., :rotary_dim], xf[..., rotary_dim:]
    a, b = rot[..., 0::2], rot[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    out = torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
    return torch.cat([out, rest], dim=-1).to(x.dtype)


gaps: list[float] = []      # smallest distance between the two best router logits, per sequence run


def toy_plain(w: dict[str, torch.Tensor], ids: list[int], cfg: ToyConfig) -> torch.Tensor:
    t = len(ids)
    pos = torch.arange(t)
    x = plain.embed(w["embed.weight"], torch.tensor(ids))
    kept: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}

    def mlp(x, p):
        hn = plain.rms_norm(x, w[p + "n2.weight"], cfg.eps)
        return x + plain.swiglu(hn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])

    def routed(x, p):
        hn = plain.rms_norm(x, w[p + "n2.weight"], cfg.eps)
        logits = hn.float() @ w[p + "moe.router.weight"].float().t()
        top2 = logits.topk(2, dim=-1).values
        gaps.append((top2[:, 0] - top2[:, 1]).min().item())
        prob = torch.softmax(logits, dim=-1)
        w1, w2 = w[p + "moe.w1"].view(3, 40, cfg.hidden_size), w[p + "moe.w2"].view(3, cfg.hidden_size, 40)
        rows = []
        for i in range(t):
            e = int(logits[i].argmax())
            hid = torch.relu(plain.linear(hn[i: i + 1], w1[e]))
            rows.append((plain.linear(hid, w2[e]).float() * prob[i, e]).to(x.dtype))
        return x + torch.cat(rows)

    def attn0(x):
        p = "layers.0."
        hn = plain.rms_norm(x, w[p + "n1.weight"], cfg.eps)
        q = plain.linear(hn, w[p + "attn.q_proj.weight"]).view(t, 4, 16)
        k = plain.linear(hn, w[p + "attn.k_proj.weight"]).view(t, 2, 16)
        v = plain.linear(hn, w[p + "attn.v_proj.weight"]).view(t, 2, 16)
        angle = pos.double()[:, None] * (torch.arange(1, 9, dtype=torch.float64) * 0.013)
        cos, sin = angle.cos().float(), angle.sin().float()
        a = plain.causal_gqa_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, 0.25, cfg.window)
        return mlp(x + plain.linear(a.reshape(t, 64), w[p + "attn.o_proj.weight"]), p)

    def ema(x):
        p = "layers.1."
        hn = plain.rms_norm(x, w[p + "n1.weight"], cfg.eps)
        u = hn.float() @ w[p + "ema.in.weight"].float().t()
        decay = torch.sigmoid(w[p + "ema.decay_logit"].float())
        s, ys = torch.zeros(cfg.hidden_size), []
        for i in range(t):
            s = decay * s + u[i]
            ys.append(s)
        y = (torch.stack(ys) @ w[p + "ema.out.weight"].float().t()).to(x.dtype)
        return routed(x + y, p)

    def attn2(x, call, reads=None):
        p = "layers.2."
        hn = plain.rms_norm(x, w[p + "n1.weight"], cfg.eps)
        q = plain.rms_norm(plain.linear(hn, w[p + "attn.q_proj.weight"]).view(t, 2, 32), w[p + "attn.q_norm.weight"], cfg.eps)
        q = rope_partial_interleaved(q, pos, 16, 5e3)
        if reads is None:
            k = plain.rms_norm(plain.linear(hn, w[p + "attn.k_proj.weight"]).view(t, 2, 32), w[p + "attn.k_norm.weight"], cfg.eps)
            kept[call] = (rope_partial_interleaved(k, pos, 16, 5e3), plain.linear(hn, w[p + "attn.v_proj.weight"]).view(t, 2, 32))
            reads = call
        k, v = kept[reads]
        a = plain.causal_gqa_attention(q, k, v, 32 ** -0.5)
        return mlp(x + plain.linear(a.reshape(t, 64), w[p + "attn.o_proj.weight"]), p)

    x = attn0(x)
    x = ema(x)
    x = attn2(x, 2)
    x = attn0(x)
    x = attn2(x, 4, reads=2)
    x = plain.rms_norm(x, w["final_norm.weight"], cfg.eps)
    return plain.linear(x, w["head.weight"]).float()


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    from tinyserve_b200.weights import write_random_model

    cfg = ToyConfig()
    folder = write_random_model(tmp_path_factory.mktemp("toy"), cfg, 7, torch.bfloat16, std_scale=8.0)
    assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyHybridForCausalLM"]
    # Prompts under which no token sits near the border between two experts: the two best router
    # logits are at least 0.4 apart (bf16 moves them by some hundredths), so a different expert in
    # the engine would be a fault and not rounding.
    reqs = {f"r{i}": random_prompt(n, cfg.vocab_size, seed) for i, (n, seed) in enumerate([(3, 37), (20, 54), (41, 68), (70, 60)])}
    w32 = plain.read_weights(folder, torch.float32)
    gaps.clear()
    want = {rid: toy_plain(w32, toks, cfg) for rid, toks in reqs.items()}
    assert len(gaps) == 4 and min(gaps) > 0.4
    return folder, cfg, reqs, want


def test_cache_groups_of_the_toy(toy) -> None:
    from tinyserve_b200.cache import CacheManager
    from tinyserve_b200.model import DecoderModel
    from tinyserve_b200.parts import KVNeed

    folder = toy[0]
    model = DecoderModel.from_folder(folder, torch.float32, "cuda")
    needs = model.cache_needs()
    assert needs == [KVNeed(2, 16, 6), StateNeed((48,), torch.float32), KVNeed(2, 32, None), KVNeed(2, 16, 6), None]
    cache = CacheManager(needs, page_size=4, num_pages=16, max_requests=2, dtype=torch.float32, device="cuda")
    assert [g.calls for g in cache.groups] == [[0, 3], [2]]        # the layer named twice has two cache entries
    assert model.tensors["layers.1.ema.decay_logit"].dtype == torch.float32


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("page", [4, 16])
def test_toy_under_every_cut(toy, dtype, page) -> None:
    from tinyserve_b200.engine.replay import Replayer
    from tinyserve_b200.model import DecoderModel

    folder, cfg, reqs, want = toy
    model = DecoderModel.from_folder(folder, dtype, "cuda")

    def run(steps):
        rep = Replayer(model, cases.max_live_tokens(steps), page_size=page)
        for g in rep.cache.groups:
            g.kv.fill_(float("nan"))
        got, fed = {}, {}
        for entries, end in steps:
            logits = rep.run_step(entries, end)
            row = 0
            for rid, toks, places in entries:
                for p in places:
                    got.setdefault(rid, {})[fed.get(rid, 0) + p] = logits[row].float().cpu()
                    row += 1
                fed[rid] = fed.get(rid, 0) + len(toks)
        assert all(g.allocator.num_used == 0 for g in rep.cache.groups) and rep.cache.state_pool.num_free == 64
        return got

    tol = {"atol": 5e-5, "rtol": 5e-5} if dtype == torch.float32 else {"atol": 0.25, "rtol": 0.1}
    plans = [cases.mixed(reqs, 3), cases.mixed(reqs, 4)]
    for rid, toks in reqs.items():
        plans += [cases.whole(rid, toks), cases.tail_decoded(rid, toks, 32), cases.portions(rid, toks, 1)]
    for steps in plans:
        got = run(steps)
        for rid in got:
            rows = torch.stack([got[rid][p] for p in range(len(reqs[rid]))])
            assert not rows.isnan().any()
            torch.testing.assert_close(rows, want[rid], **tol)


def test_window_pages_are_given_back_early(toy) -> None:
    from tinyserve_b200.engine.replay import Replayer
    from tinyserve_b200.model import DecoderModel

    folder, cfg, reqs, _ = toy
    rep = Replayer(DecoderModel.from_folder(folder, torch.float32, "cuda"), 128, page_size=4)
    toks = reqs["r3"]
    rep.run_step([("x", toks[:40], [])], [])
    win, full = rep.cache.groups[0], rep.cache.groups[1]
    assert full.allocator.num_used == 10 and win.allocator.num_used <= 3     # window 6 on pages of 4
    rep.run_step([("x", toks[40:], [])], ["x"])
    assert win.allocator.num_used == 0 and full.allocator.num_used == 0
