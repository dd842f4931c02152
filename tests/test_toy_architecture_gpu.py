"""The framework takes parts and architectures it has never seen, without a change to its
files: a toy mixer with state of its own, a toy mixer with a cache need of its own kind (one
latent vector per token, in pages of its own layout), a toy feed-forward that routes every
token to one of three experts, a toy position encoding with its own angles, a toy block with
three norms and two feed-forwards (all defined HERE), a layer with a sliding window, a partial
interleaved rotation, a layer that runs twice and a call that reads another call's cache are
registered, built from a config.json, loaded, and replayed under every cut of the work against a
plain implementation of the same toy; the variant whose mixers all allow it also decodes from
recorded steps. (The toy is no model of anyone's.)"""

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
    Block, FeedForward, Mixer, PagedNeed, PositionEncoding, Rotation, StateNeed, TensorSpec, register_block,
    register_feed_forward, register_mixer, register_position_encoding,
)

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------- the toy mixer
class ToyEMAMixer(Mixer):
    """s_t = decay * s_{t-1} + x_t Win^T;  y_t = s_t Wout^T, with s in a state slot per request."""

    recordable = frozenset({"decode"})      # decode tokens are handled on the device alone (below)

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
        if ctx.max_query_len == 1:
            # one token per request: the state rows are indexed with the step's slot ids on the
            # device, nothing of the step is read on the host, so such a step can be recorded
            # (padding rows of a recording carry the pad slot)
            slots = ctx.state_slots.long()
            s = self.decay * cache.state[slots] + u
            cache.state[slots] = s
            out.copy_((s @ self.w_out.float().t()).to(ctx.dtype))
            return out
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


# ------------------------------------- the toy mixer with a cache need of its own kind
@dataclass(frozen=True)
class LatentNeed(PagedNeed):
    """One vector of ``width`` elements per token (keys and values are the same thing here), in
    pages ``[call, page, offset, width]``: neither the shape nor the entry of ``KVNeed``."""

    width: int
    window: int | None = None

    def bytes_per_token(self, element_size: int) -> int:
        return self.width * element_size

    def allocate(self, num_calls, num_pages, page_size, dtype, device):
        return torch.zeros((num_calls, num_pages, page_size, self.width), dtype=dtype, device=device)

    def entry(self, storage, call_in_group, group, page_size):
        return LatentEntry(group, storage[call_in_group], page_size)


@dataclass
class LatentEntry:
    group: int
    latent: torch.Tensor        # [pages + 1, page_size, width]
    page_size: int


class ToyLatentMixer(Mixer):
    """c_t = x_t Wc^T is cached; y_t = softmax_j<=t(scale * (x_t Wq^T) . c_j) c_j Wo^T: one head
    whose keys and values are the cached latents."""

    def __init__(self, prefix: str, hidden_size: int, width: int) -> None:
        self.prefix, self.h, self.c = prefix, hidden_size, width

    def cache_need(self) -> LatentNeed:
        return LatentNeed(self.c)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p = prefix + self.prefix
        return [TensorSpec(p + "c.weight", (self.c, self.h)), TensorSpec(p + "q.weight", (self.c, self.h)),
                TensorSpec(p + "o.weight", (self.h, self.c))]

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p = prefix + self.prefix
        self.wc, self.wq, self.wo = tensors[p + "c.weight"], tensors[p + "q.weight"], tensors[p + "o.weight"]

    def forward(self, x, ctx, cache, writes_cache, position):
        group = ctx.kv[cache.group]
        flat = cache.latent.view(-1, self.c)                        # row = page * page_size + offset = slot
        flat[group.slots.long()] = x @ self.wc.t()
        q = (x @ self.wq.t()).float()
        out = ctx.arena.take((x.shape[0], self.h), ctx.dtype)
        row = 0
        for b, (n, total) in enumerate(zip(ctx.query_lens, ctx.context_lens)):
            pages = group.block_tables[b, : -(-total // cache.page_size)].long()
            keys = cache.latent[pages].reshape(-1, self.c)[:total].float()
            s = q[row: row + n] @ keys.t() * self.c ** -0.5
            qpos = torch.arange(total - n, total, device=x.device)[:, None]
            s = s.masked_fill(torch.arange(total, device=x.device)[None, :] > qpos, float("-inf"))
            mixed = (torch.softmax(s, dim=-1) @ keys).to(ctx.dtype)
            out[row: row + n] = mixed @ self.wo.t()
            row += n
        return out


# ------------------------------------------------------ the toy block with three norms
class ToyThreeNormBlock(Block):
    """x += mixer(n1(x)); x += ff_a(n2(x)); x += ff_b(n3(x)): six roles under names of its own."""

    roles = {"n1": "norm", "mixer": "mixer", "n2": "norm", "ff_a": "feed_forward", "n3": "norm", "ff_b": "feed_forward"}

    def forward(self, stream, ctx, caches, writes_cache, position):
        p = self.parts
        ctx.arena.next_frame()
        ctx.upcoming_weights = []
        stream.delta = p["mixer"].forward(p["n1"].forward(stream, ctx), ctx, caches.get("mixer"), writes_cache, position)
        stream.delta = p["ff_a"].forward(p["n2"].forward(stream, ctx), ctx)
        stream.delta = p["ff_b"].forward(p["n3"].forward(stream, ctx), ctx)
        stream.sumsq = None


# ------------------------------------------------- the toy feed-forward with routing
class ToyRoutedFFN(FeedForward):
    """Every token goes to the one expert with the largest router logit (32-bit) and gets
    p_e * W2_e relu(W1_e x), p the softmax of the router logits."""

    recordable = frozenset({"decode"})      # decode rows go through every expert, masked (below)

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
        if ctx.max_query_len == 1:
            # a few decode rows: every expert computes every row and the mask picks; nothing is
            # read back on the host (listing an expert's rows would be), so the step can be recorded
            out.zero_()
            for e in range(self.e):
                hid = torch.relu(x @ self.w1[e].t())
                y = ((hid @ self.w2[e].t()).float() * prob[:, None]).to(ctx.dtype)
                out += torch.where((expert == e)[:, None], y, torch.zeros_like(y))
            return out
        for e in range(self.e):
            rows = (expert == e).nonzero().flatten()
            hid = torch.relu(x[rows] @ self.w1[e].t())
            out[rows] = ((hid @ self.w2[e].t()).float() * prob[rows, None]).to(ctx.dtype)
        return out


# ------------------------------------------------------ the toy position encoding
class ToyLinearRotary(PositionEncoding):
    """Rotation angles position * (i + 1) * step: frequencies in a line, not in a geometric row.
    Hands the mixer the same kind of tables as the built-in encoding, made its own way."""

    recordable = frozenset({"decode", "prefill"})      # device tensors only

    def __init__(self, rotary_dim: int, step: float) -> None:
        self.rotary_dim, self.step = rotary_dim, step

    def key(self) -> Any:
        return ("toy_linear", self.rotary_dim, self.step)

    def prepare(self, ctx) -> Rotation:
        half = self.rotary_dim // 2
        freq = torch.arange(1, half + 1, dtype=torch.float64, device=ctx.positions.device) * self.step
        angle = ctx.positions.double()[:, None] * freq
        cos = ctx.arena.take_step((ctx.num_tokens, half), torch.float32)
        sin = ctx.arena.take_step((ctx.num_tokens, half), torch.float32)
        cos.copy_(angle.cos())
        sin.copy_(angle.sin())
        return Rotation(cos, sin, self.rotary_dim, False)


# ------------------------------------------------------------ the toy architecture
@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    vocab_size: int = 97
    hidden_size: int = 48
    window: int = 6
    eps: float = 1e-5
    latent_layer: bool = True        # the layer with the three-norm block and the latent mixer, run last
    architecture = "ToyHybridForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(d["vocab_size"], d["hidden_size"], d["window"], d["eps"], d["latent_layer"])

    def to_dict(self):
        return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "window": self.window, "eps": self.eps, "latent_layer": self.latent_layer}

    def to_spec(self) -> ModelSpec:
        h = self.hidden_size

        def norm(name):
            return PartSpec("rms_norm", {"name": name, "size": h, "eps": self.eps})

        def ffn(i):
            return PartSpec("swiglu", {"prefix": "mlp.", "hidden_size": h, "intermediate_size": i})

        def prenorm(prefix, mixer, feed_forward, position):
            return LayerSpec(prefix, "prenorm", {"mixer": mixer, "feed_forward": feed_forward,
                                                 "mixer_norm": norm("n1.weight"), "feed_forward_norm": norm("n2.weight")},
                             position)

        l0 = prenorm("layers.0.",
                     PartSpec("gqa_attention", {"prefix": "attn.", "hidden_size": h, "num_heads": 4, "num_kv_heads": 2,
                                                "head_dim": 16, "scale": 0.25, "window": self.window}),
                     ffn(64), PartSpec("toy_linear_rotary", {"rotary_dim": 16, "step": 0.013}))
        l1 = prenorm("layers.1.", PartSpec("toy_ema", {"prefix": "ema.", "hidden_size": h}),
                     PartSpec("toy_routed", {"prefix": "moe.", "hidden_size": h, "expert_size": 40, "num_experts": 3}), None)
        l2 = prenorm("layers.2.",
                     PartSpec("gqa_attention", {"prefix": "attn.", "hidden_size": h, "num_heads": 2, "num_kv_heads": 2,
                                                "head_dim": 32, "scale": 32 ** -0.5, "qk_norm": True,
                                                "qk_norm_eps": self.eps}),
                     ffn(64), PartSpec("rope", {"head_dim": 32, "rotary_dim": 16, "theta": 5e3, "pairing": "interleaved"}))
        l3 = LayerSpec("layers.3.", "toy_three_norm", {
            "n1": norm("n1.weight"), "mixer": PartSpec("toy_latent", {"prefix": "lat.", "hidden_size": h, "width": 24}),
            "n2": norm("n2.weight"), "ff_a": PartSpec("swiglu", {"prefix": "mlp_a.", "hidden_size": h, "intermediate_size": 32}),
            "n3": norm("n3.weight"), "ff_b": PartSpec("swiglu", {"prefix": "mlp_b.", "hidden_size": h, "intermediate_size": 48}),
        })
        layers = (l0, l1, l2, l3) if self.latent_layer else (l0, l1, l2)
        order = (LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(0), LayerCall(2, reads_cache_of=2))
        if self.latent_layer:
            order += (LayerCall(3),)
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=h, layers=layers, order=order,
            embedding=PartSpec("token_embedding", {"name": "embed.weight", "vocab_size": self.vocab_size, "hidden_size": h}),
            final_norm=norm("final_norm.weight"),
            head=PartSpec("lm_head", {"name": "head.weight", "tied": False, "vocab_size": self.vocab_size, "hidden_size": h}),
            max_position_embeddings=1024)


register_mixer("toy_ema", ToyEMAMixer, replace=True)
register_mixer("toy_latent", ToyLatentMixer, replace=True)
register_block("toy_three_norm", ToyThreeNormBlock, replace=True)
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

    def latent(x):
        p = "layers.3."
        hn = plain.rms_norm(x, w[p + "n1.weight"], cfg.eps)
        c = plain.linear(hn, w[p + "lat.c.weight"])                  # rounded to the working dtype, as the cache holds it
        s = plain.linear(hn, w[p + "lat.q.weight"]).float() @ c.float().t() * 24 ** -0.5
        s = s.masked_fill(torch.arange(t)[None, :] > torch.arange(t)[:, None], float("-inf"))
        x = x + plain.linear((torch.softmax(s, dim=-1) @ c.float()).to(x.dtype), w[p + "lat.o.weight"])
        for n, m in (("n2.weight", "mlp_a."), ("n3.weight", "mlp_b.")):
            hn = plain.rms_norm(x, w[p + n], cfg.eps)
            x = x + plain.swiglu(hn, w[p + m + "gate_proj.weight"], w[p + m + "up_proj.weight"], w[p + m + "down_proj.weight"])
        return x

    x = attn0(x)
    x = ema(x)
    x = attn2(x, 2)
    x = attn0(x)
    x = attn2(x, 4, reads=2)
    if cfg.latent_layer:
        x = latent(x)
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
    assert needs == [KVNeed(2, 16, 6), StateNeed((48,), torch.float32), KVNeed(2, 32, None), KVNeed(2, 16, 6), None,
                     LatentNeed(24)]
    cache = CacheManager(needs, page_size=4, num_pages=16, max_requests=2, dtype=torch.float32, device="cuda",
                         max_step_tokens=8)
    assert [g.calls for g in cache.groups] == [[0, 3], [2], [5]]   # the layer named twice has two cache entries
    # the window group holds what two requests can hold of it (window 6 + a step of 8 tokens on pages of 4)
    assert [g.num_pages for g in cache.groups] == [2 * 5, 16, 16]
    assert cache.groups[2].kv.shape == (1, 17, 4, 24) and isinstance(cache.entries[5], LatentEntry)
    assert cache.can_ever_hold(64, 8) and not cache.can_ever_hold(65, 8)
    assert model.tensors["layers.1.ema.decay_logit"].dtype == torch.float32
    assert not model.parts.recordable("decode") and not model.parts.recordable("prefill")


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


def test_a_state_mixer_decodes_from_recorded_steps(tmp_path) -> None:
    """The variant of the toy whose mixers all allow it ("decode": the attention mixer and the
    state mixer, which indexes its state rows with the step's slot ids on the device): its decode
    steps are recorded once per batch size and replayed, launched ahead of their tokens, with
    padding rows on the pad page and the pad slot. Every logits row the engine sampled from equals
    the plain toy's on the request's final sequence; prompt portions are not recorded (the state
    mixer walks them on the host)."""
    from tinyserve_b200 import LLM
    from tinyserve_b200.weights import write_random_model

    cfg = ToyConfig(latent_layer=False)
    folder = write_random_model(tmp_path, cfg, 7, torch.bfloat16, std_scale=8.0)
    w32 = plain.read_weights(folder, torch.float32)
    prompts = [random_prompt(n, cfg.vocab_size, seed) for n, seed in [(3, 37), (20, 54), (41, 68)]]
    outs = {}
    for graphs in (True, False):
        llm = LLM.from_folder(folder, dtype="float32", page_size=4, num_pages=64, max_num_seqs=4, max_batch_tokens=64,
                              chunked_prefill=True, decode_graphs=graphs, record_logits=True)
        e = llm.engine
        assert e.model.parts.recordable("decode") and not e.model.parts.recordable("prefill")
        ids = [e.add_request(p, 10) for p in prompts]
        while e.has_work():
            e.step()
        outs[graphs] = [e.requests[i].output for i in ids]
        assert (e.runner.num_graph_steps > 5) == graphs and not e.runner.prefill_graphs
        assert all(g.allocator.num_used == 0 for g in llm.cache.groups) and llm.cache.state_pool.num_free == 4
        for j, rid in enumerate(ids):
            seq = prompts[j] + outs[graphs][j]
            gaps.clear()
            want = toy_plain(w32, seq, cfg)
            assert min(gaps) > 1e-3, "a token sits on the border between two experts: choose other prompts"
            rows = {pos: row for r, pos, row in e.logits_log if r == rid}
            for pos in range(len(prompts[j]) - 1, len(seq) - 1):
                torch.testing.assert_close(rows[pos].float().cpu(), want[pos], atol=5e-5, rtol=5e-5)
    assert outs[True] == outs[False]
