"""Each part of a layer alone on the GPU against the plain implementation's function for it,
at sizes of its own, in float32 and bfloat16."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

import plain_qwen3 as plain
from tinyserve_b200.cache import CacheManager
from tinyserve_b200.engine.step import ModelRunner, StepEntry
from tinyserve_b200.parts.attention import GQAAttention
from tinyserve_b200.parts.base import ResidualStream
from tinyserve_b200.parts.embedding import LMHead, TokenEmbedding
from tinyserve_b200.parts.mlp import SwiGLU
from tinyserve_b200.parts.norm import RMSNorm
from tinyserve_b200.parts.rope import RotaryEncoding

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, want=None):
    """float32: summation order only. bfloat16: a few steps of the 8-bit mantissa at the scale
    of the largest value (inputs, intermediate activations and the output are each rounded)."""
    if dtype == torch.float32:
        return {"atol": 2e-5, "rtol": 2e-5}
    scale = 1.0 if want is None else max(1.0, float(want.abs().max()))
    return {"atol": 2e-2 * scale, "rtol": 3e-2}


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def context(dtype, needs, lens, page=8, tokens=None):
    """A step context for requests given as (context length, new tokens), all freshly cached."""
    cache = CacheManager(needs, page_size=page, num_pages=64, max_requests=8, dtype=dtype, device="cuda")
    runner = ModelRunner(SimpleNamespace(dtype=dtype, device=torch.device("cuda")), cache)
    entries = []
    for i, (total, n) in enumerate(lens):
        r = cache.new_request()
        cache.append(r, total)
        toks = tokens[i] if tokens is not None else [1] * n
        entries.append(StepEntry(r, toks))
    ctx, _, _ = runner.build_context(entries, None)
    return ctx, cache


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part_adds_then_normalises(dtype) -> None:
    size, t = 200, 11
    part = RMSNorm("w", size, 1e-5)
    w = (1 + rnd(size, seed=1, scale=0.1)).to(dtype)
    part.bind("", {"w": w.cuda()})
    ctx, _ = context(dtype, [], [(t, t)])
    resid, delta = rnd(t, size, seed=2, scale=2.0), rnd(t, size, seed=3).to(dtype)
    stream = ResidualStream(resid.cuda().clone(), delta.cuda())
    out = part.forward(stream, ctx)
    x = resid + delta.float()
    torch.testing.assert_close(stream.resid.cpu(), x, atol=0, rtol=0)
    assert stream.delta is None
    want = plain.rms_norm(x, w.float(), 1e-5)
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))
    rows = torch.tensor([4, 10], dtype=torch.int32, device="cuda")
    some = part.forward_rows(ResidualStream(resid.cuda(), delta.cuda()), rows, 2, ctx)
    torch.testing.assert_close(some.float().cpu(), want[[4, 10]], **tol(dtype))


@pytest.mark.parametrize("theta,dim", [(1e4, 16), (1e6, 128), (5e4, 48)])
def test_rotary_tables(theta, dim) -> None:
    part = RotaryEncoding(dim, dim, theta)
    ctx, _ = context(torch.float32, [], [(300, 7), (4000, 1), (1, 1)])
    tables = part.prepare(ctx)
    pos = ctx.positions.cpu().long()
    assert pos.tolist() == list(range(293, 300)) + [3999, 0]
    cos, sin = plain.rope_angles(dim, theta, pos)
    torch.testing.assert_close(tables.cos.cpu(), cos, atol=1e-7, rtol=0)
    torch.testing.assert_close(tables.sin.cpu(), sin, atol=1e-7, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,hidden", [(6, 2, 32, 72), (4, 4, 64, 100), (8, 1, 16, 64)])
def test_attention_part_whole_then_token_by_token(dtype, hq, hkv, d, hidden) -> None:
    eps, theta, t = 1e-5, 1e4, 37
    part = GQAAttention("a.", hidden, hq, hkv, d, d ** -0.5, qk_norm=True, qk_norm_eps=eps)
    rope = RotaryEncoding(d, d, theta)
    w = {"a.q_proj.weight": rnd(hq * d, hidden, seed=1, scale=0.2), "a.k_proj.weight": rnd(hkv * d, hidden, seed=2, scale=0.2),
         "a.v_proj.weight": rnd(hkv * d, hidden, seed=3, scale=0.2), "a.o_proj.weight": rnd(hidden, hq * d, seed=4, scale=0.2),
         "a.q_norm.weight": 1 + rnd(d, seed=5, scale=0.1), "a.k_norm.weight": 1 + rnd(d, seed=6, scale=0.1)}
    w = {k: v.to(dtype) for k, v in w.items()}
    bound = {"a.qkv_proj.weight": torch.cat([w["a.q_proj.weight"], w["a.k_proj.weight"], w["a.v_proj.weight"]]).cuda(),
             **{k: v.cuda() for k, v in w.items()}}
    part.bind("", bound)
    x = rnd(t, hidden, seed=7).to(dtype)
    # plain: the attention block without its norm and residual
    wf = {k: v.float() for k, v in w.items()}
    xf = x.float()
    cos, sin = plain.rope_angles(d, theta, torch.arange(t))
    q = plain.rms_norm(plain.linear(xf, wf["a.q_proj.weight"]).view(t, hq, d), wf["a.q_norm.weight"], eps)
    k = plain.rms_norm(plain.linear(xf, wf["a.k_proj.weight"]).view(t, hkv, d), wf["a.k_norm.weight"], eps)
    v = plain.linear(xf, wf["a.v_proj.weight"]).view(t, hkv, d)
    a = plain.causal_gqa_attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, d ** -0.5)
    want = plain.linear(a.reshape(t, hq * d), wf["a.o_proj.weight"])
    # whole
    ctx, cache = context(dtype, [part.cache_need()], [(t, t)])
    got = part.forward(x.cuda(), ctx, cache.entries[0], True, rope.prepare(ctx))
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype, want))
    # token by token into one cache
    cache = CacheManager([part.cache_need()], page_size=4, num_pages=32, max_requests=2, dtype=dtype, device="cuda")
    runner = ModelRunner(SimpleNamespace(dtype=dtype, device=torch.device("cuda")), cache)
    r = cache.new_request()
    rows = []
    for i in range(t):
        cache.append(r, 1)
        ctx, _, _ = runner.build_context([StepEntry(r, [1])], None)
        rows.append(part.forward(x[i: i + 1].cuda(), ctx, cache.entries[0], True, rope.prepare(ctx)).float().cpu())
    torch.testing.assert_close(torch.cat(rows), want, **tol(dtype, want))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype) -> None:
    hidden, inter, t = 72, 100, 13
    part = SwiGLU("m.", hidden, inter)
    g, u, dn = rnd(inter, hidden, seed=1, scale=0.2).to(dtype), rnd(inter, hidden, seed=2, scale=0.2).to(dtype), rnd(hidden, inter, seed=3, scale=0.2).to(dtype)
    part.bind("", {"m.gate_up_proj.weight": torch.cat([g, u]).cuda(), "m.down_proj.weight": dn.cuda()})
    x = rnd(t, hidden, seed=4).to(dtype)
    ctx, _ = context(dtype, [], [(t, t)])
    got = part.forward(x.cuda(), ctx)
    want = plain.swiglu(x.float(), g.float(), u.float(), dn.float())
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype, want))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head(dtype) -> None:
    vocab, hidden = 301, 72
    table = rnd(vocab, hidden, seed=1).to(dtype)
    emb = TokenEmbedding("e", vocab, hidden)
    emb.bind("", {"e": table.cuda()})
    toks = [[5, 300, 0, 17]]
    ctx, _ = context(dtype, [], [(4, 4)], tokens=toks)
    torch.testing.assert_close(emb.forward(ctx).cpu(), plain.embed(table, torch.tensor(toks[0])).float(), atol=0, rtol=0)
    head = LMHead("e", True, vocab, hidden, "lm_head.weight")
    head.bind("", {"e": table.cuda()})
    x = rnd(4, hidden, seed=2).to(dtype)
    out = torch.empty(4, vocab, device="cuda")
    head.forward(x.cuda(), out)
    want = plain.linear(x.float(), table.float())
    torch.testing.assert_close(out.cpu(), want, **tol(dtype, want))
    assert head.ignorable_tensors("") == {"lm_head.weight"}
