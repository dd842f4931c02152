"""Each CUDA kernel alone against its plain PyTorch reference (``kernel_refs``), in float32
and bfloat16, at sizes other than the engine's tiny models'. Pages the requests do not own are
filled with NaN, so a single read too many shows (after upstream
tests/test_triton_attention.py:13-14)."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

import kernel_refs as ref
from tinyserve_b200.engine.arena import Arena
from tinyserve_b200.kernels import ops

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype: torch.dtype) -> dict[str, float]:
    return {"atol": 1e-5, "rtol": 1e-5} if dtype == torch.float32 else {"atol": 2e-2, "rtol": 2e-2}


def rnd(*shape: int, dtype=torch.float32, seed: int = 0, scale: float = 1.0) -> torch.Tensor:
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(72, 301), (1024, 5000)])
def test_embed(dtype, hidden, vocab) -> None:
    table = rnd(vocab, hidden, dtype=dtype)
    tokens = torch.randint(0, vocab, (37,), device="cuda", dtype=torch.int32)
    out, want = torch.empty(37, hidden, device="cuda"), torch.empty(37, hidden, device="cuda")
    ops.embed(tokens, table, out)
    ref.embed(tokens, table, want)
    assert torch.equal(out, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 80, 1000, 4096])
@pytest.mark.parametrize("with_delta", [True, False])
def test_add_rms_norm(dtype, hidden, with_delta) -> None:
    t = 19
    resid = rnd(t, hidden, seed=1, scale=3.0)
    delta = rnd(t, hidden, dtype=dtype, seed=2) if with_delta else None
    w = (1 + rnd(hidden, seed=3, scale=0.1)).to(dtype)
    r1, r2 = resid.clone(), resid.clone()
    out, want = torch.empty(t, hidden, device="cuda", dtype=dtype), torch.empty(t, hidden, device="cuda", dtype=dtype)
    ops.add_rms_norm(r1, delta, w, 1e-5, out)
    ref.add_rms_norm(r2, delta, w, 1e-5, want)
    torch.testing.assert_close(r1, r2, atol=0, rtol=0)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))
    # selected rows: the stream must stay as it is
    rows = torch.tensor([3, 0, 18, 3], device="cuda", dtype=torch.int32)
    r3 = resid.clone()
    out2, want2 = torch.empty(4, hidden, device="cuda", dtype=dtype), torch.empty(4, hidden, device="cuda", dtype=dtype)
    ops.add_rms_norm(r3, delta, w, 1e-5, out2, rows=rows)
    ref.add_rms_norm(resid.clone(), delta, w, 1e-5, want2, rows=rows)
    assert torch.equal(r3, resid)
    torch.testing.assert_close(out2.float(), want2.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [256, 512, 1024, 2048])
@pytest.mark.parametrize("t", [256, 1027])
def test_add_rms_norm_of_many_rows(dtype, hidden, t) -> None:
    """From 256 rows of 256 / 512 / 1,024 / 2,048 values on, a warp takes a row; a last CTA of fewer than four rows."""
    resid = rnd(t, hidden, seed=1, scale=3.0)
    delta = rnd(t, hidden, dtype=dtype, seed=2)
    w = (1 + rnd(hidden, seed=3, scale=0.1)).to(dtype)
    for d in (delta, None):
        r1, r2 = resid.clone(), resid.clone()
        out = torch.full((t, hidden), float("nan"), device="cuda", dtype=dtype)
        want = torch.empty(t, hidden, device="cuda", dtype=dtype)
        ops.add_rms_norm(r1, d, w, 1e-5, out)
        ref.add_rms_norm(r2, d, w, 1e-5, want)
        torch.testing.assert_close(r1, r2, atol=0, rtol=0)
        torch.testing.assert_close(out.float(), want.float(), **tol(dtype))
    rows = torch.randint(0, t, (300,), device="cuda", dtype=torch.int32)
    r3 = resid.clone()
    out2 = torch.empty(300, hidden, device="cuda", dtype=dtype)
    want2 = torch.empty_like(out2)
    ops.add_rms_norm(r3, delta, w, 1e-5, out2, rows=rows)
    ref.add_rms_norm(resid.clone(), delta, w, 1e-5, want2, rows=rows)
    assert torch.equal(r3, resid)
    torch.testing.assert_close(out2.float(), want2.float(), **tol(dtype))


def test_rope_tables_far_positions() -> None:
    pos = torch.tensor([0, 1, 2, 4095, 40959, 1_000_003], device="cuda", dtype=torch.int32)
    two_i = torch.arange(0, 128, 2, dtype=torch.float64)
    inv = (1e6 ** (-two_i / 128)).cuda()
    cos, sin = torch.empty(6, 64, device="cuda"), torch.empty(6, 64, device="cuda")
    wc, ws = torch.empty_like(cos), torch.empty_like(sin)
    ops.rope_tables(pos, inv, cos, sin)
    ref.rope_tables(pos, inv, wc, ws)
    torch.testing.assert_close(cos, wc, atol=1e-7, rtol=0)
    torch.testing.assert_close(sin, ws, atol=1e-7, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [100, 176, 3072])
def test_silu_mul(dtype, inter) -> None:
    gu = rnd(23, 2 * inter, dtype=dtype, scale=3.0)
    out, want = torch.empty(23, inter, device="cuda", dtype=dtype), torch.empty(23, inter, device="cuda", dtype=dtype)
    ops.silu_mul(gu, out)
    ref.silu_mul(gu, want)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,rot,inter,norm,page", [
    (4, 2, 16, 16, False, True, 16), (4, 1, 32, 32, False, True, 8), (3, 3, 48, 48, False, True, 32),
    (16, 8, 128, 128, False, True, 16), (6, 2, 64, 32, True, False, 4), (2, 2, 256, 0, False, True, 16),
    (5, 1, 64, 64, False, True, 8), (3, 3, 256, 256, False, False, 16),
])
@pytest.mark.parametrize("write_kv", [True, False])
@pytest.mark.parametrize("t", [29, 301])       # few tokens (decode) and many (prefill) take different kernels
def test_qk_norm_rope_write(dtype, hq, hkv, d, rot, inter, norm, page, write_kv, t) -> None:
    pages = -(-t // page) + 3
    width = (hq + 2 * hkv) * d if write_kv else hq * d
    qkv = rnd(t, width, dtype=dtype, seed=4, scale=2.0)
    qw = (1 + rnd(d, seed=5, scale=0.2)).to(dtype) if norm else None
    kw = (1 + rnd(d, seed=6, scale=0.2)).to(dtype) if norm else None
    pos = torch.randint(0, 5000, (t,), device="cuda", dtype=torch.int32)
    cos = sin = None
    if rot:
        inv = (1e4 ** (-torch.arange(0, rot, 2, dtype=torch.float64) / rot)).cuda()
        cos, sin = torch.empty(t, rot // 2, device="cuda"), torch.empty(t, rot // 2, device="cuda")
        ref.rope_tables(pos, inv, cos, sin)
    slots = torch.randperm(pages * page, device="cuda")[:t].to(torch.int32)
    caches = [torch.full((pages, hkv, page, d), float("nan"), device="cuda", dtype=dtype) for _ in range(4)]
    q1, q2 = (torch.empty(t, hq, d, device="cuda", dtype=dtype) for _ in range(2))
    args = (qw, kw, 1e-6, cos, sin, rot, inter, slots)
    ops.qk_norm_rope_write(qkv, q1, *args, caches[0], caches[1], page, hq, hkv, d, write_kv)
    ref.qk_norm_rope_write(qkv, q2, *args, caches[2], caches[3], page, hq, hkv, d, write_kv)
    torch.testing.assert_close(q1.float(), q2.float(), **tol(dtype))
    for a, b in ((caches[0], caches[2]), (caches[1], caches[3])):
        assert torch.equal(a.isnan(), b.isnan()), "wrote outside the tokens' slots (or missed one)"
        torch.testing.assert_close(a.float().nan_to_num(0), b.float().nan_to_num(0), **tol(dtype))


def _attention_case(dtype, hq, hkv, d, page, lens, window, seed=0, scale=None, spike=None):
    """lens: list of (context_len, new_tokens). Builds NaN-poisoned caches with the requests'
    pages scattered, and runs kernel and reference. ``spike`` = (request, key position) makes
    one far key dominate: q and that k are aligned and scaled up."""
    b = len(lens)
    need = [-(-c // page) for c, _ in lens]
    pages = sum(need) + 5
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max(need) + 2
    tables = torch.zeros(b, width, dtype=torch.int32)
    k_cache = torch.full((pages, hkv, page, d), float("nan"), device="cuda", dtype=dtype)
    v_cache = torch.full((pages, hkv, page, d), float("nan"), device="cuda", dtype=dtype)
    at = 0
    for i, (c, _) in enumerate(lens):
        mine = perm[at: at + need[i]]
        at += need[i]
        tables[i, : need[i]] = torch.tensor(mine)
        k = rnd(c, hkv, d, dtype=dtype, seed=seed * 100 + i)
        v = rnd(c, hkv, d, dtype=dtype, seed=seed * 100 + 50 + i)
        if spike is not None and spike[0] == i:
            k[spike[1]] = k[spike[1]] * 6
        for p in range(c):
            k_cache[mine[p // page], :, p % page] = k[p]
            v_cache[mine[p // page], :, p % page] = v[p]
    qlens = [n for _, n in lens]
    t = sum(qlens)
    q = rnd(t, hq, d, dtype=dtype, seed=seed + 7)
    cu = [0]
    for n in qlens:
        cu.append(cu[-1] + n)
    if spike is not None:
        i, pos = spike
        c = lens[i][0]
        page_id = int(tables[i, pos // page])
        kk = k_cache[page_id, :, pos % page].float()          # [hkv, d]
        q[cu[i + 1] - 1] = (kk.repeat_interleave(hq // hkv, dim=0) * 0.5).to(dtype)
    dec = [i for i, n in enumerate(qlens) if n == 1]
    pre = [i for i, n in enumerate(qlens) if n > 1]
    pad = lambda xs: torch.tensor(xs + [0] * (b - len(xs)), dtype=torch.int32, device="cuda")
    ctx = SimpleNamespace(
        num_seqs=b, query_lens=qlens, cu_query_lens=torch.tensor(cu, dtype=torch.int32, device="cuda"),
        context_lens_dev=torch.tensor([c for c, _ in lens], dtype=torch.int32, device="cuda"),
        decode_seqs=pad(dec), prefill_seqs=pad(pre), num_decode=len(dec), num_prefill=len(pre),
        max_query_len=max(qlens), max_context_len=max(c for c, _ in lens), arena=Arena("cuda"))
    sc = scale if scale is not None else d ** -0.5
    out = torch.full((t, hq * d), float("nan"), device="cuda", dtype=dtype)
    want = torch.empty(t, hq * d, device="cuda", dtype=dtype)
    tables = tables.cuda()
    ops.paged_attention(q, k_cache, v_cache, page, tables, ctx, sc, window, out)
    ref.paged_attention(q, k_cache, v_cache, page, tables, ctx, sc, window, want)
    return out, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [
    (4, 2, 16, 16), (4, 1, 32, 8), (3, 3, 48, 32), (16, 8, 128, 16), (8, 1, 64, 16), (12, 2, 80, 4),
    (2, 1, 256, 16), (5, 5, 128, 64), (4, 2, 64, 8), (6, 3, 128, 8), (8, 2, 128, 32), (32, 2, 64, 48),
])
def test_attention_mixed_batch(dtype, hq, hkv, d, page) -> None:
    lens = [(1, 1), (16, 1), (17, 1), (33, 33), (64, 2), (300, 1), (129, 40), (96, 96), (500, 3), (1025, 1)]
    out, want = _attention_case(dtype, hq, hkv, d, page, lens, 0)
    assert not out.isnan().any()
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("kernel,heads_per_cta", [("tcgen05", 1), ("tcgen05", 2), ("mma", 0)])
@pytest.mark.parametrize("hq,hkv,d,page", [(16, 8, 128, 16), (4, 2, 64, 8), (8, 2, 128, 32), (6, 1, 64, 48),
                                           (5, 5, 128, 8)])
@pytest.mark.parametrize("window", [0, 150])
def test_prefill_attention_kernels(kernel, heads_per_cta, hq, hkv, d, page, window, monkeypatch) -> None:
    """Each bf16 prefill kernel by name: whole prompts, chunks on top of a long context, lengths
    around the 64 / 128 tile edges, and short chunks."""
    monkeypatch.setattr(ops, "PREFILL_ATTENTION", kernel)
    monkeypatch.setattr(ops, "PREFILL_HEADS_PER_CTA", heads_per_cta)
    lens = [(2, 2), (127, 127), (128, 128), (129, 129), (700, 700), (1000, 300), (515, 3), (260, 131), (64, 64),
            (1300, 1), (385, 256), (2500, 1400), (3000, 129)]
    out, want = _attention_case(torch.bfloat16, hq, hkv, d, page, lens, window, seed=2)
    ops.check_device_errors()
    assert not out.isnan().any()
    torch.testing.assert_close(out.float(), want.float(), **tol(torch.bfloat16))


@pytest.mark.parametrize("heads_per_cta", [1, 2])
@pytest.mark.parametrize("pos", [0, 63, 64, 127, 128, 511, 999])
def test_prefill_attention_tcgen05_far_key(heads_per_cta, pos, monkeypatch) -> None:
    monkeypatch.setattr(ops, "PREFILL_HEADS_PER_CTA", heads_per_cta)
    lens = [(1000, 200), (64, 1)]
    out, want = _attention_case(torch.bfloat16, 4, 2, 128, 16, lens, 0, spike=(0, pos), scale=1.0)
    ops.check_device_errors()
    torch.testing.assert_close(out.float(), want.float(), **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 16, 100])
def test_attention_window(dtype, window) -> None:
    lens = [(1, 1), (16, 1), (40, 40), (300, 1), (129, 40), (257, 3)]
    out, want = _attention_case(dtype, 4, 2, 32, 8, lens, window)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_decode_only_many_splits(dtype) -> None:
    lens = [(2048, 1), (1, 1), (777, 1)]
    out, want = _attention_case(dtype, 16, 8, 128, 16, lens, 0)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("window", [0, 50])
@pytest.mark.parametrize("batch", [56, 60, 74])
def test_attention_decode_grid_just_over_three_ctas_per_sm(batch, window) -> None:
    """Unsplit grids of 448 to 592 CTAs (batch x 8 kv heads) run as CTAs of three warps, four to an
    SM; every context length from one key to several tiles per warp, one far key dominating."""
    lens = [(1 + (i * 37) % 300, 1) for i in range(batch - 1)] + [(900, 1)]
    out, want = _attention_case(torch.bfloat16, 16, 8, 128, 16, lens, window, seed=5,
                                spike=(batch - 1, 3 if window == 0 else 870))
    ops.check_device_errors()
    assert not out.isnan().any()
    torch.testing.assert_close(out.float(), want.float(), **tol(torch.bfloat16))


@pytest.mark.parametrize("hq,hkv,d,page", [(16, 8, 128, 16), (14, 2, 64, 8), (40, 2, 128, 16), (5, 5, 64, 32)])
@pytest.mark.parametrize("splits", [2, 3, 5, 8])
@pytest.mark.parametrize("window", [0, 37])
def test_decode_attention_cluster_merge_gives_the_same_bits(hq, hkv, d, page, splits, window, monkeypatch) -> None:
    """2 to 8 key ranges of a request merge inside a thread-block cluster; through global memory
    (the path of more ranges) the same sums are formed in the same order."""
    monkeypatch.setattr(ops, "MAX_SPLITS", splits)
    lens = [(2048, 1), (1, 1), (777, 1), (130, 1)]
    try:
        ops.set_decode_cluster_merge(True)
        out, want = _attention_case(torch.bfloat16, hq, hkv, d, page, lens, window, seed=9, spike=(0, 1500 if window == 0 else 2030))
        ops.set_decode_cluster_merge(False)
        plain, _ = _attention_case(torch.bfloat16, hq, hkv, d, page, lens, window, seed=9, spike=(0, 1500 if window == 0 else 2030))
    finally:
        ops.set_decode_cluster_merge(True)
    ops.check_device_errors()
    assert not out.isnan().any()
    assert torch.equal(out, plain)
    torch.testing.assert_close(out.float(), want.float(), **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("new", [1, 5])
@pytest.mark.parametrize("pos", [0, 15, 16, 511, 700])
def test_attention_far_key_dominates(dtype, new, pos) -> None:
    """One key among a thousand carries almost all the weight: dropping it (a split that ends
    early, a page missed) changes the result completely."""
    lens = [(1000, new), (64, 1)]
    out, want = _attention_case(dtype, 4, 2, 64, 16, lens, 0, spike=(0, pos), scale=1.0)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("hq,hkv,d,page", [(16, 8, 128, 16), (14, 2, 64, 8), (5, 5, 64, 32), (40, 2, 128, 16),
                                           (3, 1, 128, 8)])
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("norm,rot", [(True, True), (False, True), (True, False)])
def test_decode_attention_fused(hq, hkv, d, page, window, norm, rot) -> None:
    """Norm, rotation, cache write and attention of decode tokens in one kernel, against the
    plain references of the two steps. The slot of the new token holds NaN before the call, the
    newest key is made to matter (scaled up), and the context lengths put it at the start, the
    end and the middle of a tile and of a page."""
    dtype = torch.bfloat16
    lens = [1, 2, 15, 16, 17, 33, 64, 300, 777, 1025, 2048]
    b = len(lens)
    need = [-(-c // page) for c in lens]
    pages = sum(need) + 3
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(3)).tolist()
    tables = torch.zeros(b, max(need) + 1, dtype=torch.int32)
    caches = [torch.full((pages, hkv, page, d), float("nan"), device="cuda", dtype=dtype) for _ in range(4)]
    slots, at = [], 0
    for i, c in enumerate(lens):
        mine = perm[at: at + need[i]]
        at += need[i]
        tables[i, : need[i]] = torch.tensor(mine)
        k = rnd(c - 1, hkv, d, dtype=dtype, seed=100 + i)
        v = rnd(c - 1, hkv, d, dtype=dtype, seed=150 + i)
        for p_ in range(c - 1):
            for kc, vc in ((caches[0], caches[1]), (caches[2], caches[3])):
                kc[mine[p_ // page], :, p_ % page] = k[p_]
                vc[mine[p_ // page], :, p_ % page] = v[p_]
        slots.append(mine[(c - 1) // page] * page + (c - 1) % page)
    tables = tables.cuda()
    slots = torch.tensor(slots, dtype=torch.int32, device="cuda")
    qkv = rnd(b, (hq + 2 * hkv) * d, dtype=dtype, seed=9, scale=1.5)
    for h in range(hkv):      # the new key equals the group's first query: that head looks at it alone
        qkv[:, (hq + h) * d: (hq + h + 1) * d] = qkv[:, h * (hq // hkv) * d: (h * (hq // hkv) + 1) * d]
    qw = (1 + rnd(d, seed=5, scale=0.2)).to(dtype) if norm else None
    kw = (1 + rnd(d, seed=6, scale=0.2)).to(dtype) if norm else None
    cos = sin = None
    if rot:
        pos = torch.tensor([c - 1 for c in lens], device="cuda", dtype=torch.int32)
        inv = (1e4 ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)).cuda()
        cos, sin = torch.empty(b, d // 2, device="cuda"), torch.empty(b, d // 2, device="cuda")
        ref.rope_tables(pos, inv, cos, sin)
    ar = torch.arange(b, dtype=torch.int32, device="cuda")
    ctx = SimpleNamespace(
        num_seqs=b, cu_query_lens=torch.arange(b + 1, dtype=torch.int32, device="cuda"),
        context_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda"), decode_seqs=ar, prefill_seqs=ar * 0,
        num_decode=b, num_prefill=0, max_query_len=1, max_context_len=max(lens), arena=Arena("cuda"))
    ops.FUSED_DECODE_MIN_CTAS, saved = 0, ops.FUSED_DECODE_MIN_CTAS
    try:
        assert ops.can_fuse_decode(ctx, dtype, hq, hkv, d, page, pages, d if rot else 0, False, qkv.device)
    finally:
        ops.FUSED_DECODE_MIN_CTAS = saved
    out = torch.full((b, hq * d), float("nan"), device="cuda", dtype=dtype)
    want = torch.empty(b, hq * d, device="cuda", dtype=dtype)
    ops.decode_attention_fused(qkv, qw, kw, 1e-6, cos, sin, slots, caches[0], caches[1], page, tables, ctx,
                               d ** -0.5, window, hq, out)
    q = torch.empty(b, hq, d, device="cuda", dtype=dtype)
    ref.qk_norm_rope_write(qkv, q, qw, kw, 1e-6, cos, sin, d if rot else 0, False, slots, caches[2], caches[3],
                           page, hq, hkv, d, True)
    ref.paged_attention(q, caches[2], caches[3], page, tables, ctx, d ** -0.5, window, want)
    ops.check_device_errors()
    assert not out.isnan().any()
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))
    for a, w in ((caches[0], caches[2]), (caches[1], caches[3])):
        assert torch.equal(a.isnan(), w.isnan()), "wrote outside the tokens' slots (or missed one)"
        torch.testing.assert_close(a.float().nan_to_num(0), w.float().nan_to_num(0), **tol(dtype))
    # the same step through the two separate kernels gives the same rows up to rounding
    two = torch.empty_like(out)
    for kc, vc in ((caches[0], caches[1]),):
        for i, c in enumerate(lens):
            s_ = int(slots[i])
            kc[s_ // page, :, s_ % page] = float("nan")
            vc[s_ // page, :, s_ % page] = float("nan")
    ops.qk_norm_rope_write(qkv, q, qw, kw, 1e-6, cos, sin, d if rot else 0, False, slots, caches[0], caches[1],
                           page, hq, hkv, d, True)
    ops.paged_attention(q, caches[0], caches[1], page, tables, ctx, d ** -0.5, window, two)
    torch.testing.assert_close(out.float(), two.float(), **tol(dtype))


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                                (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("m,n,k", [(1, 301, 72), (7, 80, 176), (64, 64, 16), (65, 130, 33), (200, 1000, 1024)])
def test_gemm_simt(in_dtype, out_dtype, m, n, k) -> None:
    x, w = rnd(m, k, dtype=in_dtype, seed=1), rnd(n, k, dtype=in_dtype, seed=2)
    out, want = (torch.empty(m, n, device="cuda", dtype=out_dtype) for _ in range(2))
    ops.gemm_simt(x, w, out)
    ref.gemm(x, w, want)
    t = {"atol": 1e-4, "rtol": 1e-5} if out_dtype == torch.float32 else {"atol": 2e-1, "rtol": 2e-2}
    torch.testing.assert_close(out.float(), want.float(), **t)


@pytest.mark.parametrize("dtype,out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                             (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("m,n,k", [(1, 301, 72), (8, 4096, 1024), (300, 1024, 3072), (5, 151936, 1024)])
def test_gemm(dtype, out_dtype, m, n, k) -> None:
    x, w = rnd(m, k, dtype=dtype, seed=1), rnd(n, k, dtype=dtype, seed=2, scale=0.05)
    out, want = (torch.empty(m, n, device="cuda", dtype=out_dtype) for _ in range(2))
    ops.gemm(x, w, out)
    ref.gemm(x, w, want)
    t = {"atol": 1e-4, "rtol": 1e-4} if dtype == torch.float32 else {"atol": 5e-2, "rtol": 2e-2}
    torch.testing.assert_close(out.float(), want.float(), **t)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 31, 64])
@pytest.mark.parametrize("n,k", [(16, 32), (48, 96), (1024, 2048), (4096, 1024), (151936, 1024), (1040, 3072)])
def test_gemm_skinny(out_dtype, m, n, k) -> None:
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=1), rnd(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype)
    want = torch.empty(m, n, device="cuda", dtype=out_dtype)
    ops.gemm_skinny(x, w, out)
    ref.gemm(x, w, want)
    t = {"atol": 2e-4, "rtol": 1e-4} if out_dtype == torch.float32 else {"atol": 2e-2, "rtol": 1e-2}
    torch.testing.assert_close(out.float(), want.float(), **t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [1, 8, 13, 16, 40, 128, 300, 2048])
@pytest.mark.parametrize("inter,k", [(3072, 1024), (176, 80), (48, 64), (112, 96), (1100, 200)])
def test_gemm_swiglu(dtype, m, inter, k) -> None:
    x = rnd(m, k, dtype=dtype, seed=1)
    w = rnd(2 * inter, k, dtype=dtype, seed=2, scale=0.1)
    out = torch.full((m, inter), float("nan"), device="cuda", dtype=dtype)
    want = torch.empty(m, inter, device="cuda", dtype=dtype)
    ops.gemm_swiglu(x, w, out, Arena("cuda"))
    ref.gemm_swiglu(x, w, want)
    t = {"atol": 1e-4, "rtol": 1e-4} if dtype == torch.float32 else {"atol": 3e-2, "rtol": 3e-2}
    torch.testing.assert_close(out.float(), want.float(), **t)


@pytest.mark.parametrize("m", [128, 300, 1152, 2048])
@pytest.mark.parametrize("inter,k", [(3072, 1024), (1024, 64), (1100, 200), (12288, 4096)])
def test_gemm_swiglu_by_pairs_of_ctas(m, inter, k, monkeypatch) -> None:
    """The tcgen05 product with the activation in its epilogue, 256 x 256 tiles by pairs of CTAs: the even
    CTA of a pair loads the gate rows, the odd one the up rows."""
    monkeypatch.setattr(ops, "TCGEN05_PAIR", True)
    monkeypatch.setattr(ops, "TCGEN05_MIN_FILL", 0.0)
    monkeypatch.setattr(ops, "TCGEN05_MIN_COLS", 0)
    x = rnd(m, k, dtype=torch.bfloat16, seed=1)
    w = rnd(2 * inter, k, dtype=torch.bfloat16, seed=2, scale=0.1 if k < 2048 else 0.03)
    out = torch.full((m, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
    want = torch.empty_like(out)
    ops.gemm_swiglu(x, w, out, Arena("cuda"))
    ops.check_device_errors()
    ref.gemm_swiglu(x, w, want)
    torch.testing.assert_close(out.float(), want.float(), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("m", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(1024, 2048), (1024, 3072), (96, 64), (2048, 1024), (48, 1024)])
def test_gemm_to_stream_and_normed(m, n, k) -> None:
    """The two halves of the norm fusion against the separate steps: a product that adds its
    bf16 result to the 32-bit stream and leaves the rows' sums of squares, then a product (plain
    and SwiGLU) that normalises the stream while it loads it."""
    bf = torch.bfloat16
    x = rnd(m, k, dtype=bf, seed=1)
    w = rnd(n, k, dtype=bf, seed=2, scale=0.05)
    resid = rnd(m, n, seed=3, scale=2.0)
    before = resid.clone()
    sumsq = torch.full((2 * n,), float("nan"), device="cuda")
    resid16 = torch.full((m, n), float("nan"), device="cuda", dtype=bf)
    sumsq = ops.gemm_to_stream(x, w, resid, resid16, sumsq)
    assert sumsq.shape[0] == m and sumsq.shape[1] in (n // 16, n // 8)
    delta = torch.empty(m, n, device="cuda", dtype=bf)
    ref.gemm(x, w, delta)
    want_resid = before + delta.float()
    torch.testing.assert_close(resid, want_resid, atol=2e-2, rtol=2e-2)
    assert torch.equal(resid16, resid.to(bf))
    parts = sumsq.sum(1)
    torch.testing.assert_close(parts, (resid * resid).sum(1), atol=1e-3, rtol=1e-4)
    if n % 32:
        return      # the consumer contracts over n: it needs a multiple of 32
    # consumer: norm of the stream inside the next product. The fused kernel rounds at other
    # points than the separate kernels, so both are held against the exact result: the fused error
    # may not exceed that of the separate bf16 path by more than a quarter (rms) / a factor 2 (max)
    nw = (1 + rnd(n, seed=5, scale=0.2)).to(bf)
    normed = torch.empty(m, n, device="cuda", dtype=bf)
    ref.add_rms_norm(resid.clone(), None, nw, 1e-6, normed)
    exact = resid.double() * torch.rsqrt(resid.double().pow(2).mean(-1, keepdim=True) + 1e-6) * nw.double()

    def held(out, want, truth):
        err, err_ref = (out.double() - truth).abs(), (want.double() - truth).abs()
        assert err.pow(2).mean().sqrt() <= 1.25 * err_ref.pow(2).mean().sqrt() + 1e-3
        assert err.max() <= 2 * err_ref.max() + 1e-2

    for n2 in (64, 1536, 3072):
        w2 = rnd(n2, n, dtype=bf, seed=6, scale=0.05)
        for out_dtype in (bf, torch.float32):
            out = torch.full((m, n2), float("nan"), device="cuda", dtype=out_dtype)
            want = torch.empty(m, n2, device="cuda", dtype=out_dtype)
            ops.gemm_normed(resid16, sumsq, nw, 1e-6, w2, out)
            ref.gemm(normed, w2, want)
            held(out, want, exact @ w2.double().t())
        wgu = rnd(2 * n2, n, dtype=bf, seed=7, scale=0.05)
        out = torch.full((m, n2), float("nan"), device="cuda", dtype=bf)
        want = torch.empty(m, n2, device="cuda", dtype=bf)
        ops.gemm_normed(resid16, sumsq, nw, 1e-6, wgu, out, swiglu=True)
        ref.gemm_swiglu(normed, wgu, want)
        gu = exact @ wgu.double().t()
        held(out, want, torch.nn.functional.silu(gu[:, :n2]) * gu[:, n2:])


@pytest.mark.parametrize("m", [9, 16])
def test_gemm_skinny_streaming_form_with_wide_rows(m) -> None:
    """The streaming form keeps the rows of x in shared memory; at a width of 4,096 they leave room
    for one CTA an SM only."""
    n, k = 75808, 4096
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=1), rnd(n, k, dtype=torch.bfloat16, seed=2, scale=0.02)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
    want = torch.empty_like(out)
    ops.gemm_skinny(x, w, out)
    ref.gemm(x, w, want)
    torch.testing.assert_close(out, want, atol=2e-4, rtol=1e-4)


def test_gemm_skinny_refuses_what_it_cannot_take() -> None:
    x, w = rnd(4, 80, dtype=torch.bfloat16), rnd(32, 80, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.gemm_skinny(x, w, torch.empty(4, 32, device="cuda", dtype=torch.bfloat16))
    out = torch.empty(4, 32, device="cuda", dtype=torch.bfloat16)
    ops.gemm(x, w, out)                                   # the general entry takes another kernel
    want = torch.empty_like(out)
    ref.gemm(x, w, want)
    torch.testing.assert_close(out.float(), want.float(), atol=5e-2, rtol=2e-2)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tile_n", [64, 128, 256, ops.TCGEN05_PAIR_TILE])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (128, 256, 256), (1, 72, 80), (200, 1000, 1024), (2048, 4096, 1024),
                                   (300, 1024, 3072), (77, 151936, 1024), (129, 130, 136)])
def test_gemm_tcgen05(out_dtype, tile_n, m, n, k) -> None:
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=1), rnd(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype)
    want = torch.empty(m, n, device="cuda", dtype=out_dtype)
    ops.gemm_tcgen05(x, w, out, tile_n)
    ops.check_device_errors()
    ref.gemm(x, w, want)
    t = {"atol": 2e-4, "rtol": 1e-4} if out_dtype == torch.float32 else {"atol": 2e-2, "rtol": 1e-2}
    torch.testing.assert_close(out.float(), want.float(), **t)


def test_gemm_fp32_row_does_not_depend_on_batch() -> None:
    x, w = rnd(70, 200, seed=1), rnd(333, 200, seed=2)
    full = torch.empty(70, 333, device="cuda")
    one = torch.empty(1, 333, device="cuda")
    ops.gemm(x, w, full)
    ops.gemm(x[41:42].contiguous(), w, one)
    assert torch.equal(full[41:42], one)


@pytest.mark.parametrize("vocab", [301, 4096, 151936])
def test_sample_greedy(vocab) -> None:
    logits = rnd(9, vocab, seed=3)
    logits[2, 17] = logits[2, 200] = 50.0      # a tie: the first index wins
    out = torch.empty(9, device="cuda", dtype=torch.int32)
    ops.sample(logits, out)
    assert out.tolist() == logits.argmax(-1).tolist()
    assert out[2].item() == 17


@pytest.mark.parametrize("vocab", [301, 5000])
def test_sample_temperature_and_top_p_match_reference(vocab) -> None:
    r = 12
    logits = rnd(r, vocab, seed=4, scale=2.0)
    temps = torch.tensor([0.0, 0.8, 1.0, 1.5] * 3, device="cuda")
    top_p = torch.tensor([1.0] * 4 + [0.9] * 4 + [0.3] * 4, device="cuda")
    seeds = torch.arange(r, device="cuda", dtype=torch.int64) * 7919 + (1 << 40)
    for draw in (0, 1, 5):
        draws = torch.full((r,), draw, device="cuda", dtype=torch.int64)
        out, want = (torch.empty(r, device="cuda", dtype=torch.int32) for _ in range(2))
        ops.sample(logits, out, temps, top_p, seeds, draws)
        ref.sample(logits, want, temps, top_p, seeds, draws)
        assert out.tolist() == want.tolist()


def test_sample_frequencies_follow_softmax() -> None:
    vocab, n = 8, 4096
    row = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, -3.0, 1.5, 0.2], device="cuda")
    logits = row.repeat(n, 1).contiguous()
    temps = torch.full((n,), 0.7, device="cuda")
    seeds = torch.arange(n, device="cuda", dtype=torch.int64)
    out = torch.empty(n, device="cuda", dtype=torch.int32)
    counts = torch.zeros(vocab, device="cuda")
    for draw in range(4):                                  # 16,384 independent draws
        draws = torch.full((n,), draw, device="cuda", dtype=torch.int64)
        ops.sample(logits, out, temps, None, seeds, draws)
        counts += torch.bincount(out.long(), minlength=vocab).float()
    freq = counts / (4 * n)
    torch.testing.assert_close(freq, torch.softmax(row / 0.7, -1), atol=0.015, rtol=0)
    draws = torch.zeros(n, device="cuda", dtype=torch.int64)
    # nucleus: only the tokens whose more likely tokens hold < 0.6 may appear
    top_p = torch.full((n,), 0.6, device="cuda")
    ops.sample(logits, out, temps, top_p, seeds, draws)
    p = torch.softmax(row / 0.7, -1)
    order = p.argsort(descending=True)
    above = p[order].cumsum(0) - p[order]
    allowed = set(order[above < 0.6].tolist())
    assert set(out.unique().tolist()) == allowed


def test_prefetch_l2_reads_only() -> None:
    """Prefetch requests change nothing that can be seen: they run (ragged sizes, a side stream
    joined again) and the memory reads as before; more than 8 ranges are refused."""
    ts = [rnd(1000, 1024, dtype=torch.bfloat16, seed=1), rnd(3, 5, seed=2), rnd(16 * 1024 + 8, seed=3)]
    before = [t.clone() for t in ts]
    ops.prefetch_l2(ts)
    join = ops.prefetch_l2_beside(ts + [None])
    join()
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(ts, before))
    with pytest.raises(ops.KernelError, match="at most 8"):
        ops.prefetch_l2([ts[1]] * 9)


def test_timeline_is_empty_without_the_timeline_build() -> None:
    """The library that tests and timings use carries no clock notes (they cost an atomic and two
    stores a launch); the call itself works and says so by returning nothing."""
    x = torch.zeros(4, 64, device="cuda")
    ops.silu_mul(x.to(torch.bfloat16), torch.empty(4, 32, device="cuda", dtype=torch.bfloat16))
    assert ops.build.TIMELINE or ops.timeline() == []



def test_index_checks_refuse_a_corrupted_table_before_any_launch(monkeypatch) -> None:
    """With the index checks on, a block-table entry or a cache slot that points outside the cache
    is refused on the host, before a kernel could follow it; entries that no request reaches may
    hold anything."""
    monkeypatch.setattr(ops, "CHECK_INDICES", True)
    dtype, hq, hkv, d, page, pages = torch.bfloat16, 4, 2, 64, 16, 8
    k_cache = rnd(pages, hkv, page, d, dtype=dtype, seed=1)
    v_cache = rnd(pages, hkv, page, d, dtype=dtype, seed=2)
    q = rnd(2, hq, d, dtype=dtype, seed=3)
    lens = [40, 17]
    tables = torch.tensor([[0, 1, 2, 10_000], [3, 4, 10_000, -5]], dtype=torch.int32, device="cuda")

    def ctx():
        return SimpleNamespace(
            num_seqs=2, query_lens=[1, 1], cu_query_lens=torch.tensor([0, 1, 2], dtype=torch.int32, device="cuda"),
            context_lens_dev=torch.tensor(lens, dtype=torch.int32, device="cuda"),
            decode_seqs=torch.tensor([0, 1], dtype=torch.int32, device="cuda"),
            prefill_seqs=torch.zeros(2, dtype=torch.int32, device="cuda"), num_decode=2, num_prefill=0,
            max_query_len=1, max_context_len=max(lens), arena=Arena("cuda"))

    out, want = torch.empty(2, hq * d, device="cuda", dtype=dtype), torch.empty(2, hq * d, device="cuda", dtype=dtype)
    ops.paged_attention(q, k_cache, v_cache, page, tables, ctx(), d ** -0.5, 0, out)      # the bad entries are out of reach
    ref.paged_attention(q, k_cache, v_cache, page, tables, ctx(), d ** -0.5, 0, want)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))
    tables[1, 1] = 8                                                                       # the cache has pages 0..7
    with pytest.raises(ops.KernelError, match="request 1, entry 1 is page 8"):
        ops.paged_attention(q, k_cache, v_cache, page, tables, ctx(), d ** -0.5, 0, out)
    tables[1, 1] = 4
    lens[0] = 70                                                                           # needs five pages of a table of four
    with pytest.raises(ops.KernelError, match="needs 5 pages"):
        ops.paged_attention(q, k_cache, v_cache, page, tables, ctx(), d ** -0.5, 0, out)
    qkv = rnd(2, (hq + 2 * hkv) * d, dtype=dtype, seed=4)
    slots = torch.tensor([5, pages * page], dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="cache slot 128 is outside"):
        ops.qk_norm_rope_write(qkv, torch.empty(2, hq, d, device="cuda", dtype=dtype), None, None, 1e-6, None, None, 0,
                               False, slots, k_cache, v_cache, page, hq, hkv, d, True)
    torch.cuda.synchronize()
