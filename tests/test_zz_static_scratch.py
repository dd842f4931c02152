"""The entry point that allocates nothing (``ts_decode_attention_static_scratch``): called
through its exported C symbol, its output must equal the regular entry point's, twice in a
row (the second call finds the first call's leftovers in the fixed scratch array), and a job
too large for that array must be refused without a launch. Collected last on purpose."""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

TS_STATIC_SCRATCH_FLOATS = 2 * 1024 * 1024
TS_ERR_SCRATCH_TOO_SMALL = -3
TS_ERR_BAD_ARGUMENT = -1


def _lib():
    from tinyserve_b200.kernels import build

    lib = build.library()
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = lib.ts_decode_attention_static_scratch
    fn.argtypes = [vp, vp, vp, vp, vp, i, vp, vp, vp, i, i, i, i, i, f, i, i, i, vp]
    fn.restype = i
    need = lib.ts_decode_attention_static_scratch_need
    need.argtypes = [i, i, i, i]
    need.restype = ctypes.c_longlong
    return fn, need


def _case(dtype, b, hq, hkv, d, page, lens, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    need = [-(-c // page) for c in lens]
    pages = sum(need) + 3
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    tables = torch.zeros(b, max(need), dtype=torch.int32)
    at = 0
    for r, n in enumerate(need):
        tables[r, :n] = torch.tensor(perm[at: at + n])
        at += n
    k = torch.randn(pages, hkv, page, d, generator=g, device="cuda").to(dtype)
    v = torch.randn(pages, hkv, page, d, generator=g, device="cuda").to(dtype)
    q = torch.randn(b, hq, d, generator=g, device="cuda").to(dtype)
    cu = torch.arange(b + 1, dtype=torch.int32, device="cuda")
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    seqs = torch.arange(b, dtype=torch.int32, device="cuda")
    return q, k, v, tables.cuda(), cu, ctx, seqs


def _plain(q, k, v, tables, lens, page, hq, hkv, d, window):
    """Attention of one query per request over its pages, written out in float32 (an oracle that
    shares nothing with the library)."""
    out = torch.empty(len(lens), hq * d, device="cuda")
    for r, c in enumerate(lens):
        lo = max(0, c - window) if window else 0
        pos = torch.arange(lo, c, device="cuda")
        pg = tables[r, pos // page].long()
        kk = k[pg, :, pos % page].float()                     # [keys, hkv, d]
        vv = v[pg, :, pos % page].float()
        qq = q[r].float().view(hkv, hq // hkv, d)
        s = torch.einsum("hgd,khd->hgk", qq, kk) * d ** -0.5
        out[r] = torch.einsum("hgk,khd->hgd", torch.softmax(s, -1), vv).reshape(-1)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d,splits,window", [(8, 2, 64, 6, 0), (8, 2, 64, 6, 37), (8, 2, 64, 1, 0),
                                                      (40, 2, 32, 5, 0)])
def test_static_scratch_entry_point_matches_the_regular_one(dtype, hq, hkv, d, splits, window) -> None:
    """Both entry points run the same kernels with the same key ranges and a merge in a fixed order,
    so their outputs must be equal bit for bit: a stale or half-overwritten element of the shared
    scratch array would show. ``splits`` 1 uses no scratch at all (null pointers inside); 40 / 2
    heads need three passes over a kv group. One float32 oracle written out here guards both."""
    from tinyserve_b200.kernels import ops

    fn, need = _lib()
    b, page = 5, 16
    code = 0 if dtype == torch.float32 else 1
    stream = torch.cuda.current_stream().cuda_stream
    assert 0 <= need(b, hq, d, splits) <= TS_STATIC_SCRATCH_FLOATS
    for call, lens in enumerate(([700, 33, 1, 257, 512], [90, 640, 300, 17, 1000])):
        q, k, v, tables, cu, ctx, seqs = _case(dtype, b, hq, hkv, d, page, lens, seed=call)
        got = torch.full((b, hq * d), float("nan"), device="cuda", dtype=dtype)
        st = fn(q.data_ptr(), got.data_ptr(), k.data_ptr(), v.data_ptr(), tables.data_ptr(), tables.shape[1],
                cu.data_ptr(), ctx.data_ptr(), seqs.data_ptr(), b, hq, hkv, d, page, d ** -0.5, window, splits, code,
                stream)
        assert st == 0
        # the regular entry point, with scratch from the caller and the same number of key ranges
        want = torch.empty_like(got)
        acc = torch.empty(b, hq, splits, d, device="cuda")
        ml = torch.empty(b, hq, splits, 2, device="cuda")
        st = ops._fn("ts_paged_attention_simt")(
            q.data_ptr(), want.data_ptr(), k.data_ptr(), v.data_ptr(), tables.data_ptr(), tables.shape[1],
            cu.data_ptr(), ctx.data_ptr(), seqs.data_ptr(), b, seqs.data_ptr(), 0, 1, hq, hkv, d, page,
            d ** -0.5, window, splits, acc.data_ptr() if splits > 1 else None, ml.data_ptr() if splits > 1 else None,
            code, stream)
        assert st == 0
        torch.cuda.synchronize()
        assert not got.isnan().any()
        assert torch.equal(got, want)
        tol = {"atol": 1e-5, "rtol": 1e-5} if dtype == torch.float32 else {"atol": 2e-2, "rtol": 2e-2}
        torch.testing.assert_close(got.float(), _plain(q, k, v, tables, lens, page, hq, hkv, d, window), **tol)


def test_static_scratch_refuses_what_does_not_fit() -> None:
    """Too much scratch, or more key ranges than any decode launcher of the library takes (32: the
    merge stages two floats per range in shared memory sized for that many): an error code and no
    launch."""
    fn, need = _lib()
    b, hq, d, splits = 64, 32, 128, 32
    assert need(b, hq, d, splits) > TS_STATIC_SCRATCH_FLOATS
    x = torch.zeros(16, device="cuda")
    p = x.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    st = fn(p, p, p, p, p, 1, p, p, p, b, hq, 8, d, 16, 1.0, 0, splits, 1, stream)
    assert st == TS_ERR_SCRATCH_TOO_SMALL
    assert need(1, 4, 16, 40) <= TS_STATIC_SCRATCH_FLOATS
    st = fn(p, p, p, p, p, 1, p, p, p, 1, 4, 2, 16, 16, 1.0, 0, 40, 1, stream)
    assert st == TS_ERR_BAD_ARGUMENT
    torch.cuda.synchronize()
