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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_matches_the_regular_one(dtype) -> None:
    from tinyserve_b200.kernels import ops

    fn, need = _lib()
    b, hq, hkv, d, page, splits = 5, 8, 2, 64, 16, 6
    code = 0 if dtype == torch.float32 else 1
    stream = torch.cuda.current_stream().cuda_stream
    assert 0 < need(b, hq, d, splits) <= TS_STATIC_SCRATCH_FLOATS
    for call, lens in enumerate(([700, 33, 1, 257, 512], [90, 640, 300, 17, 1000])):
        q, k, v, tables, cu, ctx, seqs = _case(dtype, b, hq, hkv, d, page, lens, seed=call)
        got = torch.full((b, hq * d), float("nan"), device="cuda", dtype=dtype)
        st = fn(q.data_ptr(), got.data_ptr(), k.data_ptr(), v.data_ptr(), tables.data_ptr(), tables.shape[1],
                cu.data_ptr(), ctx.data_ptr(), seqs.data_ptr(), b, hq, hkv, d, page, d ** -0.5, 0, splits, code, stream)
        assert st == 0
        # the regular entry point, with scratch from the caller and the same number of key ranges
        want = torch.empty_like(got)
        acc = torch.empty(b, hq, splits, d, device="cuda")
        ml = torch.empty(b, hq, splits, 2, device="cuda")
        st = ops._fn("ts_paged_attention_simt")(
            q.data_ptr(), want.data_ptr(), k.data_ptr(), v.data_ptr(), tables.data_ptr(), tables.shape[1],
            cu.data_ptr(), ctx.data_ptr(), seqs.data_ptr(), b, seqs.data_ptr(), 0, 1, hq, hkv, d, page,
            d ** -0.5, 0, splits, acc.data_ptr(), ml.data_ptr(), code, stream)
        assert st == 0
        torch.cuda.synchronize()
        assert not got.isnan().any()
        tol = {"atol": 1e-5, "rtol": 1e-5} if dtype == torch.float32 else {"atol": 2e-2, "rtol": 2e-2}
        torch.testing.assert_close(got.float(), want.float(), **tol)


def test_static_scratch_refuses_what_does_not_fit() -> None:
    fn, need = _lib()
    b, hq, d, splits = 64, 32, 128, 32
    assert need(b, hq, d, splits) > TS_STATIC_SCRATCH_FLOATS
    x = torch.zeros(16, device="cuda")
    p = x.data_ptr()
    st = fn(p, p, p, p, p, 1, p, p, p, b, hq, 8, d, 16, 1.0, 0, splits, 1, torch.cuda.current_stream().cuda_stream)
    assert st == TS_ERR_SCRATCH_TOO_SMALL
    torch.cuda.synchronize()
