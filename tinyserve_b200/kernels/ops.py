"""The operations of the product path, each one a hand-written sm_100a kernel (or, for the
plain bf16 matrix products, the vendor library, as the upstream engine uses one there).

Every function checks its arguments on the host, then launches on the current CUDA stream.
There is no CPU implementation and no alternative backend: without a CUDA device or the
compiled library these functions raise. Tensors are contiguous; ``dt`` below is the model
dtype (bfloat16 or float32) and selects the kernel instantiation.
"""

from __future__ import annotations

import ctypes
import math
import os
from typing import Any, Callable, Sequence

import torch

from . import build

_F32, _BF16 = 0, 1
_c = ctypes
_vp, _i, _f = _c.c_void_p, _c.c_int, _c.c_float


class KernelError(RuntimeError):
    """A kernel refused its arguments or the launch failed."""


_SIGNATURES: dict[str, list[Any]] = {
    "ts_embed": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ts_add_rms_norm": [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp],
    "ts_rope_tables": [_vp, _vp, _vp, _vp, _i, _i, _vp],
    "ts_silu_mul": [_vp, _vp, _i, _i, _i, _vp],
    "ts_qk_norm_rope_write": [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "ts_paged_attention_simt": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i,
                                _f, _i, _i, _vp, _vp, _i, _vp],
    "ts_prefill_attention_mma": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ts_decode_attention_mma": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp,
                                _vp, _vp],
    "ts_decode_attention_mma_slots": [_i],
    "ts_decode_attention_tma": [_vp, _vp, _vp, _vp, _c.c_longlong, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i,
                                _i, _vp, _vp, _vp, _vp],
    "ts_decode_attention_tma_fused": [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _c.c_longlong, _vp, _i, _vp,
                                      _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _vp, _vp, _vp],
    "ts_decode_attention_tma_slots": [_i],
    "ts_prefill_attention_tma": [_vp, _vp, _vp, _vp, _c.c_longlong, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f,
                                 _i, _vp, _vp],
    "ts_prefill_attention_tcgen05": [_vp, _vp, _vp, _vp, _c.c_longlong, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                     _f, _i, _i, _vp, _vp],
    "ts_gemm_skinny_normed": [_vp, _vp, _i, _vp, _f, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ts_gemm_skinny_to_stream": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "ts_gemm_skinny_to_stream_parts": [_i, _i, _i],
    "ts_prefetch_l2": [_vp, _vp, _i, _i, _vp],
    "ts_prefetch_pages": [_vp, _vp, _c.c_ulonglong, _vp, _i, _vp, _i, _i, _i, _vp],
    "ts_gemm_simt": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ts_gemm_skinny": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ts_gemm_skinny_swiglu": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "ts_gemm_tcgen05": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "ts_gemm_tcgen05_swiglu": [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "ts_sample": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
}
_fns: dict[str, Any] = {}

# Kernel classes launched with programmatic dependent launch in decode steps. Up to 16 rows: all
# classes (the L2 prefetch kernel then starts beside the product before it, and nothing small is
# left that loses from starting early); beyond: the skinny product and the attention kernels.
# Measured on B200 in the recorded decode step of Qwen3-0.6B, all classes against those two:
# batch 8 1.046 / 1.112 ms, 16 1.736 / 1.776 ms, 32 1.839 / 1.796 ms, 64 2.719 / 2.690 ms.
DEFAULT_PDL_MASK = 2 | 4
SMALL_DECODE_PDL_MASK = -1
SMALL_DECODE_ROWS = 16


def decode_pdl_mask(rows: int) -> int:
    return SMALL_DECODE_PDL_MASK if rows <= SMALL_DECODE_ROWS else DEFAULT_PDL_MASK


# Steps that carry prompt portions run large kernels, where starting early costs nothing and
# hides the launch: all classes (2,048-token prefill of Qwen3-0.6B: 7.7 ms against 8.1 ms).
PREFILL_PDL_MASK = -1
_pdl_mask = DEFAULT_PDL_MASK


def use_pdl_mask(mask: int) -> None:
    """Switch the launch-overlap mask if it differs from the current one (cheap to call per step)."""
    global _pdl_mask
    if mask != _pdl_mask:
        set_programmatic_launch(mask)

# Kernels of this library launched so far (library matrix products are not counted).
launch_count = 0


def _fn(name: str) -> Any:
    f = _fns.get(name)
    if f is None:
        lib = build.library()
        if not _fns:
            # first use of the library: overlap the launches of the kernel classes that gain from it
            lib.ts_set_programmatic_launch.argtypes = [_i]
            lib.ts_set_programmatic_launch.restype = None
            lib.ts_set_programmatic_launch(_pdl_mask)      # the default, or what the caller has set already
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = _i
        _fns[name] = f
    return f


def _check(status: int, name: str, kernels: int = 1) -> None:
    global launch_count
    if status == 0:
        launch_count += kernels
        return
    if status == -1:
        raise KernelError(f"{name}: bad argument")
    if status == -2:
        raise KernelError(f"{name}: size not supported by this kernel")
    if status == -3:
        raise KernelError(f"{name}: the job needs more scratch than the library's fixed array holds")
    raise KernelError(f"{name}: CUDA error {status}")


_stream_stack: list[int] = []


def _stream() -> int:
    if _stream_stack:
        return _stream_stack[-1]
    return torch.cuda.current_stream().cuda_stream


class stream_scope:
    """While it is open, this library's kernels go to the stream that was current when it was
    opened, without asking for the current stream at every launch (that query costs several
    microseconds, as much as the launch). Open it around a step's launches; inside it, change
    the stream only through another ``stream_scope`` opened under the new stream."""

    def __enter__(self) -> "stream_scope":
        _stream_stack.append(torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0)
        return self

    def __exit__(self, *exc: Any) -> None:
        _stream_stack.pop()


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return _F32
    if dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"dtype {dtype} is not supported (float32 or bfloat16)")


def _dev(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t: torch.Tensor | None, name: str, dtype: torch.dtype | None = None) -> int | None:
    return None if t is None else _dev(t, name, dtype)


# ------------------------------------------------------------------ elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t] = float32(table[tokens[t]])``; tokens int32 ``[T]``, table ``[V, h]`` dt."""
    t, h = out.shape
    if tokens.shape != (t,) or table.shape[1] != h:
        raise KernelError(f"embed: shapes {tuple(tokens.shape)}, {tuple(table.shape)}, {tuple(out.shape)}")
    _check(_fn("ts_embed")(_dev(tokens, "tokens", torch.int32), _dev(table, "table"),
                           _dev(out, "out", torch.float32), t, h, table.shape[0], _code(table.dtype),
                           _stream()), "embed")


def add_rms_norm(resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                 out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """``x = resid (+ delta)``; ``out = dt(x * rsqrt(mean(x^2) + eps)) * weight``.

    Without ``rows`` every row is processed and the sum is written back to ``resid``
    (float32). With ``rows`` (int32) only those rows are read, ``out`` has one row per entry
    and ``resid`` is left unchanged."""
    h = resid.shape[1]
    n = out.shape[0]
    dt = out.dtype
    if weight.shape != (h,) or out.shape[1] != h or (delta is not None and delta.shape != resid.shape):
        raise KernelError("add_rms_norm: shape mismatch")
    if rows is None and n != resid.shape[0]:
        raise KernelError("add_rms_norm: out must have one row per row of resid")
    if rows is not None and rows.shape != (n,):
        raise KernelError("add_rms_norm: rows must have one entry per row of out")
    _check(_fn("ts_add_rms_norm")(_dev(resid, "resid", torch.float32), _opt(delta, "delta", dt),
                                  _dev(weight, "weight", dt), _dev(out, "out"),
                                  _opt(rows, "rows", torch.int32), n, h, float(eps), _code(dt), _stream()),
           "add_rms_norm")


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    """``cos/sin[t, i] = float32(cos/sin(float64(positions[t]) * inv_freq[i]))``."""
    t, half = cos.shape
    if positions.shape != (t,) or inv_freq.shape != (half,) or sin.shape != cos.shape:
        raise KernelError("rope_tables: shape mismatch")
    _check(_fn("ts_rope_tables")(_dev(positions, "positions", torch.int32), _dev(inv_freq, "inv_freq", torch.float64),
                                 _dev(cos, "cos", torch.float32), _dev(sin, "sin", torch.float32), t, half,
                                 _stream()), "rope_tables")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, j] = dt(silu(gate_up[t, j])) * gate_up[t, I + j]``."""
    t, inter = out.shape
    if gate_up.shape != (t, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("silu_mul: shape or dtype mismatch")
    _check(_fn("ts_silu_mul")(_dev(gate_up, "gate_up"), _dev(out, "out"), t, inter, _code(out.dtype), _stream()),
           "silu_mul")


def qk_norm_rope_write(qkv: torch.Tensor, q_out: torch.Tensor, q_weight: torch.Tensor | None,
                       k_weight: torch.Tensor | None, eps: float, cos: torch.Tensor | None,
                       sin: torch.Tensor | None, rotary_dim: int, interleaved: bool, slots: torch.Tensor,
                       k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int, num_heads: int,
                       num_kv_heads: int, head_dim: int, write_kv: bool) -> None:
    """Per (token, head): optional RMSNorm over ``head_dim``, optional rotation of the first
    ``rotary_dim`` elements; q heads go to ``q_out``, k and v heads to the cache at the token's
    slot (only when ``write_kv``; then ``qkv`` rows hold q, k and v, else q alone)."""
    t = q_out.shape[0]
    dt = q_out.dtype
    width = (num_heads + 2 * num_kv_heads) * head_dim if write_kv else num_heads * head_dim
    if qkv.shape != (t, width) or qkv.dtype != dt or tuple(q_out.shape) != (t, num_heads, head_dim):
        raise KernelError("qk_norm_rope_write: qkv/q_out shape or dtype mismatch")
    if k_cache.dtype != dt or v_cache.dtype != dt or k_cache.shape != v_cache.shape:
        raise KernelError("qk_norm_rope_write: cache dtype/shape mismatch")
    if tuple(k_cache.shape[1:]) != (num_kv_heads, page_size, head_dim):
        raise KernelError("qk_norm_rope_write: cache layout must be [pages, kv_heads, page_size, head_dim]")
    if rotary_dim and (cos is None or sin is None or tuple(cos.shape) != (t, rotary_dim // 2)):
        raise KernelError("qk_norm_rope_write: rotary tables missing or of the wrong shape")
    if slots.shape != (t,):
        raise KernelError("qk_norm_rope_write: one slot per token")
    if write_kv:
        _check_indices("qk_norm_rope_write", None, None, page_size, k_cache.shape[0], slots)
    _check(_fn("ts_qk_norm_rope_write")(
        _dev(qkv, "qkv"), _dev(q_out, "q_out"), _opt(q_weight, "q_weight", dt), _opt(k_weight, "k_weight", dt),
        float(eps), _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), int(rotary_dim),
        int(bool(interleaved)), _dev(slots, "slots", torch.int32), _dev(k_cache, "k_cache"),
        _dev(v_cache, "v_cache"), page_size, t, num_heads, num_kv_heads, head_dim, int(bool(write_kv)),
        _code(dt), _stream()), "qk_norm_rope_write")


# ------------------------------------------------------------------ index checks
# TINYSERVE_B200_CHECK_INDICES=1 (or ``ops.CHECK_INDICES = True``): before a kernel that follows
# block tables or cache slots is launched, the step's indices are read back and checked on the
# host: every block-table entry that the launch can reach names a page of the cache, every slot
# lies inside it. A violation raises ``KernelError`` and nothing is launched, so a corrupted table
# never becomes a read outside the cache. Each check waits for the device: a debugging aid, off in
# serving (the launchers' own host checks of shapes, sizes and alignment are always on). It plays
# the part that device-side index asserts play in a debug build, without a device trap.
CHECK_INDICES = os.environ.get("TINYSERVE_B200_CHECK_INDICES", "") not in ("", "0")


def _check_indices(name: str, block_tables: torch.Tensor | None, ctx: Any, page_size: int, num_pages: int,
                   slots: torch.Tensor | None = None) -> None:
    if not CHECK_INDICES:
        return
    if torch.cuda.is_current_stream_capturing():
        return                       # nothing can be read back while a step is being recorded
    if block_tables is not None:
        lens = ctx.context_lens_dev[: ctx.num_seqs].to(torch.int64)
        if int(lens.min()) < 1:
            raise KernelError(f"{name}: a request of the step holds no token")
        need = (lens + page_size - 1) // page_size
        if int(need.max()) > block_tables.shape[1]:
            raise KernelError(f"{name}: a request needs {int(need.max())} pages, its block table holds {block_tables.shape[1]}")
        cols = torch.arange(block_tables.shape[1], device=block_tables.device)[None, :]
        used = cols < need[:, None]
        bad = used & ((block_tables < 0) | (block_tables >= num_pages))
        if bool(bad.any()):
            row, col = [int(v) for v in bad.nonzero()[0]]
            raise KernelError(f"{name}: block table of request {row}, entry {col} is page {int(block_tables[row, col])}; "
                              f"the cache has pages 0..{num_pages - 1}")
    if slots is not None and slots.numel():
        lo, hi = int(slots.min()), int(slots.max())
        if lo < 0 or hi >= num_pages * page_size:
            raise KernelError(f"{name}: cache slot {lo if lo < 0 else hi} is outside 0..{num_pages * page_size - 1}")


# -------------------------------------------------------------------- attention
# The bf16 prefill kernel for head sizes 64 / 128: "tcgen05" (tensor memory accumulators) or "mma"
# (mma.sync with TMA tiles); and how many query heads of a kv group share a CTA of the former and
# its key / value tiles (0: chosen by the size of the grid, see ``_prefill_heads_per_cta``).
PREFILL_ATTENTION = "tcgen05"
PREFILL_HEADS_PER_CTA = 0
TARGET_DECODE_CTAS = 148 * 4
MIN_KEYS_PER_SPLIT = 64
MAX_SPLITS = 32


def _prefill_heads_per_cta(ctx: Any, num_heads: int, num_kv_heads: int) -> int:
    """Two query heads of a kv group in a CTA share its key and value tiles, which is worth more
    than anything once the pairs alone give every SM a CTA (measured on B200, 16 / 8 heads of 128:
    2,048 tokens 39 us with one head, 46 us with two; 3,072 tokens 79 / 64 us; 8,192 tokens
    428 / 292 us)."""
    if (num_heads // num_kv_heads) % 2:
        return 1
    if PREFILL_HEADS_PER_CTA:
        return PREFILL_HEADS_PER_CTA
    tiles = sum(-(-n // 128) for n in ctx.query_lens if n > 1)
    return 2 if tiles * (num_heads // 2) > 148 else 1


def decode_splits(num_decode: int, num_kv_heads: int, group: int, max_context_len: int) -> int:
    """How many ranges the keys of each decoding request are cut into. Depends only on the
    shape of the step (after upstream src/tinyserve/triton_attention.py:499-510)."""
    passes = (group + 7) // 8 if group > 8 else 1
    ctas = max(1, num_decode * num_kv_heads * passes)
    want = -(-TARGET_DECODE_CTAS // ctas)
    most = max(1, max_context_len // MIN_KEYS_PER_SPLIT)
    return max(1, min(want, most, MAX_SPLITS))


CLUSTER_MERGE = True       # the TMA decode kernel merges 2 to 8 key ranges inside a thread-block cluster
CLUSTER_MAX = 8            # the portable cluster size
CLUSTER_ROOM = 18          # CTA slots left free per CTA of a cluster
CLUSTER_FILL = 0.82        # and clusters of three or more fill at most this much of the machine


def choose_splits(ctas: int, slots: int, most: int, cluster: bool = False) -> int:
    """Key ranges per request for a kernel of which ``slots`` CTAs run at once and that would
    launch ``ctas`` CTAs unsplit. A step that already gives most of the machine a CTA is not cut
    (the merge of the ranges costs more than a partly filled last round of CTAs); fewer CTAs are
    cut until they fill the machine, up to 12 ranges (measured on B200 at batch 1 to 64). Depends
    only on the shape of the step, so a recorded step always replays the same grid.

    ``cluster``: the kernel merges the ranges of a request inside a thread-block cluster, which is
    cheaper but needs all CTAs of a cluster to find room on one GPC at the same moment, while the
    kernel before it is still leaving. The more CTAs a cluster has, the more of the machine must
    stay free for that: measured at batch 1 to 24 (16 / 8 heads of 128), the best number of ranges
    was each time the largest s <= 8 with ``s * ctas <= slots - 18 s`` (batch 8: 5 ranges, 0.95 ms
    a step; 6 ranges, which fill 86% of the slots, 1.04 ms; without clusters 1.02 ms; batch 9: 5 ranges
    fill 81%, 0.97 ms, 4 ranges 0.93 ms; batch 7: 6 ranges, 76%, are the best), except at
    batch 16, where 3 ranges pass that rule and fill 86%: 1.31 ms a step, with now and then a layer
    whose attention takes twice as long, against 1.21 ms with 2 ranges. Hence the second bound on
    what clusters of three or more may fill."""
    if 2 * ctas > slots:
        return 1
    if cluster and CLUSTER_MERGE:
        for s in range(min(CLUSTER_MAX, most, MAX_SPLITS), 1, -1):
            if s * ctas <= slots - CLUSTER_ROOM * s and (s == 2 or s * ctas <= CLUSTER_FILL * slots):
                return s
        return 1
    return max(1, min(slots // ctas, most, 12, MAX_SPLITS))


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                    block_tables: torch.Tensor, ctx: Any, scale: float, window: int, out: torch.Tensor) -> None:
    """Causal attention of this step's queries over each request's cached keys and values.

    ``q`` ``[T, Hq, D]`` dt; caches ``[pages, Hkv, page_size, D]`` dt; ``block_tables``
    ``[B, W]`` int32; ``ctx`` supplies ``cu_query_lens``, ``context_lens_dev``, the lists of
    decoding and prefilling requests and the step's maxima. ``window`` 0 means all earlier
    positions. ``out`` ``[T, Hq * D]`` dt."""
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    dt = q.dtype
    if k_cache.dtype != dt or v_cache.dtype != dt or out.dtype != dt:
        raise KernelError("paged_attention: dtype mismatch")
    if tuple(k_cache.shape[1:]) != (hkv, page_size, d) or k_cache.shape != v_cache.shape:
        raise KernelError("paged_attention: cache layout must be [pages, kv_heads, page_size, head_dim]")
    if out.numel() != t * hq * d or hq % hkv:
        raise KernelError("paged_attention: out shape or head grouping")
    if d % 16 or d > 256:
        raise KernelError(f"paged_attention: head_dim={d} must be a multiple of 16 up to 256")
    if block_tables.dim() != 2 or block_tables.shape[0] != ctx.num_seqs:
        raise KernelError("paged_attention: block_tables must be [requests, width]")
    _check_indices("paged_attention", block_tables, ctx, page_size, k_cache.shape[0])
    num_prefill = ctx.num_prefill
    tma_ok = (dt == torch.bfloat16 and d in (64, 128) and (page_size == 8 or page_size % 16 == 0)
              and k_cache.shape[0] * hkv * page_size < 2 ** 31)
    if num_prefill and dt == torch.bfloat16 and d <= 128:
        # prefill rows on the tensor cores; the decode rows follow below
        if tma_ok and PREFILL_ATTENTION == "tcgen05":
            # both products as tcgen05.mma with the accumulators in tensor memory
            _check(_fn("ts_prefill_attention_tcgen05")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), k_cache.shape[0],
                _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
                _dev(ctx.context_lens_dev, "context_lens", torch.int32),
                _dev(ctx.prefill_seqs, "prefill_seqs", torch.int32), num_prefill, ctx.max_query_len,
                hq, hkv, d, page_size, float(scale), int(window),
                _prefill_heads_per_cta(ctx, hq, hkv),
                _error_word(q.device).data_ptr(), _stream()), "prefill_attention_tcgen05")
        elif tma_ok:
            _check(_fn("ts_prefill_attention_tma")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), k_cache.shape[0],
                _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
                _dev(ctx.context_lens_dev, "context_lens", torch.int32),
                _dev(ctx.prefill_seqs, "prefill_seqs", torch.int32), num_prefill, ctx.max_query_len,
                hq, hkv, d, page_size, float(scale), int(window), _error_word(q.device).data_ptr(), _stream()),
                "prefill_attention_tma")
        else:
            _check(_fn("ts_prefill_attention_mma")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
                _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
                _dev(ctx.context_lens_dev, "context_lens", torch.int32),
                _dev(ctx.prefill_seqs, "prefill_seqs", torch.int32), num_prefill, ctx.max_query_len,
                hq, hkv, d, page_size, float(scale), int(window), _stream()), "prefill_attention_mma")
        num_prefill = 0
        if not ctx.num_decode:
            return
    if dt == torch.bfloat16 and d <= 128:
        # decode rows on the tensor cores too: one CTA per (request, kv group, key range)
        ctas = ctx.num_decode * hkv * (-(-(hq // hkv) // 16))
        tma = tma_ok
        slots = _decode_slots(d, tma)
        splits = choose_splits(ctas, slots, ctx.max_context_len // 64, cluster=tma)
        part_acc = part_ml = None
        if splits > 1:
            part_acc = ctx.arena.take((ctx.num_decode, hq, splits, d), torch.float32)
            part_ml = ctx.arena.take((ctx.num_decode, hq, splits, 2), torch.float32)
        common = (_dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                  _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
                  _dev(ctx.context_lens_dev, "context_lens", torch.int32),
                  _dev(ctx.decode_seqs, "decode_seqs", torch.int32), ctx.num_decode,
                  hq, hkv, d, page_size, float(scale), int(window), splits,
                  _opt(part_acc, "part_acc"), _opt(part_ml, "part_ml"), _error_word(q.device).data_ptr(), _stream())
        if tma:
            # tiles fetched by the TMA unit (tensor copies, 128-byte swizzle)
            _check(_fn("ts_decode_attention_tma")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
                k_cache.shape[0], *common), "decode_attention_tma")
        else:
            # tiles fetched row by row with bulk copies
            _check(_fn("ts_decode_attention_mma")(
                _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), *common),
                "decode_attention_mma")
        return
    splits, part_acc, part_ml = 1, None, None
    if ctx.num_decode:
        splits = decode_splits(ctx.num_decode, hkv, hq // hkv, ctx.max_context_len)
        if splits > 1:
            part_acc = ctx.arena.take((ctx.num_decode, hq, splits, d), torch.float32)
            part_ml = ctx.arena.take((ctx.num_decode, hq, splits, 2), torch.float32)
    _check(_fn("ts_paged_attention_simt")(
        _dev(q, "q"), _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
        _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
        _dev(ctx.context_lens_dev, "context_lens", torch.int32),
        _dev(ctx.decode_seqs, "decode_seqs", torch.int32), ctx.num_decode,
        _dev(ctx.prefill_seqs, "prefill_seqs", torch.int32), num_prefill, ctx.max_query_len,
        hq, hkv, d, page_size, float(scale), int(window), splits,
        _opt(part_acc, "part_acc"), _opt(part_ml, "part_ml"), _code(dt), _stream()), "paged_attention",
        kernels=(1 if num_prefill else 0) + (1 if ctx.num_decode else 0))


# The fused decode kernel takes steps of up to this many decode tokens (0 turns it off), and
# only grids that fit the machine at once (and have at least FUSED_DECODE_MIN_CTAS CTAs). Measured
# on B200 (Qwen3-0.6B sizes, 1,024-token contexts): batches 1 to 48 gain 1 to 5 % of the step;
# larger ones (batch 56, 64) repeat the extra work in a second round of CTAs and lose 1 to 4 %.
FUSED_DECODE_MAX_ROWS = 1 << 30
FUSED_DECODE_MIN_CTAS = 0


def can_fuse_decode(ctx: Any, dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                    pages: int, rotary_dim: int, interleaved: bool, device: torch.device) -> bool:
    """Whether :func:`decode_attention_fused` takes this step and gains from it: decode tokens
    only, bf16, a head of 64 or 128, pages of 8 or a multiple of 16 positions, the whole head
    rotated with the rotate-half pairing (or no rotation at all), and a grid that fills the machine
    once. Depends only on the shape of the step, as the choice of the key ranges does."""
    if not (device.type == "cuda" and ctx.num_prefill == 0 and 0 < ctx.num_decode <= FUSED_DECODE_MAX_ROWS
            and dtype == torch.bfloat16 and head_dim in (64, 128) and (page_size == 8 or page_size % 16 == 0)
            and pages * num_kv_heads * page_size < 2 ** 31
            and (rotary_dim == 0 or (rotary_dim == head_dim and not interleaved))):
        return False
    ctas = ctx.num_decode * num_kv_heads * (-(-(num_heads // num_kv_heads) // 16))
    slots = _decode_slots(head_dim, True)
    grid = ctas * choose_splits(ctas, slots, ctx.max_context_len // 64, cluster=True)
    return min(FUSED_DECODE_MIN_CTAS, slots) <= grid <= slots


def decode_attention_fused(qkv: torch.Tensor, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                           eps: float, cos: torch.Tensor | None, sin: torch.Tensor | None, slots: torch.Tensor,
                           k_cache: torch.Tensor, v_cache: torch.Tensor, page_size: int,
                           block_tables: torch.Tensor, ctx: Any, scale: float, window: int, num_heads: int,
                           out: torch.Tensor) -> None:
    """:func:`qk_norm_rope_write` and :func:`paged_attention` of a step of decode tokens in one
    kernel: ``qkv`` ``[T, (Hq + 2 Hkv) * D]`` bf16 is the raw output of the qkv product; the new
    keys and values go to the cache at ``slots``; ``out`` ``[T, Hq * D]``. One query per request,
    no intermediate query tensor. Call only when :func:`can_fuse_decode` says so."""
    t = qkv.shape[0]
    hkv, d = k_cache.shape[1], k_cache.shape[3]
    dt = torch.bfloat16
    if qkv.dtype != dt or k_cache.dtype != dt or v_cache.dtype != dt or out.dtype != dt:
        raise KernelError("decode_attention_fused: bfloat16 only")
    if tuple(k_cache.shape[1:]) != (hkv, page_size, d) or k_cache.shape != v_cache.shape:
        raise KernelError("decode_attention_fused: cache layout must be [pages, kv_heads, page_size, head_dim]")
    if num_heads % hkv or qkv.shape != (t, (num_heads + 2 * hkv) * d) or out.numel() != t * num_heads * d:
        raise KernelError("decode_attention_fused: qkv/out shape or head grouping")
    if ctx.num_prefill or ctx.num_decode != t or block_tables.shape[0] != ctx.num_seqs or slots.shape != (t,):
        raise KernelError("decode_attention_fused: a step of decode tokens only, one token per request")
    if (cos is None) != (sin is None) or (cos is not None and tuple(cos.shape) != (t, d // 2)):
        raise KernelError("decode_attention_fused: rotary tables must be [tokens, head_dim / 2]")
    _check_indices("decode_attention_fused", block_tables, ctx, page_size, k_cache.shape[0], slots)
    ctas = t * hkv * (-(-(num_heads // hkv) // 16))
    splits = choose_splits(ctas, _decode_slots(d, True), ctx.max_context_len // 64, cluster=True)
    part_acc = part_ml = None
    if splits > 1:
        part_acc = ctx.arena.take((t, num_heads, splits, d), torch.float32)
        part_ml = ctx.arena.take((t, num_heads, splits, 2), torch.float32)
    _check(_fn("ts_decode_attention_tma_fused")(
        _dev(qkv, "qkv"), _opt(q_weight, "q_weight", dt), _opt(k_weight, "k_weight", dt), float(eps),
        _opt(cos, "cos", torch.float32), _opt(sin, "sin", torch.float32), _dev(slots, "slots", torch.int32),
        _dev(out, "out"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), k_cache.shape[0],
        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
        _dev(ctx.cu_query_lens, "cu_query_lens", torch.int32),
        _dev(ctx.context_lens_dev, "context_lens", torch.int32),
        _dev(ctx.decode_seqs, "decode_seqs", torch.int32), t, num_heads, hkv, d, page_size, float(scale),
        int(window), splits, _opt(part_acc, "part_acc"), _opt(part_ml, "part_ml"),
        _error_word(qkv.device).data_ptr(), _stream()), "decode_attention_tma_fused")


_slots_cache: dict[tuple[int, bool], int] = {}


def _decode_slots(head_dim: int, tma: bool) -> int:
    n = _slots_cache.get((head_dim, tma))
    if n is None:
        name = "ts_decode_attention_tma_slots" if tma else "ts_decode_attention_mma_slots"
        n = _slots_cache[(head_dim, tma)] = int(_fn(name)(head_dim))
    return n


# ------------------------------------------------------------------------- gemm
def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out[M, N] = x[M, K] @ w[N, K]^T`` with 32-bit accumulation. ``x`` and ``w`` share a
    dtype; ``out`` has it too, or is float32 (the logits). float32 inputs run on CUDA cores in
    true 32-bit; bfloat16 inputs use the tensor cores."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n) or x.dtype != w.dtype:
        raise KernelError(f"gemm: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)}")
    if out.dtype not in (x.dtype, torch.float32):
        raise KernelError(f"gemm: out dtype {out.dtype} for inputs {x.dtype}")
    if m == 0:
        return
    if x.dtype == torch.float32:
        _check(_fn("ts_gemm_simt")(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), m, n, k, _F32, _F32, _stream()),
               "gemm")
        return
    if m <= SKINNY_MAX_ROWS and k % 32 == 0 and n % 16 == 0 and (n * k <= SKINNY_MAX_WEIGHTS or out.dtype != x.dtype):
        gemm_skinny(x, w, out)
        return
    if m >= TCGEN05_MIN_ROWS and n >= TCGEN05_MIN_COLS and k % 8 == 0:
        tiles = tcgen05_tiles(m, n, 256)
        if tiles:
            gemm_tcgen05(x, w, out, TCGEN05_PAIR_TILE if tiles == "pairs" else 256)
            return
    _dev(x, "x"), _dev(w, "w"), _dev(out, "out")
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)                       # vendor library matrix product
    else:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)


# Up to this many rows a bf16 product streams the weights through the skinny kernel ...
SKINNY_MAX_ROWS = 16
# ... if the matrix is not larger than this (measured on B200: at the Qwen3-8B and 32B layer
# shapes the vendor library streams 15-35% faster; at the 0.6B shapes and for the output head
# the skinny kernel is level or ahead).
SKINNY_MAX_WEIGHTS = 1 << 24


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """bf16 ``out[M, N] = x[M, K] @ w[N, K]^T`` for M <= 64, K % 32 == 0, N % 16 == 0: weights
    streamed once from HBM into tensor-core fragments (``csrc/gemm_skinny.cu``)."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny: shape or dtype mismatch")
    _check(_fn("ts_gemm_skinny")(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), m, n, k, _code(out.dtype), _stream()),
           "gemm_skinny")


_error_words: dict[torch.device, torch.Tensor] = {}


def _error_word(device: torch.device) -> torch.Tensor:
    """A device int32 that kernels with bounded waits set when a wait ran out."""
    w = _error_words.get(device)
    if w is None:
        w = _error_words[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return w


# What a non-zero error word says (csrc/bounded_wait.cuh).
WAIT_FAILURES = {1: "gemm_tcgen05", 2: "prefill_attention_tcgen05", 3: "prefill_attention_tma",
                 4: "decode_attention_tma", 5: "decode_attention_mma"}


def raise_for_status(code: int, device: torch.device | str | None = None) -> None:
    """Raise ``KernelError`` for a non-zero error word read from the device (and clear the word, so
    that the next step starts clean)."""
    if code == 0:
        return
    for dev, w in _error_words.items():
        if device is None or torch.device(device) == dev:
            w.zero_()
    raise KernelError(f"kernel {WAIT_FAILURES.get(code, code)!r} gave up waiting on its pipeline (a bounded wait "
                      f"ran out): this step's results are not valid")


def check_device_errors() -> None:
    """Raise if a kernel gave up on a bounded wait since the last check (synchronises)."""
    for dev, w in _error_words.items():
        raise_for_status(int(w.item()), dev)


def set_wait_control(cycles: int | None = None, unarmed: bool = False) -> None:
    """How long the kernels' mbarrier waits may last, in clock cycles (``None``: the default, about a
    second), and the test switch ``unarmed`` that makes every kernel skip its copies so that its
    waits run out (``csrc/bounded_wait.cuh``). For the current device; call it with nothing in
    flight, and never with ``unarmed`` outside a test."""
    lib = build.library()
    lib.ts_set_wait_control.argtypes = [_c.c_longlong, _i]
    lib.ts_set_wait_control.restype = _i
    status = lib.ts_set_wait_control(int(cycles or 0), int(bool(unarmed)))
    if status != 0:
        raise KernelError(f"set_wait_control: CUDA error {status}")


# Default output-tile width of the tcgen05 product.
TCGEN05_TILE_N = 256
# 256-row tiles by pairs of CTAs (tcgen05 cta_group::2) where they fill the machine: a CTA then fetches a
# third less from L2 per flop. Measured on B200 (``python bench.py --profile gemm``), 2,048 rows, library /
# one CTA a tile / pairs: Qwen3-8B gate-up 267 / 291 / 275 us, Qwen3-32B gate-up 651 / 739 / 694 us;
# 8,192 rows of the Qwen3-8B o shape 221 / 228 / 194 us; level at the Qwen3-0.6B shapes.
TCGEN05_PAIR = True
TCGEN05_PAIR_TILE = 512      # the value of ``tile_n`` that asks for them
# The tcgen05 kernel takes the bf16 products with at least this many rows and output columns
# (measured on B200 at 2,048 rows: 17.9 / 26.6 / 564 us against the vendor library's 15.3 / 21.5 /
# 473 us for the qkv, gate-up and head shapes of Qwen3-0.6B; narrower outputs leave most SMs
# without a tile and stay with the library until the kernel learns to split K).
TCGEN05_MIN_ROWS = 128
TCGEN05_MIN_COLS = 2048
TCGEN05_MIN_FILL = 0.85
SM_COUNT = 148


def tcgen05_fills_the_machine(m: int, n: int, tile_cols: int) -> bool:
    """Whether the 128 x ``tile_cols`` output tiles of an ``m`` x ``n`` product keep the persistent
    CTAs of the tcgen05 kernel busy: the tiles fill at least 85 % of the rounds they take (one tile
    per SM and round). The kernel does not split K, so fewer tiles than SMs, or a nearly empty last
    round, leave SMs idle for a whole tile's time; those shapes go to the vendor library, which
    cuts them differently. Measured on B200, kernel by kernel (``python bench.py --profile gemm``):
    512 rows of the Qwen3-8B shapes (64 to 96 tiles) 27 / 76 / 30 us against the library's 17 / 42 /
    24 us for o / down / qkv; 2,048 x 5,120 outputs with K = 25,600 (320 tiles, 2.2 rounds) 604
    against 438 us; where the rounds are full the two are within a tenth of each other. (Cutting
    the last round's k blocks over all SMs, with the last CTA to arrive adding a tile's parts in
    the order of K, was written and passed its tests, but the reducing CTA's 128 epilogue threads
    read a tile's 128 to 384 KB of partial sums with 16 KB in flight, which cost 20 us a launch;
    the reduction has to go through bulk copies into the then idle operand buffers first.)"""
    tiles = -(-m // 128) * -(-n // tile_cols)
    rounds = -(-tiles // SM_COUNT)
    return tiles >= TCGEN05_MIN_FILL * rounds * SM_COUNT


def tcgen05_pairs_fill_the_machine(m: int, n: int, tile_cols: int) -> bool:
    """The same for tiles of 256 rows, each computed by a pair of CTAs (one tile per pair of SMs and round)."""
    tiles = -(-m // 256) * -(-n // tile_cols)
    rounds = -(-tiles // (SM_COUNT // 2))
    return tiles >= TCGEN05_MIN_FILL * rounds * (SM_COUNT // 2)


def tcgen05_tiles(m: int, n: int, tile_cols: int) -> str:
    """How the tcgen05 product cuts an ``m`` x ``n`` output: "pairs" (256-row tiles by pairs of CTAs),
    "single" (128-row tiles), or "" when neither fills the machine and the vendor library takes it."""
    if TCGEN05_PAIR and tcgen05_pairs_fill_the_machine(m, n, tile_cols):
        return "pairs"
    return "single" if tcgen05_fills_the_machine(m, n, tile_cols) else ""


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_n: int | None = None) -> None:
    """bf16 ``out[M, N] = x[M, K] @ w[N, K]^T`` with tcgen05.mma, TMA and TMEM
    (``csrc/gemm_tcgen05.cu``); K % 8 == 0, any M and N; out bf16 or float32."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tcgen05: shape or dtype mismatch")
    _check(_fn("ts_gemm_tcgen05")(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), m, n, k, _code(out.dtype),
                                  tile_n or TCGEN05_TILE_N, _error_word(x.device).data_ptr(), _stream()),
           "gemm_tcgen05")


def gemm_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, arena: Any) -> None:
    """``out[M, I] = silu(x Wgate^T) * (x Wup^T)`` with ``w_gate_up`` = gate rows then up rows,
    ``[2 I, K]``. For a few bf16 rows the product and the activation are one kernel (the gate
    and up rows of an output column are computed by the same CTA); otherwise a product into
    scratch from ``arena`` followed by the SiLU-multiply kernel; many bf16 rows of a wide matrix
    take the tcgen05 product with the activation in its epilogue."""
    m, k = x.shape
    inter = out.shape[1]
    if tuple(w_gate_up.shape) != (2 * inter, k) or out.shape[0] != m or out.dtype != x.dtype:
        raise KernelError("gemm_swiglu: shape or dtype mismatch")
    if (x.dtype == torch.bfloat16 and m <= SKINNY_MAX_ROWS and k % 32 == 0 and inter % 16 == 0
            and 2 * inter * k <= SKINNY_MAX_WEIGHTS):
        _check(_fn("ts_gemm_skinny_swiglu")(_dev(x, "x"), _dev(w_gate_up, "w_gate_up"), _dev(out, "out"), m, inter, k,
                                            _stream()), "gemm_swiglu")
        return
    tiles = tcgen05_tiles(m, inter, 128)
    if x.dtype == torch.bfloat16 and m >= TCGEN05_MIN_ROWS and 2 * inter >= TCGEN05_MIN_COLS and k % 8 == 0 and tiles:
        # many rows: the tcgen05 product with the activation in its epilogue
        _check(_fn("ts_gemm_tcgen05_swiglu")(_dev(x, "x"), _dev(w_gate_up, "w_gate_up"), _dev(out, "out"), m, inter, k,
                                             int(tiles == "pairs"), _error_word(x.device).data_ptr(), _stream()),
               "gemm_tcgen05_swiglu")
        return
    gate_up = arena.take((m, 2 * inter), x.dtype)
    gemm(x, w_gate_up, gate_up)
    silu_mul(gate_up, out)


# Steps of a few rows (decode) fold the RMSNorm into the products around it: the product that
# writes a sub-layer's output adds it to the residual stream itself and leaves a bf16 copy and the
# rows' sums of squares, and the next product normalises that copy while it loads it. It saves two
# of seven launches per layer. Measured on B200 (Qwen3-0.6B sizes, 1,024-token contexts, with the
# weights prefetched into L2): the decode step gains 6.7 % at batch 1, 6.3 % at 2, 1.3 % at 4,
# 0.9 % at 8. With the 16-row forms of the products in tiles of 16 weight rows it lost 2 % at 16 rows
# (they ran out of registers); with those in tiles of 8 weight rows it gains 1.3 % at 9 rows and is
# level at 12 and 16, hence up to 16 rows, the most the skinny kernels take. (Before the weights were
# prefetched the norm kernels hid behind the next product's weight stream and the fusion gained nothing.)
FUSE_STREAM_NORM = True
STREAM_FUSE_MAX_ROWS = 16


STREAM_FUSE_MAX_WIDTH = 2048      # 128 parts of 16 columns: what a warp of the consumer adds up


def can_stream_fuse(m: int, n: int, k: int, width: int, dtype: torch.dtype, device: torch.device) -> bool:
    """Whether a product of ``m`` rows with an ``[n, k]`` weight matrix can take part in the
    norm fusion (:func:`gemm_to_stream`, :func:`gemm_normed`) on a stream ``width`` wide: what
    the skinny kernel takes."""
    return (FUSE_STREAM_NORM and device.type == "cuda" and dtype == torch.bfloat16 and 0 < m <= STREAM_FUSE_MAX_ROWS
            and k % 32 == 0 and n % 16 == 0 and n * k <= SKINNY_MAX_WEIGHTS
            and width <= STREAM_FUSE_MAX_WIDTH)


def gemm_to_stream(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, resid16: torch.Tensor,
                   sumsq: torch.Tensor) -> torch.Tensor:
    """``resid[M, N] += bf16(x[M, K] @ w[N, K]^T)`` in place (float32 stream); ``resid16`` gets
    the new stream in bf16 and ``sumsq`` (at least ``2 N`` floats of scratch) the rows' sums of squares in
    parts: returned as a view ``[M, parts]`` with ``parts`` = ``N / 16`` or, where the kernel cuts the
    output into tiles of 8 columns, ``N / 8``; both for the product that normalises the stream next
    (:func:`gemm_normed`). bf16, ``M <= 16``."""
    m, k = x.shape
    n = w.shape[0]
    if (w.shape[1] != k or tuple(resid.shape) != (m, n) or resid.dtype != torch.float32 or sumsq.dtype != torch.float32
            or sumsq.numel() < 2 * n or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16
            or tuple(resid16.shape) != (m, n) or resid16.dtype != torch.bfloat16):
        raise KernelError("gemm_to_stream: shape or dtype mismatch")
    _check(_fn("ts_gemm_skinny_to_stream")(_dev(x, "x"), _dev(w, "w"), _dev(resid, "resid"), _dev(resid16, "resid16"),
                                           _dev(sumsq, "sumsq"), m, n, k, _stream()), "gemm_to_stream")
    parts = int(_fn("ts_gemm_skinny_to_stream_parts")(m, n, k))
    return sumsq[: m * parts].view(m, parts)


def gemm_normed(resid16: torch.Tensor, sumsq: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor,
                out: torch.Tensor, swiglu: bool = False) -> None:
    """``out = rms_norm(resid) @ w^T`` (or its SwiGLU form, ``w`` = gate rows then up rows) where
    the norm is applied inside the product: ``resid16`` ``[M, K]`` bf16 and ``sumsq`` ``[M, parts]`` as
    :func:`gemm_to_stream` returned it (at most 128 parts per row), ``norm_weight`` ``[K]`` bf16."""
    m, k = resid16.shape
    n = out.shape[1]
    if (tuple(w.shape) != ((2 * n if swiglu else n), k) or out.shape[0] != m or resid16.dtype != torch.bfloat16
            or sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.shape[0] != m or not sumsq.is_contiguous()
            or norm_weight.shape != (k,) or w.dtype != torch.bfloat16 or norm_weight.dtype != torch.bfloat16):
        raise KernelError("gemm_normed: shape or dtype mismatch")
    _check(_fn("ts_gemm_skinny_normed")(_dev(resid16, "resid16"), _dev(sumsq, "sumsq"), int(sumsq.shape[1]),
                                        _dev(norm_weight, "norm_weight"), float(eps), _dev(w, "w"), _dev(out, "out"), m, n,
                                        k, _code(out.dtype), int(bool(swiglu)), _stream()), "gemm_normed")


# -------------------------------------------------------------------- L2 prefetch
# Decode steps of a few requests fetch the weights of the products that follow the attention
# kernel into L2 while that kernel runs (it leaves memory bandwidth idle), from a kernel of their
# own on a side stream (other placements were measured and are worse: csrc/prefetch.cu). Measured on B200 at the
# Qwen3-0.6B sizes with 1,024-token contexts: with their weights in L2 the products take 2.6-3.8 us
# instead of 3.4-5.4 us each; the decode step gains 1.5 % at batch 1 and 4.7 % at batch 8, nothing
# at 16, and loses 3 % from batch 32 on, where attention needs the bandwidth itself. Fetching the
# next layer's first weights as well changed nothing.
PREFETCH_WEIGHTS = True
PREFETCH_MAX_ROWS = 16
PREFETCH_MAX_BYTES = 48 << 20          # per call: well under L2's size
_side_streams: dict[int, "torch.cuda.Stream"] = {}


# The attention kernel of a decode step lasts about this long: a fixed part and its cache at the rate
# it reaches beside the prefetch. A recorded step is recorded for the longest context it may carry,
# so the typical context is assumed for anything longer.
PREFETCH_ATTENTION_FIXED_US = 3.0
PREFETCH_ATTENTION_GBS = 4000.0
PREFETCH_TYPICAL_CONTEXT = 1024
PREFETCH_THREADS = 0             # non-zero: requests per CTA, whatever the step (measurements)
PREFETCH_SM_GBS = 150.0          # what one SM passes on of such requests (measured on B200)
PREFETCH_PIECE = 16 * 1024


def prefetch_threads(total_bytes: int, beside_us: float) -> int:
    """Requests per CTA of the prefetch kernel so that it lasts about ``beside_us`` microseconds (the
    kernel lasts until its requests are served, and it is joined again after the kernel it runs
    beside, so it should end with that one: slower and the step waits for it, faster and it takes
    bandwidth the other kernel could use)."""
    if PREFETCH_THREADS:
        return PREFETCH_THREADS
    ctas = max(1.0, total_bytes / (PREFETCH_SM_GBS * 1e3 * max(beside_us, 1.0)))
    pieces = max(1, total_bytes // PREFETCH_PIECE)
    per_cta = pieces / ctas
    return int(min(128, max(16, 16 * round(per_cta / 16))))


def prefetch_l2(tensors: Sequence[torch.Tensor], threads: int = 128) -> None:
    """Ask for the memory of ``tensors`` (contiguous, on the device; at most 8) to be brought
    into L2. Returns at once; nothing waits for the data. ``threads``: requests of 16 KB per CTA
    (16 to 128 in steps of 16; fewer means more CTAs and a higher rate, see ``prefetch_threads``)."""
    tensors = [t for t in tensors if t is not None and t.numel()]
    if not tensors:
        return
    if len(tensors) > 8:
        raise KernelError("prefetch_l2: at most 8 tensors per call")
    bases = (_c.c_void_p * len(tensors))(*[_dev(t, "tensor") for t in tensors])
    sizes = (_c.c_ulonglong * len(tensors))(*[t.numel() * t.element_size() for t in tensors])
    _check(_fn("ts_prefetch_l2")(bases, sizes, len(tensors), int(threads), _stream()), "prefetch_l2")


def prefetch_l2_beside(tensors: Sequence[torch.Tensor], threads: int = 128) -> "Callable[[], None]":
    """:func:`prefetch_l2` on a stream of its own that starts where the current stream stands,
    so that it runs beside the kernels launched next. Returns the function that makes the
    current stream wait for it again (call it after those kernels; a recording of the step
    needs every side branch joined)."""
    cur = torch.cuda.current_stream()
    side = _side_streams.get(cur.device.index)
    if side is None:
        side = _side_streams[cur.device.index] = torch.cuda.Stream(device=cur.device)
    side.wait_stream(cur)
    with torch.cuda.stream(side), stream_scope():
        prefetch_l2(tensors, threads)
    return lambda: cur.wait_stream(side)


# While the products after the attention kernel read their weights from L2, memory idles: the pages
# that the step's requests hold in the NEXT layer's cache are asked for meanwhile, on a second side
# stream that nothing waits for until the end of the step. Measured on B200 in the recorded decode
# step (Qwen3-0.6B sizes, 1,024-token contexts): batch 1 / 4 / 8 / 16: 0.792 -> 0.775, 0.804 ->
# 0.793, 0.892 -> 0.876, 1.555 -> 1.540 ms. The gain is small because the attention kernel is bound
# by its own chain of latencies more than by where its keys come from (batch 8, kernel alone: 9.7 us
# with the cache in HBM, 8.7 us with it in L2), and it needs the slow rate of 128 requests per CTA:
# at 16 to 32 per CTA the requests disturb the products and the step loses 4 to 7 %.
PREFETCH_NEXT_CACHE = True
PREFETCH_NEXT_CACHE_THREADS = 128
_cache_streams: dict[int, "torch.cuda.Stream"] = {}


def prefetch_pages_later(k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor, ctx: Any,
                         page_size: int) -> "Callable[[], None]":
    """Ask for the cache pages that the step's requests hold in ``k_cache`` / ``v_cache`` to be
    brought into L2, on a stream of its own that starts where the current stream stands and that
    nothing of the step waits for; returns the function that joins it (call it once, at the end of
    the step: a recording needs every side branch joined)."""
    cur = torch.cuda.current_stream()
    side = _cache_streams.get(cur.device.index)
    if side is None:
        side = _cache_streams[cur.device.index] = torch.cuda.Stream(device=cur.device)
    side.wait_stream(cur)
    page_bytes = k_cache[0].numel() * k_cache.element_size()
    with torch.cuda.stream(side), stream_scope():
        _check(_fn("ts_prefetch_pages")(_dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), page_bytes,
                                        _dev(block_tables, "block_tables", torch.int32), block_tables.shape[1],
                                        _dev(ctx.context_lens_dev, "context_lens", torch.int32), ctx.num_seqs,
                                        page_size, PREFETCH_NEXT_CACHE_THREADS, _stream()), "prefetch_pages")
    return lambda: cur.wait_stream(side)


PDL_ELEMENTWISE, PDL_SKINNY, PDL_ATTENTION, PDL_TCGEN05, PDL_SAMPLING, PDL_OTHER = 1, 2, 4, 8, 16, 32


def set_decode_cluster_merge(on: bool) -> None:
    """Whether decode attention merges 2 to 8 key ranges of a request inside a thread-block cluster
    (the default) or through global memory, as it does for more ranges. Same bits either way."""
    lib = build.library()
    lib.ts_set_decode_cluster_merge.argtypes = [_i]
    lib.ts_set_decode_cluster_merge.restype = None
    lib.ts_set_decode_cluster_merge(1 if on else 0)
    global CLUSTER_MERGE
    CLUSTER_MERGE = bool(on)


_TIMELINE_CLASSES = {1: "elementwise", 2: "skinny", 4: "attention", 8: "tcgen05", 16: "sampling", 32: "other"}


def timeline(capacity: int = 1 << 16) -> list[dict[str, Any]]:
    """The kernels launched since the last call, in the order they started on the device: for each
    its class, grid and block size, ``start`` (ns on the device clock when its first CTA began) and
    ``waited`` (ns when that CTA's wait for the kernels before it returned; 0 if its first thread
    never waits). Synchronises the device. Empty unless the library was built with
    ``TINYSERVE_B200_TIMELINE=1`` in the environment (a second, slower build kept apart)."""
    lib = build.library()
    lib.ts_timeline_read.argtypes = [ctypes.c_void_p, _i]
    lib.ts_timeline_read.restype = _i
    buf = (ctypes.c_uint64 * (3 * capacity))()
    n = lib.ts_timeline_read(buf, capacity)
    if n < 0:
        raise KernelError("timeline: CUDA error while reading the records")
    out = []
    for i in range(n):
        tag, start, waited = buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]
        out.append({"class": _TIMELINE_CLASSES.get(tag & 0xFF, str(tag & 0xFF)), "grid": ((tag >> 8) & 0xFFFFF, (tag >> 28) & 0xFFFF),
                    "block": tag >> 44, "start": int(start), "waited": int(waited)})
    out.sort(key=lambda r: r["start"])
    return out


def set_programmatic_launch(on: bool | int) -> None:
    """Launch this library's kernels so that each may start while its predecessor on the stream
    is draining (programmatic dependent launch); every kernel waits for its predecessor before
    it touches data. ``True`` / ``False`` turn it on / off for all kernels; an int is a mask of
    the ``PDL_*`` kernel classes. Off by default."""
    lib = build.library()
    lib.ts_set_programmatic_launch.argtypes = [_i]
    lib.ts_set_programmatic_launch.restype = None
    global _pdl_mask
    mask = (-1 if on else 0) if isinstance(on, bool) else int(on)
    lib.ts_set_programmatic_launch(mask)
    _pdl_mask = mask


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """The CUDA-core product for any dtype pairing ``gemm`` allows (slow; any size)."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n) or x.dtype != w.dtype:
        raise KernelError("gemm_simt: shape or dtype mismatch")
    _check(_fn("ts_gemm_simt")(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), m, n, k, _code(x.dtype),
                               _code(out.dtype), _stream()), "gemm_simt")


# --------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor | None = None,
           top_p: torch.Tensor | None = None, seeds: torch.Tensor | None = None,
           draws: torch.Tensor | None = None, status_out: torch.Tensor | None = None) -> None:
    """One token per row of ``logits`` ``[R, V]`` float32 into ``out`` ``[R]`` int32. With no
    ``temperature`` every row is greedy; else rows with temperature 0 are greedy and the others
    are drawn (``seeds``/``draws`` int64 ``[R]``: the request's seed and how many tokens it
    has drawn so far; ``top_p`` float32 ``[R]`` optional). ``status_out`` (int32, one element):
    receives the device's error word, which kernels with bounded waits set when a wait ran out,
    so that it reaches the host in the same copy as the tokens."""
    r, v = logits.shape
    if out.shape != (r,):
        raise KernelError("sample: one output per row")
    _check(_fn("ts_sample")(_dev(logits, "logits", torch.float32), r, v, _opt(temperature, "temperature", torch.float32),
                            _opt(top_p, "top_p", torch.float32), _opt(seeds, "seeds", torch.int64),
                            _opt(draws, "draws", torch.int64), _dev(out, "out", torch.int32),
                            None if status_out is None else _error_word(logits.device).data_ptr(),
                            _opt(status_out, "status_out", torch.int32), _stream()), "sample")
