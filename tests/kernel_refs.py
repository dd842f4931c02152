"""Plain PyTorch references of the kernels in ``tinyserve_b200.kernels.ops``, one per kernel,
with the same signatures. They run on any device. The GPU tests compare every kernel with its
reference; the host-only tests put them in the kernels' place (``use_references``) to check
the step function, the cache and the scheduler without a GPU.

Formulas: upstream src/tinyserve/layers.py (norm, rotation), src/tinyserve/attention.py
(paged attention), src/tinyserve/sampling.py (sampling).
"""

from __future__ import annotations

import math
from contextlib import contextmanager
from typing import Any

import numpy as np
import torch


def _round(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return x.to(dtype).float()


def embed(tokens, table, out) -> None:
    out.copy_(table[tokens.long()].float())


def add_rms_norm(resid, delta, weight, eps, out, rows=None) -> None:
    x = resid if rows is None else resid[rows.long()]
    if delta is not None:
        x = x + (delta if rows is None else delta[rows.long()]).float()
        if rows is None:
            resid.copy_(x)
    n = _round(x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps), out.dtype)
    out.copy_((n * weight.float()).to(out.dtype))


def rope_tables(positions, inv_freq, cos, sin) -> None:
    a = positions.double()[:, None] * inv_freq[None, :]
    cos.copy_(a.cos().float())
    sin.copy_(a.sin().float())


def silu_mul(gate_up, out) -> None:
    inter = out.shape[1]
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    out.copy_((_round(g / (1 + torch.exp(-g)), out.dtype) * u).to(out.dtype))


def _head_norm(x: torch.Tensor, w: torch.Tensor | None, eps: float, dtype: torch.dtype) -> torch.Tensor:
    xf = x.float()
    if w is None:
        return xf
    n = _round(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps), dtype)
    return _round(n * w.float(), dtype)


def _rotate(x: torch.Tensor, cos, sin, rotary_dim: int, interleaved: bool) -> torch.Tensor:
    if not rotary_dim:
        return x
    rot, rest = x[..., :rotary_dim], x[..., rotary_dim:]
    c, s = cos[:, None, :], sin[:, None, :]
    if interleaved:
        a, b = rot[..., 0::2], rot[..., 1::2]
        o = torch.stack([a * c - b * s, b * c + a * s], dim=-1).flatten(-2)
    else:
        half = rotary_dim // 2
        a, b = rot[..., :half], rot[..., half:]
        o = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
    return torch.cat([o, rest], dim=-1)


def qk_norm_rope_write(qkv, q_out, q_weight, k_weight, eps, cos, sin, rotary_dim, interleaved, slots,
                       k_cache, v_cache, page_size, num_heads, num_kv_heads, head_dim, write_kv) -> None:
    t = q_out.shape[0]
    dt = q_out.dtype
    qs = num_heads * head_dim
    q = qkv[:, :qs].view(t, num_heads, head_dim)
    q = _rotate(_head_norm(q, q_weight, eps, dt), cos, sin, rotary_dim, interleaved)
    q_out.copy_(q.to(dt))
    if not write_kv:
        return
    ks = num_kv_heads * head_dim
    k = qkv[:, qs: qs + ks].view(t, num_kv_heads, head_dim)
    v = qkv[:, qs + ks:].view(t, num_kv_heads, head_dim)
    k = _rotate(_head_norm(k, k_weight, eps, dt), cos, sin, rotary_dim, interleaved).to(dt)
    page, off = slots.long() // page_size, slots.long() % page_size
    k_cache[page, :, off] = k
    v_cache[page, :, off] = v


def paged_attention(q, k_cache, v_cache, page_size, block_tables, ctx: Any, scale, window, out) -> None:
    """Per request: gather its keys and values from the pages in position order, then plain
    causal (windowed) attention for its new tokens (upstream src/tinyserve/attention.py:62-111)."""
    t, hq, d = q.shape
    hkv = k_cache.shape[1]
    group = hq // hkv
    res = torch.zeros(t, hq, d, dtype=torch.float32, device=q.device)
    cu = ctx.cu_query_lens.tolist()
    lens = ctx.context_lens_dev.tolist()
    for b in range(ctx.num_seqs):
        r0, n, total = cu[b], cu[b + 1] - cu[b], lens[b]
        pos = torch.arange(total, device=q.device)
        lo = 0
        if window:
            lo = max(0, (total - n) - window + 1)      # pages before this may be gone
        pos = pos[lo:]
        pages = block_tables[b].long()[pos // page_size]
        k = k_cache[pages, :, pos % page_size].float().repeat_interleave(group, dim=1)   # [keys, Hq, D]
        v = v_cache[pages, :, pos % page_size].float().repeat_interleave(group, dim=1)
        qpos = torch.arange(total - n, total, device=q.device)
        hidden = pos[None, :] > qpos[:, None]
        if window:
            hidden = hidden | (pos[None, :] <= qpos[:, None] - window)
        s = torch.einsum("ihd,jhd->hij", q[r0: r0 + n].float(), k) * scale
        s = s.masked_fill(hidden, float("-inf"))
        res[r0: r0 + n] = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v)
    out.copy_(res.view(t, hq * d).to(out.dtype))


def gemm(x, w, out) -> None:
    out.copy_((x.float() @ w.float().t()).to(out.dtype))


gemm_simt = gemm


def gemm_swiglu(x, w_gate_up, out, arena=None) -> None:
    inter = out.shape[1]
    gu = torch.empty(x.shape[0], 2 * inter, dtype=x.dtype, device=x.device)
    gemm(x, w_gate_up, gu)
    silu_mul(gu, out)


# ---------------------------------------------------------------------- sampling
def _philox4x32_10(c: np.ndarray, k0: int, k1: int) -> np.ndarray:
    """c: [N, 4] uint32 counters -> [N, 4] uint32 (Philox4x32 with 10 rounds)."""
    c = c.astype(np.uint64)
    k0, k1 = np.uint64(k0), np.uint64(k1)
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    mask = np.uint64(0xFFFFFFFF)
    c0, c1, c2, c3 = c[:, 0], c[:, 1], c[:, 2], c[:, 3]
    for _ in range(10):
        p0, p1 = m0 * c0, m1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def exponential_noise(vocab: int, seed: int, draw: int) -> torch.Tensor:
    """E_i = -log(u_i): u_i from Philox keyed by the seed, counter (i // 4, draw), word i % 4,
    mapped to the 24-bit grid ((x >> 8) + 0.5) / 2^24."""
    n4 = (vocab + 3) // 4
    c = np.zeros((n4, 4), dtype=np.uint32)
    c[:, 0] = np.arange(n4, dtype=np.uint32)
    c[:, 1] = draw & 0xFFFFFFFF
    c[:, 2] = (draw >> 32) & 0xFFFFFFFF
    bits = _philox4x32_10(c, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF).reshape(-1)[:vocab]
    u = ((bits >> 8).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return -torch.log(torch.from_numpy(u))


def sample(logits, out, temperature=None, top_p=None, seeds=None, draws=None, status_out=None) -> None:
    """Greedy rows: first argmax. Others (upstream src/tinyserve/sampling.py:56-102, with
    this framework's noise): p = softmax(logits / T); with top_p < 1 keep tokens whose strictly
    more likely tokens hold less than top_p; pick argmax of log p - log E."""
    r, v = logits.shape
    res = []
    for b in range(r):
        row = logits[b].float().cpu()
        temp = 0.0 if temperature is None else float(temperature[b])
        if not temp > 0:
            res.append(int(row.argmax()))
            continue
        z = row * (np.float32(1.0) / np.float32(temp))
        e = torch.exp(z - z.max())
        keep = torch.ones(v, dtype=torch.bool)
        tp = 1.0 if top_p is None else float(top_p[b])
        if tp < 1:
            total = e.sum()
            order = torch.argsort(e, descending=True, stable=True)
            es = e[order]
            above = torch.cumsum(es, 0) - es
            # tokens of equal probability share the mass above the first of them
            first = torch.searchsorted(-es, -es, right=False)
            above = above[first]
            keep_sorted = above < tp * total
            keep = torch.zeros(v, dtype=torch.bool)
            keep[order] = keep_sorted
        noise = exponential_noise(v, int(seeds[b]), int(draws[b]))
        score = torch.where(keep, z - torch.log(noise), torch.full_like(z, -math.inf))
        res.append(int(score.argmax()))
    out.copy_(torch.tensor(res, dtype=torch.int32, device=out.device))
    if status_out is not None:
        status_out.zero_()


_NAMES = ["embed", "add_rms_norm", "rope_tables", "silu_mul", "qk_norm_rope_write", "paged_attention",
          "gemm", "gemm_simt", "gemm_swiglu", "sample"]


@contextmanager
def use_references():
    """Put the references in the kernels' place (host-only tests of the engine's logic)."""
    from tinyserve_b200.kernels import ops

    saved = {n: getattr(ops, n) for n in _NAMES}
    try:
        for n in _NAMES:
            setattr(ops, n, globals()[n])
        yield
    finally:
        for n, f in saved.items():
            setattr(ops, n, f)
