"""Grouped-query attention over the paged cache, with optional per-head q/k RMSNorm,
rotary position encoding and an optional sliding window.

Per token (upstream src/tinyserve/model.py:154-173, src/tinyserve/attention.py:89-111):
``qkv = x Wqkv^T`` (rows q, then k, then v; no bias); q and k are normalised per head over
``head_dim`` before the rotation; k (rotated) and v go to the cache at the token's slot;
query head ``h`` reads kv head ``h // (num_heads / num_kv_heads)``; scores are scaled by
``scale``, masked causally (and to the last ``window`` positions if a window is set),
soft-maxed in 32-bit and applied to v; the heads are concatenated and projected by ``Wo``.
The residual add happens in the next norm.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..kernels import ops
from .base import (EVERY_STEP, KVCacheEntry, KVNeed, LazyNormed, Mixer, ResidualStream, StepContext, TensorSpec, project,
                   project_to_stream, register_mixer)


class GQAAttention(Mixer):
    recordable = EVERY_STEP

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float, qk_norm: bool = False, qk_norm_eps: float = 1e-6,
                 window: int | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive or None, got {window}")
        if head_dim <= 0 or head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim={head_dim}: the attention kernels take head sizes in steps of 16 up to 256")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.scale = int(head_dim), float(scale)
        self.qk_norm, self.qk_norm_eps = bool(qk_norm), float(qk_norm_eps)
        self.window = None if window is None else int(window)
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.w_qkv = self.w_q = self.w_o = self.q_norm_w = self.k_norm_w = None

    def cache_need(self) -> KVNeed:
        return KVNeed(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self, prefix: str) -> list[TensorSpec]:
        p, h = prefix + self.prefix, self.hidden_size
        specs = [
            TensorSpec(p + "qkv_proj.weight", (self.q_size + 2 * self.kv_size, h),
                       merged_from=(p + "q_proj.weight", p + "k_proj.weight", p + "v_proj.weight"),
                       merged_rows=(self.q_size, self.kv_size, self.kv_size)),
            TensorSpec(p + "o_proj.weight", (h, self.q_size)),
        ]
        if self.qk_norm:
            specs += [TensorSpec(p + "q_norm.weight", (self.head_dim,), init="one_plus_normal"),
                      TensorSpec(p + "k_norm.weight", (self.head_dim,), init="one_plus_normal")]
        return specs

    def bind(self, prefix: str, tensors: Mapping[str, torch.Tensor]) -> None:
        p = prefix + self.prefix
        self.w_qkv = tensors[p + "qkv_proj.weight"]
        self.w_q = self.w_qkv[: self.q_size]          # a view: rows of q only
        self.w_o = tensors[p + "o_proj.weight"]
        if self.qk_norm:
            self.q_norm_w = tensors[p + "q_norm.weight"]
            self.k_norm_w = tensors[p + "k_norm.weight"]

    takes_lazy_input = True
    adds_to_stream = True

    def forward(self, x: "torch.Tensor | LazyNormed", ctx: StepContext, cache: KVCacheEntry, writes_cache: bool,
                position: Any, stream: ResidualStream | None = None) -> torch.Tensor | None:
        t = x.shape[0]
        x_device = cache.k.device
        arena = ctx.arena
        group = ctx.kv[cache.group]
        width = self.q_size + 2 * self.kv_size if writes_cache else self.q_size
        qkv = arena.take((t, width), ctx.dtype)
        project(x, self.w_qkv if writes_cache else self.w_q, qkv, ctx)
        # what the layer's position encoding asks to be done to q and k: a rotation, or nothing
        rot = None if position is None else position.qk_rotation()
        cos = None if rot is None else rot.cos
        sin = None if rot is None else rot.sin
        rotary_dim = 0 if rot is None else rot.rotary_dim
        interleaved = False if rot is None else rot.interleaved
        attn = arena.take((t, self.q_size), ctx.dtype)
        join = None
        if ops.PREFETCH_WEIGHTS and ctx.num_prefill == 0 and ctx.num_decode <= ops.PREFETCH_MAX_ROWS and x_device.type == "cuda":
            # decode: attention streams the cache and leaves bandwidth idle; the weights of the
            # products after it (output projection, feed-forward) come into L2 meanwhile
            ahead = [w for w in [self.w_o, *ctx.upcoming_weights] if w is not None][:8]
            nbytes = sum(w.numel() * w.element_size() for w in ahead)
            if ahead and nbytes <= ops.PREFETCH_MAX_BYTES:
                # at the rate that makes it last as long as the attention kernel is expected to: that
                # kernel's fixed part and the cache it streams
                cache_bytes = 2.0 * ctx.num_decode * min(ctx.max_context_len, ops.PREFETCH_TYPICAL_CONTEXT) \
                    * self.kv_size * self.w_o.element_size()
                beside_us = ops.PREFETCH_ATTENTION_FIXED_US + cache_bytes / (ops.PREFETCH_ATTENTION_GBS * 1e3)
                join = ops.prefetch_l2_beside(ahead, ops.prefetch_threads(nbytes, beside_us))
        if writes_cache and ops.can_fuse_decode(ctx, ctx.dtype, self.num_heads, self.num_kv_heads, self.head_dim,
                                                cache.page_size, cache.k.shape[0], rotary_dim, interleaved,
                                                cache.k.device):
            # decode tokens only: norm, rotation, cache write and attention in one kernel
            ops.decode_attention_fused(qkv, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, cos, sin, group.slots,
                                       cache.k, cache.v, cache.page_size, group.block_tables, ctx, self.scale,
                                       self.window or 0, self.num_heads, attn)
        else:
            q = arena.take((t, self.num_heads, self.head_dim), ctx.dtype)
            ops.qk_norm_rope_write(qkv, q, self.q_norm_w, self.k_norm_w, self.qk_norm_eps, cos, sin, rotary_dim,
                                   interleaved, group.slots, cache.k, cache.v, cache.page_size,
                                   self.num_heads, self.num_kv_heads, self.head_dim, writes_cache)
            ops.paged_attention(q, cache.k, cache.v, cache.page_size, group.block_tables, ctx,
                                self.scale, self.window or 0, attn)
        if join is not None:
            join()
        nxt = ctx.upcoming_caches.get("mixer")
        if (ops.PREFETCH_NEXT_CACHE and join is not None and isinstance(nxt, KVCacheEntry) and nxt.k is not cache.k
                and nxt.group in ctx.kv):
            # the products that follow read their weights from L2 and leave the memory idle: the next
            # layer's pages of these requests come into L2 meanwhile (nothing waits for them)
            later = ops.prefetch_pages_later(nxt.k, nxt.v, ctx.kv[nxt.group].block_tables, ctx, nxt.page_size)
            if not ctx.at_step_end:
                ctx.at_step_end.append(later)
        return project_to_stream(attn, self.w_o, stream, ctx)


register_mixer("gqa_attention", GQAAttention)
