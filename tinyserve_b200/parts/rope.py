"""Rotary position encoding: the per-step cos/sin tables.

Formula (upstream src/tinyserve/layers.py:61-65): ``inv_freq[i] = theta ** (-2i / rotary_dim)``
in float64, ``angle = position * inv_freq`` in float64, cos and sin taken in float64 and
rounded to float32. The rotation itself (pairs ``i`` and ``i + rotary_dim/2`` for the "half"
pairing, neighbours ``2i, 2i+1`` for "interleaved"; src/tinyserve/layers.py:84-91 has the
former) is applied by the mixer's fused kernel, which receives these tables.
"""

from __future__ import annotations

from typing import Any

import torch

from ..kernels import ops
from .base import EVERY_STEP, PositionEncoding, Rotation, StepContext, register_position_encoding

RotaryTables = Rotation      # the step's position data of a rotary encoding is the rotation itself


class RotaryEncoding(PositionEncoding):
    recordable = EVERY_STEP

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, pairing: str = "half") -> None:
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim={rotary_dim} must be even and at most head_dim={head_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing must be 'half' or 'interleaved', got {pairing!r}")
        self.head_dim, self.rotary_dim = int(head_dim), int(rotary_dim)
        self.theta, self.pairing = float(theta), pairing
        two_i = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64)
        self._inv_freq_host = self.theta ** (-two_i / self.rotary_dim)
        self._inv_freq: torch.Tensor | None = None

    def key(self) -> Any:
        return ("rope", self.rotary_dim, self.theta, self.pairing)

    def prepare(self, ctx: StepContext) -> RotaryTables:
        dev = ctx.positions.device
        if self._inv_freq is None or self._inv_freq.device != dev:
            self._inv_freq = self._inv_freq_host.to(dev)
        half = self.rotary_dim // 2
        cos = ctx.arena.take_step((ctx.num_tokens, half), torch.float32)
        sin = ctx.arena.take_step((ctx.num_tokens, half), torch.float32)
        ops.rope_tables(ctx.positions, self._inv_freq, cos, sin)
        return RotaryTables(cos, sin, self.rotary_dim, self.pairing == "interleaved")


register_position_encoding("rope", RotaryEncoding)
