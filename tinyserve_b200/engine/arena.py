"""Scratch memory of a step: a bump allocator over buffers that are reused every step.

Three regions: ``step`` holds what lives for the whole step (the residual stream, position
tables, logits); two ``frames`` alternate from layer to layer, so that the output a layer
leaves pending on the residual stream is still intact while the next layer, working in the
other frame, reads it. Nothing is allocated from the device allocator in steady state; a
region grows (once, outside any graph capture) when a step needs more than it has.
"""

from __future__ import annotations

import torch

_ALIGN = 256
_ELEMENT_SIZE: dict[torch.dtype, int] = {}


def _element_size(dtype: torch.dtype) -> int:
    n = _ELEMENT_SIZE.get(dtype)
    if n is None:
        n = _ELEMENT_SIZE[dtype] = torch.empty(0, dtype=dtype).element_size()
    return n


class _Region:
    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.buf = torch.empty(0, dtype=torch.uint8, device=device)
        self._typed: dict[torch.dtype, torch.Tensor] = {}     # ``buf`` seen as each dtype asked for so far
        self.used = 0          # offset in ``buf`` of the next take
        self.demand = 0        # bytes taken since the last reset, wherever they came from
        self.high_water = 0    # the largest demand of any step so far

    def reset(self) -> None:
        if self.high_water > self.buf.numel():
            # The last step outgrew the buffer and was served piecemeal; make one buffer that
            # holds a whole step, so that from now on nothing moves.
            self.buf = torch.empty(self.high_water // _ALIGN * _ALIGN + _ALIGN, dtype=torch.uint8, device=self.device)
            self._typed = {}
        self.used = 0
        self.demand = 0

    def take(self, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= int(s)
        size = _element_size(dtype)
        nbytes = numel * size
        self.demand = (self.demand + _ALIGN - 1) // _ALIGN * _ALIGN + nbytes
        self.high_water = max(self.high_water, self.demand)
        start = (self.used + _ALIGN - 1) // _ALIGN * _ALIGN
        end = start + nbytes
        if end > self.buf.numel():
            # Grow: views handed out earlier keep the old buffer alive until they die.
            grow = max(nbytes, 2 * self.buf.numel(), 1 << 16)
            self.buf = torch.empty((grow + _ALIGN - 1) // _ALIGN * _ALIGN, dtype=torch.uint8, device=self.device)
            self._typed = {}
            start, end = 0, nbytes
        self.used = end
        if numel == 0:
            return torch.empty(shape, dtype=dtype, device=self.device)
        typed = self._typed.get(dtype)
        if typed is None:
            typed = self._typed[dtype] = self.buf.view(dtype)     # buffer sizes are multiples of 256 bytes
        return typed[start // size: end // size].view(shape)


class Arena:
    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        self._step = _Region(self.device)
        self._frames = (_Region(self.device), _Region(self.device))
        self._current = self._step
        self._frame_index = 0

    def begin_step(self) -> None:
        self._step.reset()
        for f in self._frames:
            f.reset()
        self._current = self._step
        self._frame_index = 0

    def next_frame(self) -> None:
        self._frame_index ^= 1
        self._current = self._frames[self._frame_index]
        self._current.reset()

    def step_region(self) -> None:
        """Later takes live until the end of the step (used after the last layer)."""
        self._current = self._step

    def take(self, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self._current.take(tuple(shape), dtype)

    def take_step(self, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        return self._step.take(tuple(shape), dtype)

    @property
    def reserved_bytes(self) -> int:
        return self._step.buf.numel() + sum(f.buf.numel() for f in self._frames)
