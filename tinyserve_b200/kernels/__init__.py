"""Python entry to the hand-written CUDA kernels (``ops``) and their build (``build``)."""

from . import build, ops

__all__ = ["build", "ops"]
