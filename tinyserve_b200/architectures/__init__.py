"""Architectures this framework serves. Importing the package registers them."""

from . import qwen3  # noqa: F401  (registers Qwen3ForCausalLM)
from .qwen3 import Qwen3Config

__all__ = ["Qwen3Config"]
