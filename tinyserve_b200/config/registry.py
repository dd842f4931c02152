"""One registry from an architecture's name (``config.json["architectures"][0]``) to its
typed configuration class. The model itself is always the generic decoder built from the
``ModelSpec`` that the configuration produces, so registering a name and a config class is
all that a new architecture needs.

Reference: upstream has no registry, only a membership test for "Qwen3ForCausalLM"
(src/tinyserve/config.py:42).
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

from .base import ModelConfig, UnsupportedConfigError, read_config_json

_ARCHITECTURES: dict[str, type[ModelConfig]] = {}


def register_architecture(name: str, config_cls: type[ModelConfig], *, replace: bool = False) -> None:
    if not replace and name in _ARCHITECTURES and _ARCHITECTURES[name] is not config_cls:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = config_cls


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def config_class_for(name: str) -> type[ModelConfig]:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnsupportedConfigError(
            f"unknown architecture {name!r}; known: {known_architectures()}"
        ) from None


def config_from_dict(d: Mapping[str, Any]) -> ModelConfig:
    archs = d.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs:
        raise UnsupportedConfigError(
            f"config.json has no 'architectures' list; known: {known_architectures()}"
        )
    for name in archs:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name].from_dict(d)
    raise UnsupportedConfigError(
        f"unknown architecture {list(archs)!r}; known: {known_architectures()}"
    )


def load_config(model_dir: str | Path) -> ModelConfig:
    return config_from_dict(read_config_json(model_dir))
