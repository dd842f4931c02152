"""Typed model configuration and the data that describes how a model is put together.

Three kinds of object live here:

* ``ModelConfig``: the base of every architecture's typed view of its own ``config.json``.
  A subclass reads the keys its architecture defines (``from_dict``) and turns them into a
  ``ModelSpec`` (``to_spec``). No size or constant that ``config.json`` gives is repeated
  in code.
* ``PartSpec`` / ``LayerSpec`` / ``LayerCall`` / ``ModelSpec``: plain data. A layer is a
  block and the parts that fill the block's roles (for the pre-norm block: a mixer, a
  feed-forward and their two norms); each part is named by the key it was registered under
  (``tinyserve_b200.parts.base``) and carries its own sizes and constants as arguments. Layers may differ from one another. The order in which layers
  run is a list of ``LayerCall`` too: it may name a layer twice, and a call may read the
  cache that an earlier call wrote instead of writing its own.

Reference: the upstream engine has one frozen dataclass of eleven fields and a hard check
on the architecture name (src/tinyserve/config.py:18-79); the split into typed config and
spec data is this framework's own.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping


class UnsupportedConfigError(ValueError):
    """The ``config.json`` asks for something this framework does not implement."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered ``kind`` and the arguments it is built with."""

    kind: str
    args: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """What one layer is made of. ``prefix`` is where its tensors live in the checkpoint;
    ``block`` the registered block; ``parts`` maps each role that block names to the part that
    fills it (``PreNormBlock``: "mixer", "feed_forward", "mixer_norm", "feed_forward_norm")."""

    prefix: str
    block: str
    parts: Mapping[str, PartSpec]
    position: PartSpec | None = None  # position encoding the mixers apply; None = none


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers``. ``reads_cache_of`` is ``None`` when the call
    owns a cache entry of its own (it writes this step's keys/values or state there), or
    the index of an EARLIER call in the order whose cache entry it reads without writing.
    """

    layer: int
    reads_cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the generic decoder needs to build a model, derived from a config."""

    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple[LayerSpec, ...]
    order: tuple[LayerCall, ...]
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    max_position_embeddings: int

    def __post_init__(self) -> None:
        for n, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise UnsupportedConfigError(f"order[{n}] names layer {call.layer} of {len(self.layers)}")
            src = call.reads_cache_of
            if src is not None:
                if not 0 <= src < n:
                    raise UnsupportedConfigError(
                        f"order[{n}] reads the cache of call {src}, which is not an earlier call"
                    )
                if self.order[src].reads_cache_of is not None:
                    raise UnsupportedConfigError(
                        f"order[{n}] reads the cache of call {src}, which owns no cache itself"
                    )


class ModelConfig:
    """Base class of the typed configurations. Subclasses are frozen dataclasses."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that ``from_dict`` would read back to this object."""
        raise NotImplementedError

    def to_spec(self) -> ModelSpec:
        raise NotImplementedError


def read_config_json(model_dir: str | Path) -> dict[str, Any]:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with path.open(encoding="utf-8") as f:
        d = json.load(f)
    if not isinstance(d, dict):
        raise UnsupportedConfigError(f"{path} does not hold a JSON object")
    return d
