"""Random-weights mode: make a model folder (``config.json`` + ``model.safetensors``) from a
configuration and a seed, or the same tensors directly on a device.

Law: matrices and tables N(0, std), norm weights 1 + N(0, std), std 0.02 unless the part
says otherwise. Each tensor draws from its own generator seeded by (seed, tensor name), so
a tensor's values do not depend on which other tensors exist or in which order they are
made. Upstream has no such mode; its tests build ``randn(shape) * 0.5`` dictionaries from
the expected shapes (tests/test_model.py:14-17).
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Iterable

import torch
from safetensors.torch import save_file

from ..config.base import ModelConfig
from ..parts.base import TensorSpec
from .loader import merge_specs


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def _draw(name: str, shape: tuple[int, ...], init: str, std: float, seed: int,
          device: torch.device | str) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(_seed_for(seed, name))
    t = torch.randn(shape, generator=g, dtype=torch.float32, device=device) * std
    if init == "one_plus_normal":
        t += 1.0
    elif init != "normal":
        raise ValueError(f"unknown init law {init!r} for {name}")
    return t


def random_checkpoint_tensors(specs: Iterable[TensorSpec], seed: int, dtype: torch.dtype,
                              device: torch.device | str = "cpu") -> dict[str, torch.Tensor]:
    """Tensors under the names a checkpoint stores (sources of merged tensors, not merged)."""
    out: dict[str, torch.Tensor] = {}
    for spec in merge_specs(specs).values():
        if spec.merged_from:
            for name, rows in zip(spec.merged_from, spec.merged_rows):
                out[name] = _draw(name, (rows, *spec.shape[1:]), spec.init, spec.std, seed, device).to(dtype)
        else:
            out[spec.name] = _draw(spec.name, spec.shape, spec.init, spec.std, seed, device).to(dtype)
    return out


def random_bound_tensors(specs: Iterable[TensorSpec], seed: int, dtype: torch.dtype,
                         device: torch.device | str) -> dict[str, torch.Tensor]:
    """The same values as ``random_checkpoint_tensors`` laid out as the parts bind them
    (merged), made tensor by tensor on ``device`` so that no host copy of a large model is
    ever held. Values differ between CPU and CUDA generators; use a folder for parity."""
    out: dict[str, torch.Tensor] = {}
    for spec in merge_specs(specs).values():
        if spec.merged_from:
            t = torch.empty(spec.shape, dtype=dtype, device=device)
            row = 0
            for name, rows in zip(spec.merged_from, spec.merged_rows):
                t[row: row + rows] = _draw(name, (rows, *spec.shape[1:]), spec.init, spec.std, seed, device).to(dtype)
                row += rows
            out[spec.name] = t
        else:
            out[spec.name] = _draw(spec.name, spec.shape, spec.init, spec.std, seed, device).to(dtype)
    return out


def write_random_model(model_dir: str | Path, config: ModelConfig, seed: int,
                       dtype: torch.dtype = torch.bfloat16, std_scale: float = 1.0) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with random weights.

    ``std_scale`` multiplies every standard deviation (tests use a larger spread so that
    greedy output is not one repeated token)."""
    from ..model import build_parts  # late: model imports the parts registries

    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    specs = build_parts(config.to_spec()).tensor_specs()
    if std_scale != 1.0:
        specs = [TensorSpec(**{**s.__dict__, "std": s.std * std_scale}) for s in specs]
    tensors = random_checkpoint_tensors(specs, seed, dtype)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(model_dir / "model.safetensors"))
    d = config.to_dict()
    d["torch_dtype"] = str(dtype).replace("torch.", "")
    (model_dir / "config.json").write_text(json.dumps(d, indent=2) + "\n", encoding="utf-8")
    return model_dir
