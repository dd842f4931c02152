"""Reading a model folder's safetensors by tensor name.

Every ``*.safetensors`` file of the folder is read (sharded checkpoints need no index
file). The set of tensors is checked against what the model's parts declare
(``TensorSpec``): all problems — missing names, unexpected names, wrong shapes — are
collected into ONE ``WeightLoadError``. A merged tensor (``qkv_proj`` from q/k/v,
``gate_up_proj`` from gate/up) may be stored merged or as its sources. Floating-point
tensors are cast to the run's dtype (bfloat16 for serving), except those a part marks
``keep_32bit`` when the file stores them in 32-bit; integer tables become int32.

Behaviour after upstream src/tinyserve/weights.py:51-129 (strict name/shape check with one
message, a tied checkpoint's extra ``lm_head.weight`` skipped, non-finite values refused,
q/k/v and gate/up stacked by rows).
"""

from __future__ import annotations

from pathlib import Path
from typing import Iterable, Mapping

import torch
from safetensors import safe_open

from ..parts.base import TensorSpec


class WeightLoadError(RuntimeError):
    """The folder's tensors do not match what the configuration says the model holds."""


def merge_specs(specs: Iterable[TensorSpec]) -> dict[str, TensorSpec]:
    """Specs by name; two parts may declare the same tensor (tied head) if they agree."""
    out: dict[str, TensorSpec] = {}
    for s in specs:
        old = out.get(s.name)
        if old is not None and (old.shape != s.shape or old.merged_from != s.merged_from):
            raise WeightLoadError(f"{s.name} is declared twice with different shapes: {old.shape} and {s.shape}")
        out.setdefault(s.name, s)
    return out


def checkpoint_names(specs: Mapping[str, TensorSpec]) -> dict[str, tuple[int, ...]]:
    """Names and shapes as a checkpoint conventionally stores them (sources, not merged)."""
    out: dict[str, tuple[int, ...]] = {}
    for s in specs.values():
        if s.merged_from:
            for name, rows in zip(s.merged_from, s.merged_rows):
                out[name] = (rows, *s.shape[1:])
        else:
            out[s.name] = s.shape
    return out


def _cast(t: torch.Tensor, spec: TensorSpec, dtype: torch.dtype) -> torch.dtype:
    if spec.integer or not t.dtype.is_floating_point:
        return torch.int32
    if spec.keep_32bit and t.dtype == torch.float32:
        return torch.float32
    return dtype


def load_tensors(model_dir: str | Path, specs: Iterable[TensorSpec], dtype: torch.dtype,
                 device: torch.device | str, ignorable: Iterable[str] = ()) -> dict[str, torch.Tensor]:
    model_dir = Path(model_dir)
    files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise WeightLoadError(f"no *.safetensors files in {model_dir}")
    wanted = merge_specs(specs)
    ignorable = set(ignorable)

    # name -> (file, shape) of everything the folder holds
    present: dict[str, tuple[Path, tuple[int, ...]]] = {}
    for file in files:
        with safe_open(str(file), framework="pt", device="cpu") as f:
            for name in f.keys():
                present[name] = (file, tuple(f.get_slice(name).get_shape()))

    missing: list[str] = []
    wrong: list[str] = []
    consumed: set[str] = set()
    plan: dict[str, tuple[str, ...]] = {}   # spec name -> file tensor names to stack
    for spec in wanted.values():
        if spec.name in present:
            consumed.add(spec.name)
            shape = present[spec.name][1]
            if shape != spec.shape:
                wrong.append(f"{spec.name}: shape {shape}, expected {spec.shape}")
            plan[spec.name] = (spec.name,)
            continue
        if spec.merged_from:
            ok = True
            for src, rows in zip(spec.merged_from, spec.merged_rows):
                if src not in present:
                    missing.append(src)
                    ok = False
                    continue
                consumed.add(src)
                expect = (rows, *spec.shape[1:])
                if present[src][1] != expect:
                    wrong.append(f"{src}: shape {present[src][1]}, expected {expect}")
                    ok = False
            if ok:
                plan[spec.name] = spec.merged_from
            continue
        missing.append(spec.name)
    unexpected = sorted(set(present) - consumed - ignorable)

    problems: list[str] = []
    if missing:
        problems.append(f"{len(missing)} missing: {sorted(missing)}")
    if unexpected:
        problems.append(f"{len(unexpected)} unexpected: {unexpected}")
    if wrong:
        problems.append(f"{len(wrong)} with a wrong shape: " + "; ".join(sorted(wrong)))
    if problems:
        raise WeightLoadError(f"{model_dir} does not match its config.json:\n  " + "\n  ".join(problems))

    handles = {file: safe_open(str(file), framework="pt", device="cpu") for file in files}
    out: dict[str, torch.Tensor] = {}
    try:
        for name, sources in plan.items():
            spec = wanted[name]
            parts = [handles[present[s][0]].get_tensor(s) for s in sources]
            target = _cast(parts[0], spec, dtype)
            if len(parts) == 1:
                t = parts[0].to(device=device, dtype=target)
            else:
                t = torch.empty(spec.shape, dtype=target, device=device)
                row = 0
                for part in parts:
                    t[row: row + part.shape[0]] = part.to(device=device, dtype=target)
                    row += part.shape[0]
            if t.dtype.is_floating_point and not bool(torch.isfinite(t).all()):
                raise WeightLoadError(f"{name} has inf or nan after casting to {target}")
            out[name] = t.contiguous()
    finally:
        handles.clear()
    return out
