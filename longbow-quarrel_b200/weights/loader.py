"""Weights from safetensors by tensor name.

The reference walks the GGUF tensor table, maps names to slots and converts dtypes
as it goes (internal/engine/engine.go:736-1104), and notices a missing tensor only
when inference starts (engine.go:1316-1324).  Here the model says which names and
shapes it needs, and one error lists everything that is wrong with the file.

Kept as stored where possible: bfloat16 stays bfloat16, a tensor stored in 32-bit
stays in 32-bit, float16 becomes bfloat16, integer tables become int32.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile
from .spec import WeightSpec


class WeightsError(ValueError):
    """The checkpoint does not hold what the model needs; lists every fault."""

    def __init__(self, where, missing, unexpected, wrong_shape, other=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.other = list(other)
        lines = [f"{where}: the checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " +
                         "; ".join(f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in self.wrong_shape))
        for msg in self.other:
            lines.append("  " + msg)
        super().__init__("\n".join(lines))


def _open_files(folder: Path) -> list[SafetensorsFile]:
    single = folder / "model.safetensors"
    index = folder / "model.safetensors.index.json"
    if single.is_file():
        return [SafetensorsFile(single)]
    if index.is_file():
        shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        return [SafetensorsFile(folder / s) for s in shards]
    raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")


def _keep_dtype(t: torch.Tensor, spec: WeightSpec) -> torch.Tensor:
    if spec.integer:
        return t.to(torch.int32)
    if t.dtype in (torch.float32, torch.bfloat16):
        return t
    if t.dtype in (torch.float16,):
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    raise SafetensorsError(f"dtype {t.dtype} is not a weight dtype")


def load_weights(folder, table: dict[str, WeightSpec], device) -> dict[str, torch.Tensor]:
    """Every tensor of `table` on `device`.  A name with a `fallback` that is absent
    from the file is left out of the result (the part then reads the fallback)."""
    folder = Path(folder)
    files = _open_files(folder)
    where: dict[str, SafetensorsFile] = {}
    other = []
    for f in files:
        for name in f.names():
            if name in where:
                other.append(f"tensor {name} appears in both {where[name].path.name} and {f.path.name}")
            where[name] = f
    missing, wrong = [], []
    for name, spec in table.items():
        if name not in where:
            if spec.fallback is not None and spec.fallback in table:
                continue
            missing.append(name)
        elif where[name].shape(name) != tuple(spec.shape):
            wrong.append((name, tuple(spec.shape), where[name].shape(name)))
        elif spec.integer == where[name].dtype(name).is_floating_point:
            other.append(f"tensor {name} has dtype {where[name].dtype(name)}, expected "
                         f"{'an integer' if spec.integer else 'a floating-point'} type")
    unexpected = [n for n in where if n not in table]
    if missing or wrong or unexpected or other:
        raise WeightsError(folder, missing, unexpected, wrong, other)
    out = {}
    for name, spec in table.items():
        if name in where:
            out[name] = _keep_dtype(where[name].tensor(name), spec).to(device, non_blocking=False).contiguous()
    for f in files:
        f.close()
    return out
