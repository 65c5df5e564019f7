"""Random weights from a configuration and a seed.

The reference has no such mode: its tests write small GGUF files with constant
data by hand (internal/engine/engine_test.go:17-157).  Each tensor is drawn from
its own generator, seeded by the model seed and the tensor's name, so a tensor's
values do not depend on which other tensors exist or in which order they are made.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .safetensors_io import write_safetensors
from .spec import WeightSpec


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, spec: WeightSpec, seed: int, dtype: torch.dtype, device="cpu",
                  std: float = 0.02, gain_std: float = 0.1) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(tensor_seed(seed, name))
    if spec.integer:
        return torch.randint(0, 1 << 16, spec.shape, generator=gen, device=device, dtype=torch.int32)
    if spec.init == "gain":
        t = torch.ones(spec.shape, dtype=torch.float32, device=device)
        if gain_std:
            t += gain_std * torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32)
        return t.to(dtype)
    # Large tensors are drawn in the target dtype to keep the peak memory at one copy.
    draw = torch.float32 if spec.shape and _numel(spec.shape) < (1 << 26) else dtype
    t = torch.randn(spec.shape, generator=gen, device=device, dtype=draw)
    return (t * std).to(dtype)


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def random_weights(table: dict[str, WeightSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device="cpu", std: float = 0.02, gain_std: float = 0.1) -> dict[str, torch.Tensor]:
    """Every tensor of `table` (a tied head has no entry in its model's table)."""
    return {name: random_tensor(name, spec, seed, dtype, device, std, gain_std) for name, spec in table.items()}


def write_random_model(folder, config_dict: dict, table: dict[str, WeightSpec], seed: int,
                       dtype: torch.dtype = torch.bfloat16, std: float = 0.02, gain_std: float = 0.1) -> Path:
    """A model folder (config.json, model.safetensors) with random weights."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config_dict, indent=2))
    tensors = random_weights(table, seed, dtype, "cpu", std, gain_std)
    write_safetensors(folder / "model.safetensors", tensors, {"format": "pt", "seed": seed})
    return folder
