"""The description of a model as data: which parts make each layer, with which
sizes and constants, and in which order the layers run.

An architecture's `describe(config)` returns a ModelSpec; the engine builds the
parts it names from the part registry.  Nothing here knows an architecture.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """A part by the name it is registered under, with its parameters."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One block: how its parts are arranged, and the parts.

    prefix  what the tensor names of this layer's parts start with.
    """
    prefix: str
    mixer: PartSpec
    ffn: PartSpec
    norm1: PartSpec
    norm2: PartSpec
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `cache` names the cache entry the layer's mixer works on
    (entries are numbered by the model's describe function); with `writes_cache`
    false the mixer only reads that entry, which another layer has written."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    name: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    stop_tokens: tuple[int, ...] = ()
    bos_token: int | None = None
