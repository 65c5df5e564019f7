"""The description of a model as data: which parts make each layer, with which
sizes and constants, and in which order the layers run.

An architecture's `describe(config)` returns a ModelSpec; the engine builds the
parts it names from the part registry.  Nothing here knows an architecture.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """A part by the name it is registered under, with its parameters."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One block: how its parts are arranged, and the parts by the names that the arrangement gives
    their places.

    prefix       what the tensor names of this layer's parts start with.
    parts        place -> part.  Which places there are is the arrangement's business: "pre_norm" has
                 `norm1`, `mixer`, `norm2`, `ffn`; an arrangement with a third norm or with two branches
                 side by side names more places and needs no change here.
    arrangement  the block class (registered under the role "block") that reads `parts`.
    """
    prefix: str
    parts: Mapping[str, PartSpec]
    arrangement: str = "pre_norm"

    def part(self, place: str) -> PartSpec:
        try:
            return self.parts[place]
        except KeyError:
            raise ValueError(f"layer {self.prefix!r}: the arrangement {self.arrangement!r} needs a part in the "
                             f"place {place!r} (given: {', '.join(sorted(self.parts)) or 'none'})") from None


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
