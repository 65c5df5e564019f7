"""How a part names the tensors it needs."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part reads from the checkpoint.

    shape     the exact shape it must have.
    init      how the random-weights mode fills it: "normal" (N(0, std)) or "gain"
              (1 + N(0, gain_std)).
    fallback  full name of another tensor that stands in when this one is absent
              (a tied output head reads the embedding table).
    integer   the tensor is an integer table (kept as int32).
    full_precision  the part computes with this tensor in 32-bit whatever the model's precision (norm
              gains): a loader that converts tensors to the model's precision leaves it as stored.
    """
    shape: tuple[int, ...]
    init: str = "normal"
    fallback: str | None = None
    integer: bool = False
    full_precision: bool = False
