"""Sampling parameters, with the reference's names and meanings.

SamplerConfig of the reference (internal/engine/types_base.go:7-15): Temperature,
TopK, TopP, RepPenalty, Seed.  Temperature 0 is greedy; top_k <= 0 and top_p outside
(0, 1) switch those filters off; a repetition penalty <= 1 does nothing; seed 0 asks
for a seed from the clock (internal/engine/sampler.go:18-21)."""
from __future__ import annotations

import time
from dataclasses import dataclass

HISTORY_WINDOW = 64  # the penalty looks at the last 64 tokens (internal/engine/sampler.go:256-259)


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, found {self.temperature}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be > 0, found {self.repetition_penalty}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0

    @property
    def uses_history(self) -> bool:
        return self.repetition_penalty > 1.0

    def resolved_seed(self) -> int:
        return self.seed if self.seed != 0 else time.time_ns() & 0x7FFF_FFFF_FFFF_FFFF
