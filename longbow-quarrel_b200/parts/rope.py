"""Rotary position encoding with half-split pairs (element i with i + head_dim/2),
angle = position * f_i, f_i = theta^(-2i/head_dim)
(internal/device/kernels.metal:430-463 rope_f16; internal/device/cpu_ref.go:100-131).

The reference has no frequency scaling.  `scaling` of type "llama3" rescales f_i by
wavelength: kept above the high-frequency bound, divided by `factor` below the
low-frequency bound, blended in between.  Frequencies and angles are worked out in
float64 on the host and tabulated as float32 cos/sin, so every kernel and every
way of cutting the work reads the same angles.
"""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, Runtime
from .registry import register_part


def rope_frequencies(head_dim: int, theta: float, scaling=None) -> torch.Tensor:
    """f_i for i < head_dim / 2, float64."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * i / head_dim)
    if scaling is None:
        return f
    n0 = float(scaling.original_max_position_embeddings)
    lo, hi, factor = float(scaling.low_freq_factor), float(scaling.high_freq_factor), float(scaling.factor)
    wavelen = 2.0 * math.pi / f
    smooth = (n0 / wavelen - lo) / (hi - lo)
    blended = (1.0 - smooth) * f / factor + smooth * f
    out = torch.where(wavelen > n0 / lo, f / factor, blended)
    return torch.where(wavelen < n0 / hi, f, out)


@register_part("position", "rope")
class Rope(PositionEncoding):
    graph_safe = True

    def __init__(self, runtime: Runtime, head_dim: int, theta: float, scaling=None):
        self.runtime, self.head_dim, self.theta, self.scaling = runtime, head_dim, float(theta), scaling
        self._tables = None

    def tables(self):
        if self._tables is None:
            key = ("rope", self.head_dim, self.theta, self.scaling, self.runtime.max_context)
            if key not in self.runtime.shared:
                f = rope_frequencies(self.head_dim, self.theta, self.scaling)
                pos = torch.arange(self.runtime.max_context, dtype=torch.float64)
                ang = pos[:, None] * f[None, :]
                self.runtime.shared[key] = (torch.cos(ang).to(torch.float32).to(self.runtime.device).contiguous(),
                                            torch.sin(ang).to(torch.float32).to(self.runtime.device).contiguous())
            self._tables = self.runtime.shared[key]
        return self._tables
