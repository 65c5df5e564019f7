"""RMS norm: y = x / sqrt(mean(x^2) + eps) * gain, computed in 32-bit
(internal/device/kernels.metal:905-942 rmsnorm_f32_to_f16_v4; the gains are
promoted to 32-bit at load, internal/engine/engine.go:788-792)."""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import Norm, Runtime
from .registry import register_part


@register_part("norm", "rms_norm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, runtime: Runtime, size: int, eps: float, name: str = "weight"):
        self.runtime, self.size, self.eps, self.name = runtime, size, float(eps), name
        self.gain: torch.Tensor | None = None

    def weights(self):
        return {self.name: WeightSpec((self.size,), init="gain", full_precision=True)}

    def load(self, tensors):
        self.gain = tensors[self.name].to(torch.float32).contiguous()

    def forward(self, x, rows=None):
        return ops.rmsnorm(x, self.gain, self.eps, self.runtime.act_dtype, rows)

    def foldable(self, n_rows):
        if self.gain is None or not linear.can_defer_norm(n_rows, self.size, self.runtime.act_dtype):
            return None
        return self.gain, self.eps
