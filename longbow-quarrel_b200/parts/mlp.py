"""Gated feed-forward: y = (up(x) * act(gate(x))) . Wd^T, act = SiLU without clamp
(internal/device/metal.go:1464-1474; internal/device/cpu_ref.go:133-149 CPUSwiGLU).
Gate and up are one matrix product over the stacked weight [2F, D]."""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import FeedForward, Runtime, StepContext
from .registry import register_part

DEFAULT_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


@register_part("ffn", "gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: dict | None = None):
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} is not supported (supported: 'silu')")
        self.runtime, self.D, self.F = runtime, hidden_size, intermediate_size
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.w_gu: linear.LinearWeight | None = None
        self.w_down: linear.LinearWeight | None = None

    def weights(self):
        n = self.names
        return {n["gate"]: WeightSpec((self.F, self.D)), n["up"]: WeightSpec((self.F, self.D)),
                n["down"]: WeightSpec((self.D, self.F))}

    def load(self, tensors):
        n = self.names
        self.w_gu = linear.LinearWeight(torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0))
        self.w_down = linear.LinearWeight(tensors[n["down"]])

    def forward(self, h, ctx: StepContext, residual):
        gu = linear.linear(h, self.w_gu, self.runtime.act_dtype)
        act = ops.swiglu(gu)
        linear.linear(act, self.w_down, self.runtime.act_dtype, residual=residual)
