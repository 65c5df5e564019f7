"""Gated feed-forward: y = (up(x) * act(gate(x))) . Wd^T, act = SiLU without clamp
(internal/device/metal.go:1464-1474; internal/device/cpu_ref.go:133-149 CPUSwiGLU).
Gate and up are one matrix product over the stacked weight [2F, D]."""
from __future__ import annotations

import torch

from ..kernels import linear
from ..weights.spec import WeightSpec
from .base import FeedForward, Runtime, StepContext
from .registry import register_part

DEFAULT_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


@register_part("ffn", "gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True
    folds_norm = True

    def __init__(self, runtime: Runtime, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: dict | None = None):
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} is not supported (supported: 'silu')")
        self.runtime, self.D, self.F = runtime, hidden_size, intermediate_size
        self.names = {**DEFAULT_NAMES, **(names or {})}
        self.w_gu: linear.LinearWeight | None = None
        self.block = 0
        self.w_down: linear.LinearWeight | None = None

    def weights(self):
        n = self.names
        return {n["gate"]: WeightSpec((self.F, self.D)), n["up"]: WeightSpec((self.F, self.D)),
                n["down"]: WeightSpec((self.D, self.F))}

    def load(self, tensors):
        n = self.names
        gate, up = tensors[n["gate"]], tensors[n["up"]]
        if gate.dtype != up.dtype:
            gate, up = gate.to(torch.float32), up.to(torch.float32)
        # bfloat16 kernels apply SwiGLU in the product's epilogue over interleaved rows.
        self.block = linear.GATE_UP_BLOCK if (self.runtime.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16
                                              and self.F % linear.GATE_UP_BLOCK == 0) else 0
        stacked = linear.interleave_gate_up(gate, up) if self.block else torch.cat([gate, up], dim=0)
        self.w_gu = linear.LinearWeight(stacked)
        self.w_down = linear.LinearWeight(tensors[n["down"]])

    def forward(self, h, ctx: StepContext, residual, emit=None):
        act = linear.linear_swiglu(h, self.w_gu, self.block)
        if emit is None:
            linear.linear(act, self.w_down, self.runtime.act_dtype, residual=residual)
            return None
        return linear.linear(act, self.w_down, self.runtime.act_dtype, residual=residual, emit=emit)[1]
