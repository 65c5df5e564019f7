"""Token embedding and output head.

Embedding: row `token` of the table, no multiplier, promoted to the 32-bit residual
stream (internal/device/kernels.metal:465-467; internal/engine/engine.go:1365-1375).
Head: logits = n . W^T in 32-bit (internal/engine/engine.go:1561;
internal/device/kernels.metal:1172-1194), reading the embedding table when the
model ties them (internal/engine/engine.go:1108-1111).
"""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from ..weights.spec import WeightSpec
from .base import Part, Runtime
from .registry import register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, name: str):
        self.runtime, self.vocab_size, self.hidden_size, self.name = runtime, vocab_size, hidden_size, name
        self.table: torch.Tensor | None = None

    def weights(self):
        return {self.name: WeightSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.table = tensors[self.name]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return ops.embedding(self.table, tokens)


@register_part("head", "linear_head")
class LinearHead(Part):
    """`tied_to` names the tensor (of another part) that the head reads when it has
    none of its own; with `tied` true it never has its own."""

    graph_safe = True

    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int, name: str, tied_to: str | None = None,
                 tied: bool = False):
        self.runtime, self.vocab_size, self.hidden_size = runtime, vocab_size, hidden_size
        self.name, self.tied_to, self.tied = name, tied_to, tied
        self.weight: linear.LinearWeight | None = None

    def weights(self):
        if self.tied:
            return {}
        return {self.name: WeightSpec((self.vocab_size, self.hidden_size), fallback=self.tied_to)}

    def borrows(self):
        return [self.tied_to] if self.tied_to is not None else []

    def load(self, tensors):
        w = tensors.get(self.name)
        if w is None:
            w = tensors[self.tied_to]
        self.weight = linear.LinearWeight(w)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return linear.linear(h, self.weight, torch.float32)
