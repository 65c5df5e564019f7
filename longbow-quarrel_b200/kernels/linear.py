"""y = x . W^T (+ residual): the one matrix product of the decoder, and the choice
of kernel for it.

float32 inputs always take the FFMA kernel (true 32-bit, fixed summation order).
bfloat16 inputs take the tensor-core kernels once a weight has been prepared for
them; `LinearWeight` keeps what those kernels need beside the tensor.
"""
from __future__ import annotations

import torch

from . import ops


class LinearWeight:
    """A weight [N, K] as stored, plus per-kernel preparations made on first use."""

    def __init__(self, tensor: torch.Tensor):
        if tensor.dim() != 2:
            raise ops.KernelError(f"a linear weight must be 2-D, found shape {tuple(tensor.shape)}")
        self.tensor = tensor.contiguous()
        self.N, self.K = self.tensor.shape
        self.prepared: dict = {}


def linear(a: torch.Tensor, weight: LinearWeight, out_dtype: torch.dtype,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] . W^T -> [M, N] in out_dtype; with `residual` (float32 [M, N]) the sum
    residual + a . W^T is written into residual and returned."""
    if a.dtype == torch.bfloat16 and weight.tensor.dtype == torch.bfloat16:
        from . import tensorcore
        out = tensorcore.linear_bf16(a, weight, out_dtype, residual)
        if out is not None:
            return out
    return ops.gemm_plain(a, weight.tensor, out_dtype, residual)
