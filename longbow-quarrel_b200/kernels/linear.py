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


GATE_UP_BLOCK = 8


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows of gate and up [F, K] alternating in blocks of 8: the layout whose product
    the fused SwiGLU epilogues read (a tile of 16 output columns holds 8 gate values and
    the 8 up values that go with them)."""
    F, K = gate.shape
    b = GATE_UP_BLOCK
    return torch.stack([gate.reshape(F // b, b, K), up.reshape(F // b, b, K)], dim=1).reshape(2 * F, K).contiguous()


def linear_swiglu(a: torch.Tensor, weight: LinearWeight, block: int) -> torch.Tensor:
    """act(a . Wg^T) * (a . Wu^T) for the stacked weight [2F, K]; block 0 = gate rows
    then up rows, block 8 = interleaved."""
    if block == GATE_UP_BLOCK and a.dtype == torch.bfloat16 and weight.tensor.dtype == torch.bfloat16:
        from . import tensorcore
        out = tensorcore.linear_swiglu_bf16(a, weight)
        if out is not None:
            return out
    gu = linear(a, weight, a.dtype)
    return ops.swiglu(gu, block)
