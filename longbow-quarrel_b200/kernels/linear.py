"""y = x . W^T (+ residual): the one matrix product of the decoder, and the choice
of kernel for it.

float32 inputs always take the FFMA kernel (true 32-bit, fixed summation order).
bfloat16 inputs take the tensor-core kernels once a weight has been prepared for
them; `LinearWeight` keeps what those kernels need beside the tensor.
"""
from __future__ import annotations

import os

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
        # The weight that the same stream reads after this one in a step (see `recording`): the
        # kernels for few rows ask for its first bytes while they run out.
        self.next: LinearWeight | None = None

    @property
    def next_tensor(self):
        return self.next.tensor if self.next is not None else None


_log: list | None = None


class recording:
    """While active, the products note their weights in the order of use; at the end every weight
    learns which one follows it (the last one is followed by the first: the next step)."""

    def __enter__(self):
        global _log
        _log = []
        return self

    def __exit__(self, *exc):
        global _log
        log, _log = _log, None
        if exc[0] is None and len(log) > 1:
            for w, after in zip(log, log[1:] + log[:1]):
                if after is not w:
                    w.next = after
        return False


def note(weight: "LinearWeight") -> None:
    if _log is not None:
        _log.append(weight)


FOLD_NORMS = os.environ.get("LQ_FOLD_NORMS", "1") != "0"      # 0: every norm runs as a kernel of its own


FOLD_MAX_ROWS = int(os.environ.get("LQ_FOLD_MAX_ROWS", "8"))       # measured on B200: 3 % of a decode step at 1 row, 1.4 % at 8, a loss at 16


def can_defer_norm(rows: int, width: int, dtype: torch.dtype) -> bool:
    """Whether a product of `rows` rows should leave the next RMS norm's rows unfinished (and the
    product after it finishes them): the kernel for few rows of bfloat16 does both."""
    return FOLD_NORMS and dtype == torch.bfloat16 and rows <= FOLD_MAX_ROWS and width % 8 == 0


def _plain_rows(a):
    return a.finish() if isinstance(a, ops.NormedRows) else a


def linear(a, weight: LinearWeight, out_dtype: torch.dtype, residual: torch.Tensor | None = None,
           emit: tuple | None = None):
    """a [M, K] . W^T -> [M, N] in out_dtype; with `residual` (float32 [M, N]) the sum
    residual + a . W^T is written into residual and returned.
    `a` may be ops.NormedRows.  With emit = (gain, eps) of the RMS norm that reads the residual
    next, returns (residual, rows) where rows are that norm's ops.NormedRows, or None when the
    kernel for this shape does not make them."""
    note(weight)
    if a.dtype == torch.bfloat16 and weight.tensor.dtype == torch.bfloat16:
        from . import tensorcore
        out = tensorcore.linear_bf16(a, weight, out_dtype, residual, emit)
        if out is not None:
            return out
    out = ops.gemm_plain(_plain_rows(a), weight.tensor, out_dtype, residual)
    return (out, None) if emit is not None else out


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
            note(weight)
            return out
    gu = linear(a, weight, a.dtype)
    return ops.swiglu(gu, block)
