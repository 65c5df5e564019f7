"""Tensor-core paths of the bfloat16 matrix products."""
from __future__ import annotations

import torch

from . import ops


def linear_bf16(a, weight, out_dtype, residual):
    """a [M, K] bf16 . W^T; returns None when no tensor-core kernel takes this product."""
    M, K = a.shape
    if K % 8:
        return None
    if M <= ops.SKINNY_MAX_ROWS:
        if residual is not None:
            return ops.gemm_skinny(a, weight.tensor, ops.EPI_RESID, residual)
        if out_dtype == torch.float32:
            return ops.gemm_skinny(a, weight.tensor, ops.EPI_F32)
        return ops.gemm_skinny(a, weight.tensor, ops.EPI_BF16)
    if residual is not None:
        return ops.gemm_tc(a, weight.tensor, ops.EPI_RESID, residual)
    return ops.gemm_tc(a, weight.tensor, ops.EPI_F32 if out_dtype == torch.float32 else ops.EPI_BF16)


def linear_swiglu_bf16(a, weight):
    """a . W^T over rows interleaved in blocks of 8 (gate, up), then up * silu(gate)."""
    M, K = a.shape
    if K % 8:
        return None
    if M <= ops.SKINNY_MAX_ROWS:
        return ops.gemm_skinny(a, weight.tensor, ops.EPI_SWIGLU)
    return ops.gemm_tc(a, weight.tensor, ops.EPI_SWIGLU)
