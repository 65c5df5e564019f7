"""Tensor-core paths of the bfloat16 matrix products: which kernel takes which shape.

rows <= 16   gemm_skinny: W streamed through registers into mma.sync (the fastest stream of W
             measured: 6.9-7.0 TB/s on the LM head at 1 to 8 rows); see ops.streams_through_registers
more rows    gemm_tc: 128 x 256 tiles, TMA ring, tcgen05 with two accumulators in tensor memory;
             with few tiles (few rows, narrow weight) it cuts the contraction into ranges so that
             every SM streams a share of W

Measured on B200 at 64 rows, weights of 34 / 50 / 117 / 235 MB (us): gemm_tc 15 / 19 / 30 / 53,
gemm_skinny 24 / 63 / 74 / 193; at 17 rows gemm_tc 13 / 15 / 26 / 52, gemm_skinny 11 / 19 / 31 / 64.
"""
from __future__ import annotations

import torch

from . import ops


def _decode_kernel(M: int, N: int, K: int):
    return ops.gemm_skinny if ops.streams_through_registers(M, N) else ops.gemm_tc


def _rows_for(fn, a):
    """Unfinished rows of a norm go to the kernel that finishes them; every other kernel gets plain rows."""
    return a if fn is ops.gemm_skinny or not isinstance(a, ops.NormedRows) else a.finish()


def linear_bf16(a, weight, out_dtype, residual, emit=None):
    """a [M, K] bf16 . W^T; returns None when no tensor-core kernel takes this product."""
    M, K = a.shape
    if K % 8:
        return None
    fn = _decode_kernel(M, weight.N, K)
    a = _rows_for(fn, a)
    more = {"next_w": weight.next_tensor} if fn is ops.gemm_skinny else {}
    if residual is not None:
        if emit is not None:
            if fn is ops.gemm_skinny:
                return fn(a, weight.tensor, ops.EPI_RESID, residual, emit=emit, **more)
            return fn(a, weight.tensor, ops.EPI_RESID, residual), None
        return fn(a, weight.tensor, ops.EPI_RESID, residual, **more)
    return fn(a, weight.tensor, ops.EPI_F32 if out_dtype == torch.float32 else ops.EPI_BF16, **more)


def linear_swiglu_bf16(a, weight):
    """a . W^T over rows interleaved in blocks of 8 (gate, up), then up * silu(gate)."""
    M, K = a.shape
    if K % 8:
        return None
    fn = _decode_kernel(M, weight.N, K)
    more = {"next_w": weight.next_tensor} if fn is ops.gemm_skinny else {}
    return fn(_rows_for(fn, a), weight.tensor, ops.EPI_SWIGLU, **more)
