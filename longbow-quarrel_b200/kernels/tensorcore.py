"""Tensor-core paths of the bfloat16 matrix products: which kernel takes which shape.

rows <= 16   gemm_skinny: W streamed through registers into mma.sync (fastest measured stream
             of W: the loads of all warps keep more bytes in flight than one TMA unit does)
rows <= 64   gemm_stream: W streamed by TMA in equal shares over all SMs into tcgen05 -- or
             gemm_skinny where the weight is small enough that gemm_stream's fixed cost (filling
             its ring, adding parked pieces: about 15 us) outweighs its better rate per row
more rows    gemm_tc: 128 x 256 tiles, TMA ring, tcgen05 with two accumulators in tensor memory
"""
from __future__ import annotations

import torch

from . import ops


# Measured on B200 (us, gemm_skinny / gemm_stream), weights of 34, 50, 117 and 235 MB:
#   32 rows: 12 / 23, 21 / 22, 33 / 40, 71 / 59        64 rows: 24 / 36, 63 / 31, 74 / 53, 193 / 73
# Inside a decode step of 8 layers: 32 rows 2.15 ms with gemm_skinny for the three smaller weights against
# 2.26 ms without; 64 rows 3.43 ms with it for the smallest against 3.38 ms without.
SKINNY_BYTES_32 = 128 << 20     # up to 32 rows gemm_skinny takes weights up to this size


def _decode_kernel(M: int, N: int, K: int):
    if M <= ops.SKINNY_BEST_ROWS:
        return ops.gemm_skinny
    return ops.gemm_skinny if M <= 32 and 2 * N * K <= SKINNY_BYTES_32 else ops.gemm_stream


def _rows_for(fn, a):
    """Unfinished rows of a norm go to the kernel that finishes them; every other kernel gets plain rows."""
    return a if fn is ops.gemm_skinny or not isinstance(a, ops.NormedRows) else a.finish()


def linear_bf16(a, weight, out_dtype, residual, emit=None):
    """a [M, K] bf16 . W^T; returns None when no tensor-core kernel takes this product."""
    M, K = a.shape
    if K % 8:
        return None
    fn = _decode_kernel(M, weight.N, K) if M <= ops.SKINNY_MAX_ROWS else ops.gemm_tc
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
    fn = _decode_kernel(M, weight.N, K) if M <= ops.SKINNY_MAX_ROWS else ops.gemm_tc
    more = {"next_w": weight.next_tensor} if fn is ops.gemm_skinny else {}
    return fn(_rows_for(fn, a), weight.tensor, ops.EPI_SWIGLU, **more)
