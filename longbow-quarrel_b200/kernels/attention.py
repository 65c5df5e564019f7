"""Attention over the paged cache: the choice of kernel, and the work lists that the prompt kernels read."""
from __future__ import annotations

import numpy as np
import torch

from . import ops

USE_TC_PREFILL = True        # head_dim 64 and 128: prefill attention on tcgen05 instead of mma.sync
MAX_SPLITS = 32
KEYS_PER_SPLIT = 128         # a slice shorter than this is not worth a block of its own

def resident_blocks(device) -> int:
    """Blocks of the decode kernel that run at a time: one (8 warps, ~200 KB of key/value rings) per SM."""
    return ops.sm_count(device)


def decode_splits(n_tokens: int, Hkv: int, group_tiles: int, max_kv: int, resident: int) -> int:
    """How many slices to cut each sequence's keys into: as many as still run in one wave."""
    blocks = max(1, n_tokens * Hkv * group_tiles)
    return max(1, min(resident // blocks, MAX_SPLITS, -(-max_kv // KEYS_PER_SPLIT)))


# ------------------------------------------------------------------ work lists of the prompt kernels
def query_blocks(size: int):
    """Builder of the work list of a prompt kernel whose blocks take `size` query rows: blocks of at most
    `size` consecutive rows of one sequence, as int32 [4, n] = (sequence, first row, rows, first position),
    the blocks with the most keys first.  A step of one token per sequence needs none."""
    def build(step) -> np.ndarray:
        if step.max_new == 1:
            return np.zeros(0, dtype=np.int32)
        qb = [(b, step.cu[b] + r, min(size, n - r), p + r)
              for b, (p, n) in enumerate(zip(step.past, step.new)) for r in range(0, n, size)]
        qb.sort(key=lambda e: -e[3])
        return np.asarray(qb, dtype=np.int32).reshape(-1, 4).T.copy()
    return build


PREFILL_LISTS = {"query_blocks64": query_blocks(64), "query_blocks128": query_blocks(128)}


def prefill_kernel(dtype: torch.dtype, hd: int, page_size: int = 64) -> str | None:
    """Which prompt kernel takes queries of this dtype and head size: "tc" (tcgen05), "mma" (mma.sync),
    or None (the plain kernel)."""
    if dtype != torch.bfloat16 or page_size != 64:
        return None
    if USE_TC_PREFILL and hd in (64, 128):
        return "tc"
    if hd % 16 == 0 and hd <= 128:
        return "mma"
    return None


def step_needs(dtype: torch.dtype, hd: int) -> dict:
    """The work lists that attention of this dtype and head size reads in steps with prompts."""
    kind = prefill_kernel(dtype, hd)
    name = {"tc": "query_blocks128", "mma": "query_blocks64"}.get(kind)
    return {name: PREFILL_LISTS[name]} if name else {}


def _blocks(ctx, name):
    flat = ctx.extra.get(name)
    if flat is None or flat.numel() == 0:
        return None
    return tuple(flat.view(4, -1))


def attention(qkv, cache_view, ctx, H, Hkv, hd, scale, window, next_w=None):
    """Rows of qkv hold q in their left H*hd columns.  Returns [T, H*hd].  next_w: the weights the
    stream reads after the attention (the decode kernel asks for their first bytes as it ends)."""
    aligned = qkv.stride(0) % 8 == 0
    if not ctx.decode and aligned:
        kind = prefill_kernel(qkv.dtype, hd, cache_view.page_size)
        if kind == "tc":
            blocks = _blocks(ctx, "query_blocks128")
            if blocks is not None:
                return ops.attn_prefill_tc(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.slots,
                                           ctx.kv_len, blocks, H, Hkv, hd, cache_view.page_size, scale, window)
            kind = "mma" if "query_blocks64" in ctx.extra else None
        if kind == "mma":
            blocks = _blocks(ctx, "query_blocks64")
            if blocks is not None:
                return ops.attn_prefill(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.slots,
                                        ctx.kv_len, blocks, H, Hkv, hd, cache_view.page_size, scale, window)
    if ctx.decode and aligned and qkv.dtype == torch.bfloat16 and hd <= 128 and hd % 16 == 0 \
            and cache_view.page_size % 16 == 0:
        n_splits = decode_splits(ctx.T, Hkv, -(-(H // Hkv) // 16), ctx.max_kv, resident_blocks(qkv.device))
        return ops.attn_decode(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.tok_pos,
                               ctx.tok_seq, ctx.slots, H, Hkv, hd, cache_view.page_size, scale, window, n_splits,
                               next_w=next_w, early_loads=True)      # a decode step: one new token per sequence
    return ops.attention_plain(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.tok_pos,
                               ctx.tok_seq, ctx.slots, H, Hkv, hd, cache_view.page_size, scale, window)
