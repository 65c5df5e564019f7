"""Attention over the paged cache: the choice of kernel."""
from __future__ import annotations

import torch

from . import ops

USE_TC_PREFILL = True        # head_dim 64 and 128: prefill attention on tcgen05 instead of mma.sync
RESIDENT_BLOCKS = 148        # one block of the decode kernel (8 warps, ~200 KB of key/value rings) per SM
MAX_SPLITS = 32
KEYS_PER_SPLIT = 128         # a slice shorter than this is not worth a block of its own


def decode_splits(n_tokens: int, Hkv: int, group_tiles: int, max_kv: int) -> int:
    """How many slices to cut each sequence's keys into: as many as still run in one wave."""
    blocks = max(1, n_tokens * Hkv * group_tiles)
    return max(1, min(RESIDENT_BLOCKS // blocks, MAX_SPLITS, -(-max_kv // KEYS_PER_SPLIT)))


def attention(qkv, cache_view, ctx, H, Hkv, hd, scale, window, next_w=None):
    """Rows of qkv hold q in their left H*hd columns.  Returns [T, H*hd].  next_w: the weights the
    stream reads after the attention (the decode kernel asks for their first bytes as it ends)."""
    fast = qkv.dtype == torch.bfloat16 and hd <= 128 and hd % 8 == 0 and qkv.stride(0) % 8 == 0
    if (fast and not ctx.decode and hd in (64, 128) and cache_view.page_size == 64 and USE_TC_PREFILL
            and getattr(ctx, "query_blocks128", None) is not None):
        return ops.attn_prefill_tc(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.slots,
                                   ctx.kv_len, ctx.query_blocks128, H, Hkv, hd, cache_view.page_size, scale, window)
    if fast and not ctx.decode and cache_view.page_size == 64 and ctx.query_blocks is not None:
        return ops.attn_prefill(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.slots,
                                ctx.kv_len, ctx.query_blocks, H, Hkv, hd, cache_view.page_size, scale, window)
    if fast and ctx.decode:
        n_splits = decode_splits(ctx.T, Hkv, -(-(H // Hkv) // 16), ctx.max_kv)
        return ops.attn_decode(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.tok_pos,
                               ctx.tok_seq, ctx.slots, H, Hkv, hd, cache_view.page_size, scale, window, n_splits,
                               next_w=next_w, early_loads=True)      # a decode step: one new token per sequence
    return ops.attention_plain(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.tok_pos,
                               ctx.tok_seq, ctx.slots, H, Hkv, hd, cache_view.page_size, scale, window)
