"""Attention over the paged cache: the choice of kernel."""
from __future__ import annotations

from . import ops


def attention(qkv, cache_view, ctx, H, Hkv, hd, scale, window):
    """Rows of qkv hold q in their left H*hd columns.  Returns [T, H*hd]."""
    return ops.attention_plain(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.tok_pos,
                               ctx.tok_seq, ctx.slots, H, Hkv, hd, cache_view.page_size, scale, window)
