"""Attention over the paged cache: the choice of kernel, and the work lists that the prompt kernels read."""
from __future__ import annotations

import numpy as np
import torch

from . import ops

USE_TC_PREFILL = True        # head_dim 64 and 128: prefill attention on tcgen05 instead of mma.sync
BALANCED_DECODE = True       # steps of single tokens: the keys of all sequences cut into equal shares (else equal slices per sequence)
MAX_SPLITS = 32
KEYS_PER_SPLIT = 128         # a slice shorter than this is not worth a block of its own

def resident_blocks(device, hd: int = 128) -> int:
    """Blocks of the decode kernel that run at a time: one (8 warps, ~200 KB of key/value rings) per SM,
    two where the rings are half as large (head_dim up to 64)."""
    return ops.sm_count(device) * (2 if hd <= 64 else 1)


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


# ------------------------------------------------------------------ work list of the decode kernel
MIN_PART_TILES = KEYS_PER_SPLIT // 16      # the same floor in the kernel's 16-key tiles
DECODE_TILE = 16


def decode_teams(B: int, Hkv: int, group_tiles: int, resident: int) -> int:
    """Room in the work list of a batch of B tokens: the teams of blocks (one block per kv head and row
    tile each) that run as one wave, and at least one team per token.  Not more: with parts for one and a
    half to three waves, steps of sequences of unequal lengths ran 0 to 12 % slower (3B and 8B layer sizes,
    batches of 8 to 32), because a block of a later wave starts its loads from nothing."""
    return min(max(B, resident // max(1, Hkv * group_tiles)), 65535)


def decode_work_size(B: int, teams: int) -> int:
    return teams + 1 + 5 * teams


def cut_decode_work(positions, window: int, teams: int, max_parts: int = MAX_SPLITS) -> np.ndarray:
    """The decode kernel's work list for tokens at these positions: every token's keys cut into parts of
    nearly the same length for all tokens, as short as `teams` parts in all allow, so that a long sequence
    gets more parts than a short one and the blocks finish together (with the same number of slices for
    every sequence, the blocks of the longest would still run when all others are done).  The longest
    parts come first.  int32 [teams + 1 + 5 * teams]: for each team the offset of its segments (here one
    each, or none), then (token, first tile, last tile + 1, part, parts of the token) per segment, in the
    kernel's 16-key tiles counted from the first one the token sees (its window's first tile).  No part
    is shorter than MIN_PART_TILES unless it is a whole token, and no token gets more than max_parts."""
    pos = np.asarray(positions, dtype=np.int64)
    B = len(pos)
    if teams < B:
        raise ValueError(f"{B} tokens need at least as many teams, not {teams}")
    first = np.where((window > 0) & (pos >= window), pos - window + 1, 0) // DECODE_TILE
    tiles = pos // DECODE_TILE + 1 - first
    most = np.minimum(max_parts, np.maximum(1, tiles // MIN_PART_TILES))       # parts a token may have
    n = np.ones(B, dtype=np.int64)
    if teams > B and most.max() > 1:
        # The best common length is some token's length over some count of parts: try them all at once.
        counts = np.arange(1, min(max_parts, teams - B + 1) + 1)
        lengths = np.unique(-(-tiles[:, None] // counts[None, :]))
        need = np.minimum(-(-tiles[None, :] // lengths[:, None]), most[None, :])
        fits = need.sum(axis=1) <= teams
        n = need[np.argmax(fits)]              # lengths ascend: the first that fits is the shortest
    tok = np.repeat(np.arange(B), n)
    part = np.arange(len(tok)) - np.repeat(np.cumsum(n) - n, n)
    lo, hi = part * tiles[tok] // n[tok], (part + 1) * tiles[tok] // n[tok]
    order = np.argsort(lo - hi, kind="stable")
    out = np.zeros(decode_work_size(B, teams), dtype=np.int32)
    out[:teams + 1] = np.minimum(np.arange(teams + 1), len(tok))
    seg = out[teams + 1:teams + 1 + 5 * len(tok)].reshape(-1, 5)
    seg[:, 0], seg[:, 1], seg[:, 2], seg[:, 3], seg[:, 4] = tok[order], lo[order], hi[order], part[order], n[tok][order]
    return out


def decode_work(H: int, Hkv: int, window: int | None, device, hd: int = 128):
    """Builder of the decode kernel's work list for attention of these head counts and this window: empty
    for a step with prompts."""
    group_tiles = -(-(H // Hkv) // 16)

    def build(step) -> np.ndarray:
        if step.max_new != 1:
            return np.zeros(0, dtype=np.int32)
        return cut_decode_work(np.asarray(step.past), int(window or 0),
                               decode_teams(step.B, Hkv, group_tiles, resident_blocks(device, hd)))
    return build


def decode_work_name(H: int, Hkv: int, window: int | None) -> str:
    return f"decode_work:{H}:{Hkv}:{int(window or 0)}"


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


def decode_kernel(dtype: torch.dtype, hd: int) -> bool:
    """Whether single tokens of this dtype and head size go to the split decode kernel."""
    return dtype == torch.bfloat16 and hd % 16 == 0 and hd <= 128


def step_needs(dtype: torch.dtype, hd: int, H: int | None = None, Hkv: int | None = None, window: int | None = None,
               device=None) -> dict:
    """The work lists that attention of this dtype and head size reads: the query blocks of steps with
    prompts, and (when the head counts are given) the balanced segments of steps of single tokens."""
    kind = prefill_kernel(dtype, hd)
    name = {"tc": "query_blocks128", "mma": "query_blocks64"}.get(kind)
    needs = {name: PREFILL_LISTS[name]} if name else {}
    if H is not None and Hkv and BALANCED_DECODE and decode_kernel(dtype, hd):
        needs[decode_work_name(H, Hkv, window)] = decode_work(H, Hkv, window, device, hd)
    return needs


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
    if ctx.decode and aligned and decode_kernel(qkv.dtype, hd) and cache_view.page_size % 16 == 0:
        work = ctx.extra.get(decode_work_name(H, Hkv, window))
        if work is not None and work.numel():
            teams = decode_teams(ctx.T, Hkv, -(-(H // Hkv) // 16), resident_blocks(qkv.device, hd))
            if work.numel() == decode_work_size(ctx.T, teams):
                return ops.attn_decode(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.tok_pos,
                                       ctx.tok_seq, ctx.slots, H, Hkv, hd, cache_view.page_size, scale, window,
                                       min(MAX_SPLITS, teams), next_w=next_w, early_loads=True, work=work, teams=teams)
        n_splits = decode_splits(ctx.T, Hkv, -(-(H // Hkv) // 16), ctx.max_kv, resident_blocks(qkv.device, hd))
        return ops.attn_decode(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.tok_pos,
                               ctx.tok_seq, ctx.slots, H, Hkv, hd, cache_view.page_size, scale, window, n_splits,
                               next_w=next_w, early_loads=True)      # a decode step: one new token per sequence
    return ops.attention_plain(qkv, cache_view.k_pages, cache_view.v_pages, cache_view.page_table, ctx.tok_pos,
                               ctx.tok_seq, ctx.slots, H, Hkv, hd, cache_view.page_size, scale, window)
