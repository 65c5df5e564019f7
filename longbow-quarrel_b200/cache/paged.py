"""Storage of keys and values for one group of cache entries with the same needs.

The reference keeps, per layer, two tensors [window, kv_heads * head_dim] for its
one sequence (internal/engine/kv_cache_sliding_window.go:77-92) and, in its paged
variant, blocks of 16 tokens behind a block table (internal/engine/kv_cache_paged.go:15-42).
Here every sequence of a batch has its own length, so storage is a pool of pages of
`page_size` tokens, [entry][page][kv_head][token][head_dim], and each slot has a row
of page numbers.  A group whose layers attend to a window only gives pages back as
they fall out of the window, so it holds a window's worth of pages per sequence.
"""
from __future__ import annotations

import numpy as np
import torch

from .group import CacheGroup
from .slots import CacheError

NO_PAGE = -1


class PagedKVGroup(CacheGroup):
    def __init__(self, entries: list[int], n_kv_heads: int, head_dim: int, window: int | None, n_pages: int,
                 page_size: int, max_slots: int, max_pages_per_seq: int, dtype: torch.dtype, device):
        self.entries = list(entries)
        self.index = {e: i for i, e in enumerate(self.entries)}
        self.n_kv_heads, self.head_dim, self.window = n_kv_heads, head_dim, window
        self.page_size, self.n_pages, self.max_pages_per_seq = page_size, n_pages, max_pages_per_seq
        shape = (len(self.entries), n_pages, n_kv_heads, page_size, head_dim)
        # Kernels that load whole pages multiply the rows beyond a sequence's length by probability zero,
        # which needs finite values there: the pool starts zero-filled, and a page that is handed out
        # again has the rows that its new owner's step does not write cleared first (`_to_clear`).
        self.k_pages = torch.zeros(shape, dtype=dtype, device=device)
        self.v_pages = torch.zeros(shape, dtype=dtype, device=device)
        self.table = np.full((max_slots, max_pages_per_seq), NO_PAGE, dtype=np.int32)
        self.table_dev = torch.full((max_slots, max_pages_per_seq), NO_PAGE, dtype=torch.int32, device=device)
        self._free = list(range(n_pages - 1, -1, -1))
        self._dirty: set[int] = set()
        self._to_clear: list[tuple[int, int]] = []      # (page, first row that the step does not write)

    def _snapshot(self) -> torch.Tensor:
        """The next of four pinned copies of the table (its last upload, four uploads ago, has long been read)."""
        if not hasattr(self, "_staged"):
            self._staged, self._turn = [], 0
        if len(self._staged) < 4:
            self._staged.append((torch.empty(self.table.shape, dtype=torch.int32).pin_memory(), torch.cuda.Event()))
            self._turn = len(self._staged) - 1
        else:
            self._turn = (self._turn + 1) % 4
            self._staged[self._turn][1].synchronize()
        return self._staged[self._turn][0]

    @property
    def n_free_pages(self) -> int:
        return len(self._free)

    def pages_of(self, slot: int) -> list[int]:
        row = self.table[slot]
        return [int(p) for p in row if p != NO_PAGE]

    def first_needed(self, length: int) -> int:
        """The lowest position a later token of a sequence of `length` tokens can attend to."""
        if self.window is None:
            return 0
        return max(0, length - self.window + 1)

    def reserve(self, slot: int, old_len: int, new_len: int) -> None:
        """Make sure positions [old_len, new_len) have pages."""
        if new_len <= old_len:
            return
        first, last = old_len // self.page_size, (new_len - 1) // self.page_size
        if last >= self.max_pages_per_seq:
            raise CacheError(f"a sequence of {new_len} tokens exceeds the context the cache was sized for "
                             f"({self.max_pages_per_seq * self.page_size} tokens)")
        need = [p for p in range(first, last + 1) if self.table[slot, p] == NO_PAGE]
        if len(need) > len(self._free):
            raise CacheError(f"the cache is full: {len(need)} more pages of {self.page_size} tokens are needed, "
                             f"{len(self._free)} of {self.n_pages} are free")
        for p in need:
            page = self._free.pop()
            self.table[slot, p] = page
            written_to = min(new_len - p * self.page_size, self.page_size)
            if written_to < self.page_size:
                self._to_clear.append((page, written_to))
        if need:
            self._dirty.add(slot)

    def trim(self, slot: int, length: int) -> None:
        """Give back the pages that lie wholly below the window of a sequence of `length` tokens."""
        if self.window is None:
            return
        keep_from = self.first_needed(length) // self.page_size
        row = self.table[slot]
        for p in range(keep_from):
            if row[p] != NO_PAGE:
                self._free.append(int(row[p]))
                row[p] = NO_PAGE
                self._dirty.add(slot)

    def commit(self, slot: int, length: int) -> None:
        self.trim(slot, length)

    def reserve_one_each(self, slots, old_lens) -> None:
        # One more token needs a page only where it starts one.
        starts = (old_lens % self.page_size) == 0
        if starts.any():
            for slot, old in zip(slots[starts].tolist(), old_lens[starts].tolist()):
                self.reserve(slot, old, old + 1)

    def commit_one_each(self, slots, new_lens) -> None:
        if self.window is None:
            return
        # A page falls out of the window only when the window's lower end reaches the next page.
        ends = (np.maximum(new_lens - self.window + 1, 0) % self.page_size) == 0
        for slot, length in zip(slots[ends].tolist(), new_lens[ends].tolist()):
            self.trim(slot, length)

    def release(self, slot: int) -> None:
        row = self.table[slot]
        for p in np.nonzero(row != NO_PAGE)[0]:
            self._free.append(int(row[p]))
        row[:] = NO_PAGE
        self._dirty.add(slot)

    def upload(self) -> None:
        """Copy the rows of the page table that changed to the device, and clear the unwritten ends of
        pages that were handed out since the last step."""
        if self._dirty:
            lo, hi = min(self._dirty), max(self._dirty) + 1
            if self.table_dev.is_cuda:
                # Through a snapshot in pinned memory, so that the copy neither makes the host wait nor reads rows
                # that the host changes afterwards (a step queued ahead may still be waiting for it when a finished
                # sequence's row is wiped).  Rows between the changed ones are the same on both sides already.
                stage = self._snapshot()
                stage[lo:hi].copy_(torch.from_numpy(self.table[lo:hi]))
                self.table_dev[lo:hi].copy_(stage[lo:hi], non_blocking=True)
                self._staged[self._turn][1].record()
            else:
                self.table_dev[lo:hi].copy_(torch.from_numpy(self.table[lo:hi]))
            self._dirty.clear()
        if self._to_clear:
            todo, self._to_clear = self._to_clear, []
            if self.k_pages.is_cuda:
                from ..kernels import ops
                ops.clear_page_tails(self.k_pages, self.v_pages, todo)
            else:                                   # bookkeeping tests keep their pools on the CPU
                for page, first in todo:
                    self.k_pages[:, page, :, first:].zero_()
                    self.v_pages[:, page, :, first:].zero_()

    def view(self, entry: int) -> "KVView":
        return KVView(self, entry)

    def nbytes(self) -> int:
        return 2 * self.k_pages.numel() * self.k_pages.element_size()

    def pages_in_use(self) -> int:
        return self.n_pages - len(self._free)


class KVView:
    """What a mixer gets of its cache entry: the entry's pages and the group's page table."""

    def __init__(self, group: PagedKVGroup, entry: int):
        i = group.index[entry]
        self.k_pages = group.k_pages[i]
        self.v_pages = group.v_pages[i]
        self.page_table = group.table_dev
        self.page_size = group.page_size
        self.window = group.window
        self.n_kv_heads, self.head_dim = group.n_kv_heads, group.head_dim
