"""The cache of a model: a slot for each live sequence; keys and values for each
cache entry (a layer's run), grouped by need, each group with storage of its own;
fixed-size state per sequence; and each sequence's own length.

Sized by `max_tokens`: the most tokens that live sequences hold at any time, each
sequence's count rounded up to whole pages.
"""
from __future__ import annotations

import numpy as np
import torch

from ..parts.base import KVNeed, StateNeed
from .paged import KVView, PagedKVGroup
from .slots import CacheError, SlotAllocator
from .state import StateGroup

PAGE_SIZE = 64


class Cache:
    def __init__(self, needs: dict[int, KVNeed | StateNeed | None], max_tokens: int, max_context: int,
                 dtype: torch.dtype, device, max_slots: int | None = None, page_size: int = PAGE_SIZE):
        if max_tokens < 1:
            raise CacheError("max_tokens must be positive")
        self.page_size = page_size
        self.n_pages = -(-max_tokens // page_size)
        self.max_context = max_context
        self.max_slots = max_slots or min(self.n_pages, 1024)
        pages_per_seq = -(-min(max_context, self.n_pages * page_size) // page_size)
        self.slots = SlotAllocator(self.max_slots)
        self.lengths = np.zeros(self.max_slots, dtype=np.int64)
        self.device, self.dtype = device, dtype

        kv: dict[KVNeed, list[int]] = {}
        st: dict[StateNeed, list[int]] = {}
        for entry, need in sorted(needs.items()):
            if isinstance(need, KVNeed):
                kv.setdefault(need, []).append(entry)
            elif isinstance(need, StateNeed):
                st.setdefault(need, []).append(entry)
            elif need is not None:
                raise CacheError(f"cache entry {entry}: unknown need {need!r}")
        self.kv_groups = [PagedKVGroup(entries, need.n_kv_heads, need.head_dim, need.window, self.n_pages, page_size,
                                       self.max_slots, pages_per_seq, dtype, device)
                          for need, entries in kv.items()]
        self.state_groups = [StateGroup(entries, need.shape, need.dtype, self.max_slots, device)
                             for need, entries in st.items()]
        self._views: dict[int, object] = {}
        for g in self.kv_groups:
            for e in g.entries:
                self._views[e] = KVView(g, e)
        for g in self.state_groups:
            for e in g.entries:
                self._views[e] = g.view(e)

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        for g in self.state_groups:
            g.reset(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)
        for g in self.kv_groups:
            g.release(slot)
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        return int(self.lengths[slot])

    # ------------------------------------------------------------------ a step's bookkeeping
    def reserve(self, slot: int, n_new: int) -> None:
        """Room for n_new more tokens of the sequence in `slot`, in every group."""
        if not self.slots.is_live(slot):
            raise CacheError(f"slot {slot} is not live")
        old = int(self.lengths[slot])
        if old + n_new > self.max_context:
            raise CacheError(f"sequence would reach {old + n_new} tokens; the context limit is {self.max_context}")
        for g in self.kv_groups:
            g.reserve(slot, old, old + n_new)

    def commit(self, slot: int, n_new: int) -> None:
        """The step stored n_new tokens; pages that fell out of a window go back to their pool."""
        self.lengths[slot] += n_new
        for g in self.kv_groups:
            g.trim(slot, int(self.lengths[slot]))

    def upload(self) -> None:
        for g in self.kv_groups:
            g.upload()

    def view(self, entry: int):
        """KVView or state tensor of a cache entry (None for an entry without cache)."""
        return self._views.get(entry)

    # ------------------------------------------------------------------ accounting (tests, stats)
    def pages_in_use(self) -> int:
        return sum(g.n_pages - g.n_free_pages for g in self.kv_groups)

    def bytes(self) -> int:
        n = sum(g.k_pages.numel() * g.k_pages.element_size() * 2 for g in self.kv_groups)
        return n + sum(g.data.numel() * g.data.element_size() for g in self.state_groups)
