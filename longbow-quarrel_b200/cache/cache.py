"""The cache of a model: a slot for each live sequence; keys and values for each
cache entry (a layer's run), grouped by need, each group with storage of its own;
fixed-size state per sequence; and each sequence's own length.

Sized by `max_tokens`: the most tokens that live sequences hold at any time, each
sequence's count rounded up to whole pages.
"""
from __future__ import annotations

import numpy as np
import torch

from ..parts.base import CacheNeed
from .group import CacheGroup, CacheSizing
from .paged import PagedKVGroup
from .slots import CacheError, SlotAllocator
from .state import StateGroup

PAGE_SIZE = 64


class Cache:
    def __init__(self, needs: dict[int, CacheNeed | None], max_tokens: int, max_context: int,
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
        sizing = CacheSizing(self.n_pages, page_size, self.max_slots, pages_per_seq, max_context, dtype, device)

        # Entries with equal needs share a group; each need makes the group that suits it.
        by_need: dict[CacheNeed, list[int]] = {}
        for entry, need in sorted(needs.items()):
            if need is None:
                continue
            if not isinstance(need, CacheNeed):
                raise CacheError(f"cache entry {entry}: {need!r} is no CacheNeed")
            by_need.setdefault(need, []).append(entry)
        self.groups: list[CacheGroup] = [need.make_group(entries, sizing) for need, entries in by_need.items()]
        self._views: dict[int, object] = {}
        for g in self.groups:
            for e in g.entries:
                self._views[e] = g.view(e)

    @property
    def kv_groups(self) -> list[PagedKVGroup]:
        return [g for g in self.groups if isinstance(g, PagedKVGroup)]

    @property
    def state_groups(self) -> list[StateGroup]:
        return [g for g in self.groups if isinstance(g, StateGroup)]

    # ------------------------------------------------------------------ slots
    def alloc_slot(self) -> int:
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        for g in self.groups:
            g.start(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)
        for g in self.groups:
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
        for g in self.groups:
            g.reserve(slot, old, old + n_new)

    def commit(self, slot: int, n_new: int) -> None:
        """The step stored n_new tokens; pages that fell out of a window go back to their pool."""
        self.lengths[slot] += n_new
        for g in self.groups:
            g.commit(slot, int(self.lengths[slot]))

    def reserve_one_each(self, slots: list[int]) -> np.ndarray:
        """Room for one more token of every sequence in `slots`; returns their lengths so far.  The same as
        reserve(slot, 1) for each, with the bookkeeping of all sequences done at once."""
        live = self.slots.is_live
        for slot in slots:
            if not live(slot):
                raise CacheError(f"slot {slot} is not live")
        idx = np.asarray(slots, dtype=np.int64)
        old = self.lengths[idx]
        if len(idx) and int(old.max()) + 1 > self.max_context:
            raise CacheError(f"sequence would reach {int(old.max()) + 1} tokens; the context limit is {self.max_context}")
        for g in self.groups:
            g.reserve_one_each(idx, old)
        return old

    def commit_one_each(self, slots: list[int]) -> None:
        idx = np.asarray(slots, dtype=np.int64)
        self.lengths[idx] += 1
        new = self.lengths[idx]
        for g in self.groups:
            g.commit_one_each(idx, new)

    def upload(self) -> None:
        for g in self.groups:
            g.upload()

    def view(self, entry: int):
        """What the mixer of a cache entry works on (None for an entry without cache)."""
        return self._views.get(entry)

    # ------------------------------------------------------------------ accounting (tests, stats)
    def pages_in_use(self) -> int:
        return sum(g.pages_in_use() for g in self.groups)

    def bytes(self) -> int:
        return sum(g.nbytes() for g in self.groups)
