"""Slots: one for each live sequence.  A slot is a row in every per-sequence table
of the cache (page tables, lengths, fixed-size state); it is handed out when a
sequence starts and given back when it ends, and is then used again."""
from __future__ import annotations


class CacheError(RuntimeError):
    pass


class SlotAllocator:
    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise CacheError("a cache needs at least one slot")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))  # pop() hands out the lowest first
        self._live: set[int] = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"no free slot: all {self.n_slots} slots hold live sequences")
        slot = self._free.pop()
        self._live.add(slot)
        return slot

    def free(self, slot: int) -> None:
        if slot not in self._live:
            raise CacheError(f"slot {slot} is not live (freed twice, or never handed out)")
        self._live.remove(slot)
        self._free.append(slot)

    def is_live(self, slot: int) -> bool:
        return slot in self._live

    @property
    def n_live(self) -> int:
        return len(self._live)

    @property
    def n_free(self) -> int:
        return len(self._free)
